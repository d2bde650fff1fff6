"""The serial part of a chunked linear recurrence on the `chunk_scan` kernel, with its backward.

`chunk_scan(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)` evaluates, chunk after chunk,

    X  = P S + W V
    O  = Qd S + Mqk V + Mqb X
    S' = lam * S + Kd^T V + Bd^T X

for per-chunk matrices that the caller formed for all chunks at once (fp32, [B, H, n, 64, ...];
`lam` [B, H, n, dk]). The state stays in tensor memory across the chunks of a (row, head). The
backward runs the same kernel over the chunks in reverse for the gradients that follow the
state (dX, dS), then batched matmuls for the gradient of every operand.

Reference: ``architecture/recurrent/chunkwise.py:40-441``, ``affine_scan.py:120-149``.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

PAD = 128   # the kernel's head dims


def supported(dk: int, dv: int, device) -> bool:
    return device.type == "cuda" and dk <= PAD and dv <= PAD


def _pad_last(x: torch.Tensor, to: int) -> torch.Tensor:
    return x if x.shape[-1] == to else F.pad(x, (0, to - x.shape[-1]))


def _rows(top: Optional[torch.Tensor], bottom: Optional[torch.Tensor], like: torch.Tensor, width: int) -> torch.Tensor:
    """[top; bottom] as one bf16 [B*H*n*128, width] operand (a missing block is zeros)."""
    b, h, n = like.shape[:3]
    out = torch.zeros(b, h, n, 128, width, dtype=torch.bfloat16, device=like.device)
    if top is not None:
        out[..., :64, :top.shape[-1]] = top
    if bottom is not None:
        out[..., 64:, :bottom.shape[-1]] = bottom
    return out


def _run(a1, aux1, aux3, a4, v, lam, s0, *, want_out: bool, reverse: bool):
    from . import kernels as K

    b, h, n = v.shape[:3]
    dev = v.device
    out = K._out(b, h, n, 64, PAD, dtype=torch.bfloat16, device=dev, op="chunk_scan out") if want_out else None
    x = K._out(b, h, n, 64, PAD, dtype=torch.bfloat16, device=dev, op="chunk_scan x")
    states = K._out(b, h, n, PAD, PAD, dtype=torch.bfloat16, device=dev, op="chunk_scan states")
    last = K._out(b, h, PAD, PAD, dtype=torch.float32, device=dev, op="chunk_scan last")
    K.ops().chunk_scan(a1, aux1, aux3 if want_out else None, a4, v, lam, s0, out, x, states, last,
                       K.status_word(dev), b * h, n, reverse)
    K._count()
    return out, x, states, last


class _ChunkScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0):
        dk, dv = Qd.shape[-1], V.shape[-1]
        a1 = _rows(P, Qd, V, PAD)
        aux1 = _rows(W, Mqk, V, 64)
        aux3 = (Mqb if Mqb is not None else torch.zeros_like(Mqk)).to(torch.bfloat16).contiguous()
        a4 = _rows(Kd, Bd, V, PAD)
        v = _pad_last(V, PAD).to(torch.bfloat16).contiguous()
        lam_p = F.pad(lam.float(), (0, PAD - dk), value=1.0).contiguous()
        s0 = None
        if S0 is not None:
            s0 = F.pad(S0.float(), (0, PAD - dv, 0, PAD - dk)).contiguous()
        out, x, states, last = _run(a1, aux1, aux3, a4, v, lam_p, s0, want_out=True, reverse=False)
        ctx.save_for_backward(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam_p, x, states)
        ctx.dims = (dk, dv, S0 is not None)
        return out[..., :dv].float(), last[..., :dk, :dv].clone()

    @staticmethod
    def backward(ctx, d_out, d_last):
        # the operand gradients are fp32 matmuls over bf16-rounded states: TF32 loses nothing more
        before = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = d_out.is_cuda or before
        try:
            return _ChunkScan._backward(ctx, d_out, d_last)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = before

    @staticmethod
    def _backward(ctx, d_out, d_last):
        P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam_p, x, states = ctx.saved_tensors
        dk, dv, has_s0 = ctx.dims
        rank1 = P is not None
        d_out = d_out.float()
        # dX = Bd dS' + Mqb^T dO ;  dS = lam dS' + [Qd; P]^T [dO; dX], over the chunks in reverse
        a1 = _rows(Bd, None, V, PAD)
        aux1 = _rows(Mqb.transpose(-1, -2) if rank1 else None, None, V, 64)
        a4 = _rows(Qd, P, V, PAD)
        go = _pad_last(d_out, PAD).to(torch.bfloat16).contiguous()
        s0 = None
        if d_last is not None:
            s0 = F.pad(d_last.float(), (0, PAD - dv, 0, PAD - dk)).contiguous()
        _, dx, dsp, ds0 = _run(a1, aux1, None, a4, go, lam_p, s0, want_out=False, reverse=True)
        dX = dx[..., :dv].float()
        dSp = dsp[..., :dk, :dv].float()          # gradient of the state after each chunk
        S = states[..., :dk, :dv].float()         # the state each chunk started from
        X = x[..., :dv].float()
        Vf = V.float()
        St, dSpt = S.transpose(-1, -2), dSp.transpose(-1, -2)
        dQd = d_out @ St
        dMqk = d_out @ Vf.transpose(-1, -2)
        dKd = Vf @ dSpt
        dV = Mqk.float().transpose(-1, -2) @ d_out + Kd.float() @ dSp
        dP = dW = dMqb = dBd = None
        if rank1:
            dP = dX @ St
            dW = dX @ Vf.transpose(-1, -2)
            dMqb = d_out @ X.transpose(-1, -2)
            dBd = X @ dSpt
            dV = dV + W.float().transpose(-1, -2) @ dX
        dlam = (S * dSp).sum(-1)
        dS0 = ds0[..., :dk, :dv].clone() if has_s0 else None
        return dP, dQd, dW, dMqk, dMqb, dKd, dBd, dV, dlam, dS0


def chunk_scan(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0=None):
    """(O [B, H, n, 64, dv] fp32, the last state [B, H, dk, dv] fp32). P, W, Mqb, Bd may all be
    None (a recurrence without the rank-one term)."""
    return _ChunkScan.apply(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)
