"""Plain PyTorch statements of every op: the CPU path and the oracle of every kernel.

Each function computes in fp32 (or the input dtype on CPU when it is fp32 already)
with no fusion and no cleverness, so that a CUDA kernel can be compared against it.
The math follows the reference's slow paths: whole-logits cross-entropy
(``architecture/logits.py:200``), ``xla`` attention (``parallel/context.py:130``),
dequantise-then-multiply for MXFP8 (``architecture/precision/blockscaled.py:307-372``),
dense MoE (``architecture/experts/moe.py:587``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

MX_BLOCK = 32
E4M3_MAX = 448.0


# ------------------------------------------------------------------ norms / rope
def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float,
            zero_centered: bool = False) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1.0 + w if zero_centered else w)
    return y.to(x.dtype)


def layernorm(x, weight, bias, eps: float, zero_centered: bool = False):
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1.0 + w if zero_centered else w)
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def rope_tables(positions: torch.Tensor, dim: int, base: float, inv_freq=None):
    """cos/sin of shape positions.shape + (dim/2,), fp32."""
    if inv_freq is None:
        inv_freq = base ** (-torch.arange(0, dim, 2, dtype=torch.float32,
                                          device=positions.device) / dim)
    ang = positions.float().unsqueeze(-1) * inv_freq
    return ang.cos(), ang.sin()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
         interleaved: bool = False) -> torch.Tensor:
    """Rotate x[..., T, H, D] (cos/sin: [..., T, R/2], R <= D rotated dims)."""
    r = cos.shape[-1] * 2
    xf = x.float()
    rot, rest = xf[..., :r], xf[..., r:]
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    if interleaved:
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    else:
        a, b = rot[..., : r // 2], rot[..., r // 2:]
        out = torch.cat((a * c - b * s, a * s + b * c), dim=-1)
    return torch.cat((out, rest), dim=-1).to(x.dtype)


def rmsnorm_rope(x, weight, cos, sin, eps: float):
    """Per-head RMSNorm over D then RoPE by halves: the QK-norm + RoPE fusion."""
    return rope(rmsnorm(x, weight, eps), cos, sin)


# ------------------------------------------------------------------ activations
def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    if name == "swish":
        return F.silu(x)
    if name == "gelu":
        return F.gelu(x)
    if name == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name == "relu":
        return F.relu(x)
    if name == "relu2":
        return F.relu(x).square()
    if name == "sigmoid":
        return torch.sigmoid(x)
    if name == "tanh":
        return torch.tanh(x)
    if name == "softplus":
        return F.softplus(x)
    if name == "situ":
        return 4.0 * torch.tanh(x / 4.0) * torch.sigmoid(x)
    raise ValueError(f"unknown activation {name!r}")


def glu(gate: torch.Tensor, up: torch.Tensor, name: str = "swish",
        limit: Optional[float] = None, up_offset: float = 0.0) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (activation(g, name) * (u + up_offset)).to(gate.dtype)


# ------------------------------------------------------------------ MXFP8
def e8m0_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """Biased E8M0 exponent byte of scale = 2^ceil(log2(amax/448)), clamped to ±127."""
    ratio = amax.float() * (1.0 / E4M3_MAX)
    mant, exp = torch.frexp(ratio)  # ratio = mant * 2^exp, mant in [0.5, 1)
    e = torch.where(mant > 0.5, exp, exp - 1).clamp(-127, 127)
    e = torch.where(ratio < 2.0 ** -126, torch.full_like(e, -127), e)  # zero / denormal
    return (e + 127).to(torch.uint8)


def quant_mxfp8(x: torch.Tensor):
    """Quantise along the last dim in blocks of 32: returns (e4m3 values as
    torch.float8_e4m3fn, uint8 E8M0 scales [..., K/32])."""
    k = x.shape[-1]
    assert k % MX_BLOCK == 0
    xb = x.float().unflatten(-1, (k // MX_BLOCK, MX_BLOCK))
    amax = xb.abs().amax(-1)
    e = e8m0_from_amax(amax)
    scale = torch.exp2(e.float() - 127.0).unsqueeze(-1)
    q = (xb / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.flatten(-2), e


def dequant_mxfp8(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    k = q.shape[-1]
    qb = q.float().unflatten(-1, (k // MX_BLOCK, MX_BLOCK))
    return (qb * torch.exp2(e.float() - 127.0).unsqueeze(-1)).flatten(-2)


def swizzle_scales(e: torch.Tensor) -> torch.Tensor:
    """Lay [R, K/32] scale bytes out in the tensor-core scale-factor tiling: one
    512-byte tile per (128 rows x 4 scale columns); inside a tile row i's 4 bytes sit
    at (i % 32) * 16 + (i // 32) * 4. R and K/32 are padded up (pad byte 127 = 1.0)."""
    r, c = e.shape
    rp, cp = -(-r // 128) * 128, -(-c // 4) * 4
    full = torch.full((rp, cp), 127, dtype=torch.uint8, device=e.device)
    full[:r, :c] = e
    t = full.view(rp // 128, 4, 32, cp // 4, 4)  # rb, i//32, i%32, cb, byte
    return t.permute(0, 3, 2, 1, 4).contiguous().view(-1)


def unswizzle_scales(s: torch.Tensor, r: int, c: int) -> torch.Tensor:
    rp, cp = -(-r // 128) * 128, -(-c // 4) * 4
    t = s.view(rp // 128, cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return t.reshape(rp, cp)[:r, :c].contiguous()


def gemm_mxfp8(aq, ae, bq, be) -> torch.Tensor:
    """C = dequant(A) @ dequant(B)^T with A [M,K], B [N,K] quantised along K."""
    return dequant_mxfp8(aq, ae) @ dequant_mxfp8(bq, be).t()


# ------------------------------------------------------------------ attention
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
              window: Optional[int] = None, sinks: Optional[torch.Tensor] = None,
              softcap: Optional[float] = None, scale: Optional[float] = None,
              segments: Optional[torch.Tensor] = None) -> tuple:
    """Softmax attention on [B, T, H, D] queries and [B, S, G, D] keys/values (GQA:
    H % G == 0). `sinks` ([H]) adds one extra logit per head to the softmax
    denominator only. `segments` ([B, T] ints, or a pair ([B, T], [B, S]) for queries and keys)
    confines attention to equal ids.
    Returns (out [B, T, H, Dv], lse [B, H, T])."""
    b, t, h, d = q.shape
    s, g = k.shape[1], k.shape[2]
    scale = d ** -0.5 if scale is None else scale
    qf = q.float().transpose(1, 2)  # b h t d
    kf = k.float().transpose(1, 2).repeat_interleave(h // g, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(h // g, dim=1)
    logits = (qf @ kf.transpose(-1, -2)) * scale
    if softcap is not None:
        logits = softcap * torch.tanh(logits / softcap)
    qi = torch.arange(t, device=q.device).unsqueeze(-1) + (s - t)
    ki = torch.arange(s, device=q.device).unsqueeze(0)
    keep = torch.ones(t, s, dtype=torch.bool, device=q.device)
    if causal:
        keep &= ki <= qi
    if window is not None:
        keep &= ki > qi - window
    keep = keep.expand(b, 1, t, s)
    if segments is not None:
        # one tensor for self-attention, or (the queries' ids, the keys' ids) when they differ
        seg_q, seg_k = segments if isinstance(segments, (tuple, list)) else (segments, segments)
        keep = keep & (seg_q[:, None, :, None] == seg_k[:, None, None, :])
    logits = logits.masked_fill(~keep, float("-inf"))
    if sinks is not None:
        sink = sinks.float().view(1, h, 1, 1).expand(b, h, t, 1)
        full = torch.cat((logits, sink), dim=-1)
        lse = torch.logsumexp(full, dim=-1)
    else:
        lse = torch.logsumexp(logits, dim=-1)
    p = torch.exp(logits - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    out = (p @ vf).transpose(1, 2)
    return out.to(q.dtype), lse


# ------------------------------------------------------------------ loss
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, mask: Optional[torch.Tensor],
                  z_weight: float = 0.0, softcap: Optional[float] = None):
    """Sum over kept positions of -log p(target) (+ z * logZ^2); returns (sum, count)."""
    lf = logits.float()
    if softcap is not None:
        lf = softcap * torch.tanh(lf / softcap)
    logz = torch.logsumexp(lf, dim=-1)
    picked = lf.gather(-1, targets.unsqueeze(-1).long()).squeeze(-1)
    per_tok = logz - picked
    if z_weight:
        per_tok = per_tok + z_weight * logz.square()
    if mask is None:
        return per_tok.sum(), torch.tensor(float(per_tok.numel()), device=logits.device)
    m = mask.float()
    return (per_tok * m).sum(), m.sum()


# ------------------------------------------------------------------ MoE
def router_scores(logits: torch.Tensor, kind: str) -> torch.Tensor:
    lf = logits.float()
    if kind == "softmax":
        return torch.softmax(lf, dim=-1)
    if kind == "sigmoid":
        return torch.sigmoid(lf)
    if kind == "sqrtsoftplus":
        return torch.sqrt(F.softplus(lf))
    raise ValueError(kind)


def router_topk(logits: torch.Tensor, top_k: int, kind: str = "softmax",
                normalize: bool = True, scaling: float = 1.0,
                bias: Optional[torch.Tensor] = None):
    """Scores, top-k (by score + optional selection bias), weights of the picks.
    Returns (weights [T,k] fp32, experts [T,k] int64, scores [T,E] fp32)."""
    scores = router_scores(logits, kind)
    select = scores if bias is None else scores + bias.float()
    _, idx = torch.topk(select, top_k, dim=-1)
    w = scores.gather(-1, idx)
    if normalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return w * scaling, idx, scores


def moe_dense(x, w_gate_up, w_down, weights, experts, act: str = "swish",
              limit=None, up_offset: float = 0.0):
    """Every token through its picks, one expert at a time. x [T,d]; w_gate_up
    [E, 2f, d] (gate rows then up rows); w_down [E, d, f]."""
    t, d = x.shape
    e, f2, _ = w_gate_up.shape
    f = f2 // 2
    out = torch.zeros(t, d, dtype=torch.float32, device=x.device)
    xf = x.float()
    for ex in range(e):
        tok, slot = (experts == ex).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ w_gate_up[ex].float().t()
        a = glu(h[:, :f], h[:, f:], act, limit, up_offset)
        y = a @ w_down[ex].float().t()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1).float())
    return out.to(x.dtype)


# ------------------------------------------------------------------ optimizer
def adamw_step(p, g, m, v, *, lr: float, b1: float, b2: float, eps: float, wd: float,
               step: int, grad_scale: float = 1.0) -> None:
    """In-place decoupled AdamW on fp32 master `p` with bias correction (optax's)."""
    gf = g.float() * grad_scale
    m.mul_(b1).add_(gf.to(m.dtype), alpha=1 - b1)
    v.mul_(b2).add_((gf * gf).to(v.dtype), alpha=1 - b2)
    mh = m.float() / (1 - b1 ** step)
    vh = v.float() / (1 - b2 ** step)
    upd = mh / (vh.sqrt() + eps) + wd * p.float()
    p.add_(upd.to(p.dtype), alpha=-lr)
