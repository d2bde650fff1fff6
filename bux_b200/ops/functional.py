"""Differentiable ops: the sm_100a kernels behind ``torch.autograd.Function`` on CUDA,
the plain PyTorch statements (`reference`) elsewhere.

The switch is `kernels_on(x)`: a CUDA bf16 tensor takes the native kernels unless
``BUX_KERNELS=off`` (the reference's global kernel switch, ``kernels.py:28-54``), in
which case the library path (torch matmul / SDPA) runs instead: that is the
baseline the kernels are measured against, never a silent fallback.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import reference as ref

_OFF = os.environ.get("BUX_KERNELS", "").lower() == "off"


def set_kernels(on: bool) -> None:
    global _OFF
    _OFF = not on


def kernels_on(x: torch.Tensor) -> bool:
    return x.is_cuda and not _OFF and x.dtype == torch.bfloat16


def _K():
    from . import kernels

    return kernels


# ------------------------------------------------------------------ norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        K = _K()
        xc = x.contiguous()
        y, rstd = K.rmsnorm_fwd(xc, None if w is None else w.float().contiguous(), eps)
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x, w, rstd = ctx.saved_tensors
        dx, dw = K.rmsnorm_bwd(x, None if w is None else w.float().contiguous(), dy.contiguous(), rstd)
        return dx, (None if w is None else dw.to(w.dtype)), None


def rmsnorm(x, weight, eps: float = 1e-6, zero_centered: bool = False):
    if kernels_on(x) and x.shape[-1] % 8 == 0:
        w = weight
        if zero_centered and w is not None:
            w = w + 1.0
        return _RMSNorm.apply(x, w, eps)
    return ref.rmsnorm(x, weight, eps, zero_centered)


class _NormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, eps):
        K = _K()
        xc = x if K.token_stride(x) is not None else x.contiguous()  # a slice of qkv is read in place
        wf = None if w is None else w.float().contiguous()
        y, rstd = K.norm_rope_fwd(xc, wf, cos, sin, eps)
        ctx.save_for_backward(xc, w, cos, sin, rstd)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x, w, cos, sin, rstd = ctx.saved_tensors
        wf = None if w is None else w.float().contiguous()
        dx, dw = K.norm_rope_bwd(x, wf, cos, sin, rstd, dy.contiguous(), ctx.eps)
        return dx, (None if w is None else dw.to(w.dtype)), None, None, None


def rmsnorm_rope(x, weight, cos, sin, eps: float = 1e-6):
    """Per-head RMSNorm (weight [D] or None for RoPE only) then RoPE by halves.
    x: [B, T, H, D]; cos/sin: [B, T, D/2] fp32."""
    d = x.shape[-1]
    if kernels_on(x) and d in (64, 128, 256) and cos.shape[-1] * 2 == d:
        c2 = cos.reshape(-1, d // 2).float().contiguous()
        s2 = sin.reshape(-1, d // 2).float().contiguous()
        return _NormRope.apply(x, weight, c2, s2, eps)
    y = x if weight is None else ref.rmsnorm(x, weight, eps)
    return ref.rope(y, cos, sin)


def rope(x, cos, sin, interleaved: bool = False):
    if not interleaved:
        return rmsnorm_rope(x, None, cos, sin)
    return ref.rope(x, cos, sin, interleaved=True)


# ------------------------------------------------------------------ GLU
class _GLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, row_scale, kind, limit, up_offset):
        K = _K()
        hc = h.contiguous()
        rs = None if row_scale is None else row_scale.float().contiguous()
        ctx.save_for_backward(hc, rs)
        ctx.cfg = (kind, limit, up_offset)
        return K.glu_fwd(hc, kind, rs, limit, up_offset)

    @staticmethod
    def backward(ctx, dout):
        K = _K()
        h, rs = ctx.saved_tensors
        kind, limit, up_offset = ctx.cfg
        dh, drs = K.glu_bwd(h, dout.contiguous(), kind, rs, limit, up_offset)
        return dh, drs, None, None, None


def glu(h, kind: str = "swish", row_scale=None, limit: Optional[float] = None,
        up_offset: float = 0.0):
    """act(gate) * (up + offset) on h = [..., 2f] (gate columns first), optionally
    times a per-row scale (a router weight)."""
    f = h.shape[-1] // 2
    K_ok = kernels_on(h) and f % 8 == 0 and kind in ("swish", "quick_gelu", "gelu_tanh", "relu2")
    if K_ok:
        return _GLU.apply(h, row_scale, kind, float(limit or 0.0), float(up_offset))
    out = ref.glu(h[..., :f], h[..., f:], kind, limit, up_offset)
    if row_scale is not None:
        out = (out.float() * row_scale.unsqueeze(-1).float()).to(h.dtype)
    return out


# ------------------------------------------------------------------ linear
_wq_cache: dict = {}


def _quant_weight(w: torch.Tensor):
    """(rowwise q, sf, colwise q, sf) of a weight. A parameter's copies are cached until the
    optimizer changes it (forward, replay and backward of a step share them); a temporary
    tensor (a weight gathered from shards for one block) is quantised each time: caching it
    would keep a copy of every gathered weight alive."""
    K = _K()
    if not isinstance(w, torch.nn.Parameter):
        return K.quant_mxfp8(w.detach().reshape(-1, w.shape[-1]), rowwise=True, colwise=True)
    key = (w.data_ptr(), tuple(w.shape))
    hit = _wq_cache.get(key)
    if hit is not None and hit[0] == w._version:
        return hit[1]
    q = K.quant_mxfp8(w.detach().reshape(-1, w.shape[-1]), rowwise=True, colwise=True)
    _wq_cache[key] = (w._version, q)
    return q


def clear_weight_cache() -> None:
    _wq_cache.clear()


class _LinearBF16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, arrival):
        K = _K()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        ctx.save_for_backward(x2, w)
        ctx.shape = x.shape
        if arrival is not None:
            # w's rows are arriving from the ranks that own them (a sharded weight): the GEMM's
            # producer warp waits, per tile of output columns, for the owner's flag
            flags, epoch, rows = arrival
            y = K.gemm_bf16(x2, w, wait_flags=flags, wait_epoch=epoch, wait_rows=rows, wait_on_n=True)
        else:
            y = K.gemm_bf16(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm_bf16(dy2, w, b_mn=True).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None:
                K.gemm_bf16(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=True)
                dw = None
            else:
                dw = K.gemm_bf16(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None


class _LinearMX(torch.autograd.Function):
    """y = x·W^T with the GEMMs of `passes` in MXFP8: operands are quantised along the dimension
    each pass contracts (fprop K, dgrad N, wgrad M), as the reference's block-scaled
    linear does (architecture/precision/blockscaled.py:81-204). x^T is kept in MXFP8 for an
    MXFP8 wgrad; a pass that is not listed multiplies in bf16 and keeps its operand in bf16."""

    @staticmethod
    def forward(ctx, x, w, passes):
        K = _K()
        x2 = x.reshape(-1, x.shape[-1])
        m, k = x2.shape
        n = w.shape[0]
        need_w = w.requires_grad
        mx_w = "wgrad" in passes
        if "fprop" in passes:
            xq, xsf, xtq, xtsf = K.quant_mxfp8(x2, rowwise=True, colwise=need_w and mx_w)
            wq, wsf, _, _ = _quant_weight(w)
            y = K.gemm_mxfp8(xq, xsf, wq, wsf, m, n, k)
        else:
            x2 = x2.contiguous()
            y = K.gemm_bf16(x2, w)
            xtq = xtsf = None
            if need_w and mx_w:
                _, _, xtq, xtsf = K.quant_mxfp8(x2, rowwise=False, colwise=True)
        if mx_w:
            ctx.save_for_backward(xtq, xtsf, w)
        else:
            ctx.save_for_backward(x2.contiguous(), None, w)
        ctx.dims = (m, n, k, x.shape, passes)
        return y.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        xt, xtsf, w = ctx.saved_tensors
        m, n, k, shape, passes = ctx.dims
        dy2 = dy.reshape(-1, n).contiguous()
        need_dx, need_dw = ctx.needs_input_grad[:2]
        mx_d, mx_w = "dgrad" in passes, "wgrad" in passes
        gq = gsf = gtq = gtsf = None
        if (need_dx and mx_d) or (need_dw and mx_w):
            gq, gsf, gtq, gtsf = K.quant_mxfp8(dy2, rowwise=need_dx and mx_d, colwise=need_dw and mx_w)
        dx = dw = None
        if need_dx and mx_d:
            _, _, wtq, wtsf = _quant_weight(w)
            n_pad = wtq.shape[1]
            if n_pad != n:  # dy quantised along N must be padded like W^T
                gq2 = torch.zeros(m, n_pad, dtype=gq.dtype, device=gq.device)
                gq2[:, :n] = gq
                gq = gq2
            dx = K.gemm_mxfp8(gq, gsf, wtq, wtsf, m, k, n_pad).view(shape)
        elif need_dx:
            dx = K.gemm_bf16(dy2, w, b_mn=True).view(shape)
        if need_dw:
            main = getattr(w, "main_grad", None)
            if mx_w:
                m_pad = gtq.shape[1]
                if main is not None:
                    K.gemm_mxfp8(gtq, gtsf, xt, xtsf, n, k, m_pad, out=main, accumulate=True)
                else:
                    dw = K.gemm_mxfp8(gtq, gtsf, xt, xtsf, n, k, m_pad)
            elif main is not None:
                K.gemm_bf16(dy2, xt, a_mn=True, b_mn=True, out=main, accumulate=True)
            else:
                dw = K.gemm_bf16(dy2, xt, a_mn=True, b_mn=True)
        return dx, dw, None


class _LinearF32Out(torch.autograd.Function):
    """fp32 logits on the bf16 tensor cores. Products of bf16 values are exact in the fp32
    accumulator; an fp32 weight enters as hi + lo (two bf16 halves, 16 mantissa bits
    together) stacked into one GEMM whose two column halves are added."""

    @staticmethod
    def forward(ctx, x, w):
        K = _K()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        n = w.shape[0]
        if w.dtype == torch.float32:
            hi = w.to(torch.bfloat16)
            lo = (w - hi.float()).to(torch.bfloat16)
            y2 = K.gemm_bf16(x2, torch.cat((hi, lo), dim=0), out_dtype=torch.float32, bn=256 if 2 * n > 128 else 128)
            y = y2[:, :n] + y2[:, n:]
            wb = hi
        else:
            y = K.gemm_bf16(x2, w, out_dtype=torch.float32, bn=128 if n <= 128 else 256)
            wb = w
        ctx.save_for_backward(x2, wb)
        ctx.shape, ctx.w_dtype = x.shape, w.dtype
        return y.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x2, wb = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm_bf16(dy2, wb, b_mn=True).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw = K.gemm_bf16(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(ctx.w_dtype)
        return dx, dw


def linear_f32(x, w, bias=None):
    """x·W^T (+ bias) in fp32 (router logits, gates)."""
    k, n = x.shape[-1], w.shape[0]
    if (kernels_on(x) and x.dtype == torch.bfloat16 and w.dtype in (torch.bfloat16, torch.float32)
            and k % 8 == 0 and n % 8 == 0):
        y = _LinearF32Out.apply(x, w)
        return y if bias is None else y + bias.float()
    return F.linear(x.float(), w.float(), None if bias is None else bias.float())


PASSES = ("fprop", "dgrad", "wgrad")


def linear(x, w, bias=None, fmt: str = "bf16", passes=PASSES):
    """x [..., in] times w [out, in]^T (+ bias). `fmt`: "bf16" (compute dtype), "mxfp8" or
    "nvfp4"; `passes`: which of the projection's three GEMMs multiply in the format (the others
    in the compute dtype)."""
    k, n = x.shape[-1], w.shape[0]
    passes = tuple(passes)
    if not passes:
        fmt = "bf16"
    if fmt == "nvfp4" and k % 16 == 0 and n % 16 == 0:
        from . import nvfp4

        return nvfp4.linear(x, w, bias, passes=passes)
    if kernels_on(x) and w.dtype == torch.bfloat16 and k % 8 == 0 and n % 8 == 0:
        if fmt in ("mxfp8", "mxfp8_2d") and k % 128 == 0 and n % 128 == 0:
            y = _LinearMX.apply(x, w, passes)
        else:
            y = _LinearBF16.apply(x, w, getattr(w, "_bux_arrival", None))
        return y if bias is None else y + bias.to(y.dtype)
    if fmt in ("mxfp8", "mxfp8_2d") and k % 32 == 0 and not x.is_cuda and "fprop" in passes:
        return ref_linear_mxfp8(x, w, bias)
    return F.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))


def ref_linear_mxfp8(x, w, bias=None):
    """Fake-quantised linear with straight-through gradients: the CPU statement of the
    MXFP8 forward (the backward stays in the compute dtype)."""
    xq = ref.dequant_mxfp8(*ref.quant_mxfp8(x.detach())).to(x.dtype)
    wq = ref.dequant_mxfp8(*ref.quant_mxfp8(w.detach())).to(w.dtype)
    xs = x + (xq - x).detach()
    ws = w + (wq - w).detach()
    return F.linear(xs, ws.to(xs.dtype), None if bias is None else bias.to(xs.dtype))


# ------------------------------------------------------------------ causal depthwise convolution
class _CausalConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, position):
        K = _K()
        x = x.contiguous()
        wf = w.float().contiguous()
        pos = None if position is None else position.to(torch.int32).contiguous()
        ctx.save_for_backward(x, wf, pos)
        ctx.meta = (w.dtype, None if bias is None else bias.dtype)
        return K.causal_conv(x, wf, None if bias is None else bias.float().contiguous(), pos)

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        x, wf, pos = ctx.saved_tensors
        w_dtype, b_dtype = ctx.meta
        dy = dy.contiguous()
        dx = K.causal_conv(dy, wf, None, pos, bwd=True) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            dw, db = K.causal_conv_wgrad(x, dy, wf.shape[1], pos, bias=b_dtype is not None)
            dw = dw.to(w_dtype)
            db = None if db is None else db.to(b_dtype)
        return dx, dw, db, None


def causal_conv(x, w, bias=None, position=None):
    """Causal depthwise convolution over the tokens of [B, T, C] rows: y[t] = Σ_j w[:, j] x[t-j]
    (+ bias); taps that would reach across a document start (`position` < j) are dropped."""
    taps = w.shape[1]
    if kernels_on(x) and x.dim() == 3 and x.shape[-1] % 8 == 0 and taps <= 8:
        return _CausalConv.apply(x, w, bias, position)
    t = x.shape[1]
    wx = w.to(x.dtype)
    y = x * wx[:, 0]
    for j in range(1, min(taps, t)):
        shifted = F.pad(x[:, : t - j], (0, 0, j, 0))
        if position is not None:
            shifted = shifted * (position >= j).unsqueeze(-1).to(x.dtype)
        y = y + shifted * wx[:, j]
    return y if bias is None else y + bias.to(y.dtype)


# ------------------------------------------------------------------ attention
# Activation checkpointing may keep attention outputs across the replay of a block: the
# first run appends (o, lse) here, the replay takes them back in the same order instead of
# running the forward kernel again. ("save", list) / ("load", iterator) / None.
attention_replay = None


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sinks, causal, window, scale, segments):
        K = _K()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        sk = None if sinks is None else sinks.float().contiguous()
        # documents packed into a row: per-query first key and per-key last query
        row_lo, key_hi = K.document_bounds(segments) if segments is not None else (None, None)
        mode = attention_replay
        if mode is not None and mode[0] == "load":
            o, lse = next(mode[1])
        else:
            o, lse = K.attn_fwd(q, k, v, causal=causal, window=window, sinks=sk, scale=scale, row_lo=row_lo)
            if mode is not None:
                mode[1].append((o, lse))
        ctx.save_for_backward(q, k, v, o, lse, sk, row_lo, key_hi)
        ctx.cfg = (causal, window, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        K = _K()
        q, k, v, o, lse, sk, row_lo, key_hi = ctx.saved_tensors
        causal, window, scale = ctx.cfg
        dq, dk, dv, dsk = K.attn_bwd(q, k, v, o, do.contiguous(), lse, causal=causal, window=window,
                                     sinks=sk, scale=scale, row_lo=row_lo, key_hi=key_hi)
        return dq.to(q.dtype), dk, dv, dsk, None, None, None, None


def attention(q, k, v, *, causal: bool = True, window: Optional[int] = None, sinks=None,
              softcap: Optional[float] = None, scale: Optional[float] = None, segments=None):
    """[B,T,H,D] x [B,S,G,D] softmax attention; returns [B,T,H,D]."""
    d = q.shape[-1]
    packed = segments is not None
    native = (kernels_on(q) and d in (64, 128) and v.shape[-1] == d and softcap is None
              and (not packed or (causal and q.shape[1] == k.shape[1] and torch.is_tensor(segments))))
    if native:
        return _Attention.apply(q, k, v, sinks, causal, int(window or 0), scale, segments)
    if (q.is_cuda and softcap is None and segments is None and sinks is None and window is None
            and q.dtype in (torch.bfloat16, torch.float16)):
        # library baseline (BUX_KERNELS=off, or a head dim the kernel does not take)
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                             is_causal=causal, scale=scale, enable_gqa=True)
        return out.transpose(1, 2)
    out, _ = ref.attention(q, k, v, causal=causal, window=window, sinks=sinks, softcap=softcap,
                           scale=scale, segments=segments)
    return out
