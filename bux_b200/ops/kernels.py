"""Thin Python wrappers over ``torch.ops.bux_b200``: allocate outputs, pass shapes.

No autograd here (see `functional`). Every function takes CUDA tensors and raises if
the native library is missing: the GPU path never falls back to eager PyTorch.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _build, checks

KIND_BF16, KIND_MXFP8 = 0, 1
MODE_DENSE, MODE_GROUPED_ROWS, MODE_GROUPED_K = 0, 1, 2
OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_BF16_ACC = 0, 1, 2, 3
ACT_KINDS = {"swish": 0, "quick_gelu": 1, "gelu_tanh": 2, "relu2": 3}

_status: dict = {}
launches = 0  # kernels launched through this module (bench.py reports it)


def ops():
    _build.load(required=True)
    return torch.ops.bux_b200


def _out(*shape, dtype, device, op: str, fill=None) -> torch.Tensor:
    """A kernel's output buffer: between guard regions when kernel checks are on."""
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    return checks.guarded_empty(shape, dtype, device, op, fill)


def _count(n: int = 1) -> None:
    global launches
    launches += n


def status_word(device) -> torch.Tensor:
    """Per-device int32[2] the kernels' bounded waits report into."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device, what: str = "kernel") -> None:
    """Raise if any bounded wait of a kernel on `device` ran out (synchronises)."""
    st = status_word(device)
    code, count = st.tolist()
    if code:
        st.zero_()
        raise RuntimeError(
            f"{what}: a bounded device wait ran out (kernel {code >> 24}, site {(code >> 16) & 0xff}, "
            f"block {code & 0xffff}; {count} waits in total)")


# ------------------------------------------------------------------ GEMM
def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
              out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
              accumulate: bool = False, bn: int = 256, sms: int = 0, wait_flags=None, wait_epoch: int = 0,
              wait_rows: int = 0, m_rotate: int = 0, wait_on_k: bool = False, wait_on_n: bool = False) -> torch.Tensor:
    """C = A · B^T. A is [M,K] (or stored [K,M] with a_mn), B is [N,K] (or [K,N] with b_mn).
    With `wait_flags` (int32[senders]) an operand is being written by peer GPUs in blocks
    of `wait_rows` rows per sender (rows of A, of the contraction with `wait_on_k`, or rows of B
    with `wait_on_n`: a weight whose shards arrive from their owners):
    a tile's loads wait for its sender's flag to reach `wait_epoch`; `m_rotate` (tiles)
    starts the walk at this rank's own rows."""
    m, k = (a.shape[1], a.shape[0]) if a_mn else a.shape
    n = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = _out(m, n, dtype=out_dtype, device=a.device, op="gemm_bf16")
    kind = OUT_BF16 if out.dtype == torch.bfloat16 else (OUT_F32_ACC if accumulate else OUT_F32)
    ops().gemm(a, b, out, None, None, None, status_word(a.device), KIND_BF16, MODE_DENSE, m, n, k, k, 1,
               a_mn, b_mn, kind, bn, sms, wait_flags, wait_epoch, wait_rows, m_rotate, wait_on_k, wait_on_n)
    _count()
    return out


def _tile_width(n: int) -> int:
    """256-wide tiles halve the operand traffic per FLOP; taken when they tile N exactly."""
    return 256 if n % 256 == 0 else 128


def gemm_mxfp8(aq, asf, bq, bsf, m: int, n: int, k: int, *, out=None, out_dtype=torch.bfloat16,
               accumulate: bool = False, bn: Optional[int] = None, sms: int = 0) -> torch.Tensor:
    """C[m,n] = dequant(A)[m,k] · dequant(B)[n,k]^T; scales in the tiled layout."""
    bn = _tile_width(n) if bn is None else bn
    if out is None:
        out = _out(m, n, dtype=out_dtype, device=aq.device, op="gemm_mxfp8")
    kind = OUT_BF16 if out.dtype == torch.bfloat16 else (OUT_F32_ACC if accumulate else OUT_F32)
    ops().gemm(aq.view(torch.uint8), bq.view(torch.uint8), out, asf, bsf, None, status_word(aq.device),
               KIND_MXFP8, MODE_DENSE, m, n, k, k, 1, False, False, kind, bn, sms)
    _count()
    return out


def grouped_gemm(a, b, offsets: torch.Tensor, n: int, k: int, *, kind: int = KIND_BF16, asf=None,
                 bsf=None, b_mn: bool = False, out=None, bn: Optional[int] = None, sms: int = 0,
                 wait_flags=None, wait_epoch: int = 0) -> torch.Tensor:
    """Rows of `a` ([R,k], sorted by group; offsets int32[G+1]) times group g's weight.
    b: [G*n, k] (K-major) or [G*k, n] (b_mn). Returns [R, n] bf16."""
    bn = _tile_width(n) if bn is None else bn
    groups = offsets.numel() - 1
    if out is None:
        out = _out(a.shape[0], n, dtype=torch.bfloat16, device=a.device, op="grouped_gemm")
    if kind == KIND_MXFP8:
        a, b = a.view(torch.uint8), b.view(torch.uint8)
    ops().gemm(a, b, out, asf, bsf, offsets, status_word(a.device), kind, MODE_GROUPED_ROWS,
               a.shape[0], n, k, k, groups, False, b_mn, OUT_BF16, bn, sms, wait_flags, wait_epoch)
    _count()
    return out


def grouped_gemm_k(a, b, offsets: torch.Tensor, m: int, n: int, *, kind: int = KIND_BF16, asf=None,
                   bsf=None, a_mn: bool = False, b_mn: bool = False, out=None,
                   accumulate: bool = False, bn: Optional[int] = None, sms: int = 0,
                   out_dtype=torch.float32) -> torch.Tensor:
    """out[g] (+)= A[:, kg] · B[:, kg]^T for each group's contraction range kg (weight
    gradients of grouped experts). K-major: a [m, Ktot], b [n, Ktot]; MN-major: a [Ktot, m],
    b [Ktot, n]. Returns [G, m, n] in `out_dtype` (fp32, or bf16 written straight from the
    accumulator when that is what the gradient is kept in)."""
    bn = _tile_width(n) if bn is None else bn
    groups = offsets.numel() - 1
    ktot = a.shape[0] if a_mn else a.shape[1]
    if out is None:
        out = _out(groups, m, n, dtype=out_dtype, device=a.device, op="grouped_gemm_k")
        accumulate = False
    if kind == KIND_MXFP8:
        a, b = a.view(torch.uint8), b.view(torch.uint8)
    if out.dtype == torch.bfloat16:
        okind = OUT_BF16_ACC if accumulate else OUT_BF16   # the sum is rounded to bf16 after every call
    else:
        okind = OUT_F32_ACC if accumulate else OUT_F32
    ops().gemm(a, b, out, asf, bsf, offsets, status_word(a.device), kind, MODE_GROUPED_K, m, n, ktot,
               ktot, groups, a_mn, b_mn, okind, bn, sms)
    _count()
    return out


# ------------------------------------------------------------------ MXFP8 quantiser
def sf_bytes(rows: int, cols: int) -> int:
    """Bytes of the tiled scale tensor of a [rows, cols] matrix quantised along cols."""
    return (-(-rows // 128)) * (-(-(cols // 32) // 4)) * 512


def quant_mxfp8_batched(x: torch.Tensor, *, rowwise: bool = True, colwise: bool = False):
    """Quantise every matrix of a stack x [E, R, C] (R % 128 == 0 when colwise).
    Returns (q_row [E*R, C], sf_row, q_col [E*C, R], sf_col): the 2-D views a grouped
    GEMM takes as its per-group operand."""
    e, r, c = x.shape
    dev = x.device
    q_row = sf_row = q_col = sf_col = None
    if rowwise:
        assert r % 128 == 0 or e == 1, "rowwise scale tiles of a stack need R % 128 == 0"
        q_row = _out(e * r, c, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8_batched q_row")
        sf_row = _out(e * sf_bytes(r, c), dtype=torch.uint8, device=dev, op="quant_mxfp8_batched sf_row")
    if colwise:
        assert r % 128 == 0 and c % 128 == 0
        q_col = _out(e * c, r, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8_batched q_col")
        sf_col = _out(e * sf_bytes(c, r), dtype=torch.uint8, device=dev, op="quant_mxfp8_batched sf_col")
    xc = x.contiguous()
    ops().quant_mxfp8(xc, None, None, None if q_row is None else q_row.view(torch.uint8), sf_row,
                      None if q_col is None else q_col.view(torch.uint8), sf_col, r, c, r, e, r * c)
    _count()
    return q_row, sf_row, q_col, sf_col


def quant_mxfp8(x: torch.Tensor, *, rowwise: bool = True, colwise: bool = False,
                row_index: Optional[torch.Tensor] = None, rows: Optional[int] = None,
                row_scale: Optional[torch.Tensor] = None):
    """Quantise bf16 x [R, C] along C (rowwise) and/or along R (colwise; a transposed
    copy [C, R_pad]). With `row_index` (int32[rows]) output row r reads x[row_index[r]]
    (negative: zeros); with `row_scale` (fp32[rows]) it is multiplied by row_scale[r] and
    rounded to bf16 first. Returns (q_row, sf_row, q_col, sf_col); unused ones are None."""
    x2 = x.reshape(-1, x.shape[-1])
    c = x2.shape[1]
    r = rows if rows is not None else (row_index.numel() if row_index is not None else x2.shape[0])
    dev = x.device
    q_row = sf_row = q_col = sf_col = None
    if rowwise:
        q_row = _out(r, c, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8 q_row")
        sf_row = _out(sf_bytes(r, c), dtype=torch.uint8, device=dev, op="quant_mxfp8 sf_row")
    r_pad = -(-r // 128) * 128
    if colwise:
        # the kernel writes every byte of both outputs, padding included
        q_col = _out(c, r_pad, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8 q_col")
        sf_col = _out(sf_bytes(c, r_pad), dtype=torch.uint8, device=dev, op="quant_mxfp8 sf_col")
    ops().quant_mxfp8(x2, row_index, row_scale, None if q_row is None else q_row.view(torch.uint8), sf_row,
                      None if q_col is None else q_col.view(torch.uint8), sf_col, r, c, r_pad, 1, 0)
    _count()
    return q_row, sf_row, q_col, sf_col


def quant_mxfp8_glu(h: torch.Tensor, dout: Optional[torch.Tensor] = None, kind: str = "swish", *,
                    rowwise: bool = True, colwise: bool = False, limit: float = 0.0, up_offset: float = 0.0,
                    row_scale: Optional[torch.Tensor] = None):
    """MXFP8 copies of glu(h) [R, f] (`dout` None), or of the gradient of h [R, 2f] for the
    output gradient `dout` [R, f], computed from h [R, 2f] inside the quantiser: the bf16
    activation (gradient) is never written. Same values as `quant_mxfp8(glu_fwd(h))` /
    `quant_mxfp8(glu_bwd(h, dout))`. `row_scale` (fp32 [rows], activation only) multiplies each
    row before it is rounded, as `glu_fwd(h, kind, row_scale)`. Returns (q_row, sf_row, q_col, sf_col)."""
    r, f2 = h.shape
    c = f2 if dout is not None else f2 // 2
    dev = h.device
    q_row = sf_row = q_col = sf_col = None
    if rowwise:
        q_row = _out(r, c, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8_glu q_row")
        sf_row = _out(sf_bytes(r, c), dtype=torch.uint8, device=dev, op="quant_mxfp8_glu sf_row")
    r_pad = -(-r // 128) * 128
    if colwise:
        q_col = _out(c, r_pad, dtype=torch.float8_e4m3fn, device=dev, op="quant_mxfp8_glu q_col")
        sf_col = _out(sf_bytes(c, r_pad), dtype=torch.uint8, device=dev, op="quant_mxfp8_glu sf_col")
    ops().quant_mxfp8_glu(h, dout, row_scale, None if q_row is None else q_row.view(torch.uint8), sf_row,
                          None if q_col is None else q_col.view(torch.uint8), sf_col, r_pad,
                          ACT_KINDS[kind], float(limit), float(up_offset))
    _count()
    return q_row, sf_row, q_col, sf_col


def quant_nvfp4(x: torch.Tensor):
    """NVFP4 of bf16 x [R, C] along its rows (1 x 16 blocks, to nearest): (packed uint8 [R, C/2],
    two E2M1 codes per byte with the lower column in the low nibble; E4M3 scale bytes [R, C/16];
    the fp32 tensor scale). Bit-equal to `nvfp4.pack(nvfp4.quantize(x))`."""
    r, c = x.shape
    tensor_scale = (x.abs().max().float().clamp_min(1e-30) / (6.0 * 448.0)).reshape(1)
    packed = _out(r, c // 2, dtype=torch.uint8, device=x.device, op="quant_nvfp4 packed")
    scales = _out(r, c // 16, dtype=torch.uint8, device=x.device, op="quant_nvfp4 scales")
    ops().quant_nvfp4(x.contiguous(), tensor_scale, packed, scales)
    _count()
    return packed, scales, tensor_scale


# ------------------------------------------------------------------ norms / rope / glu
def rmsnorm_fwd(x, w, eps: float):
    y = _out(x.shape, dtype=x.dtype, device=x.device, op="rmsnorm_fwd y")
    rstd = _out(x.numel() // x.shape[-1], dtype=torch.float32, device=x.device, op="rmsnorm_fwd rstd")
    ops().rmsnorm_fwd(x, w, y, rstd, eps)
    _count()
    return y, rstd


def rmsnorm_bwd(x, w, dy, rstd, need_dw: bool = True):
    dx = _out(x.shape, dtype=x.dtype, device=x.device, op="rmsnorm_bwd dx")
    dw = (_out(x.shape[-1], dtype=torch.float32, device=x.device, op="rmsnorm_bwd dw", fill=0.0)
          if need_dw and w is not None else None)
    ops().rmsnorm_bwd(x, w, dy, rstd, dx, dw)
    _count()
    return dx, dw


def token_stride(x) -> Optional[int]:
    """Elements between tokens of x [..., T, H, D] when heads are dense and the leading
    dimensions collapse into one (a column slice of a fused projection); else None."""
    d, h = x.shape[-1], x.shape[-2]
    if x.stride(-1) != 1 or x.stride(-2) != d or x.dim() < 3:
        return None
    step = x.stride(-3)
    for i in range(x.dim() - 4, -1, -1):
        if x.stride(i) != x.shape[i + 1] * x.stride(i + 1):
            return None
    return step if step % 8 == 0 and x.data_ptr() % 16 == 0 else None


def norm_rope_fwd(x, w, cos, sin, eps: float):
    """x: [..., T, H, D], dense or a column slice (see `token_stride`); cos/sin: [tokens, D/2] fp32."""
    d, h = x.shape[-1], x.shape[-2]
    tokens = x.numel() // (h * d)
    y = _out(x.shape, dtype=x.dtype, device=x.device, op="norm_rope_fwd y")
    rstd = _out(tokens * h, dtype=torch.float32, device=x.device, op="norm_rope_fwd rstd") if w is not None else None
    ops().norm_rope(False, x, w, cos, sin, y, rstd, None, None, tokens, h, d, token_stride(x), h * d, eps)
    _count()
    return y, rstd


def norm_rope_bwd(x, w, cos, sin, rstd, dy, eps: float):
    d, h = x.shape[-1], x.shape[-2]
    tokens = x.numel() // (h * d)
    dx = _out(x.shape, dtype=x.dtype, device=x.device, op="norm_rope_bwd dx")
    dw = _out(d, dtype=torch.float32, device=x.device, op="norm_rope_bwd dw", fill=0.0) if w is not None else None
    ops().norm_rope(True, x, w, cos, sin, dx, rstd, dy, dw, tokens, h, d, token_stride(x), h * d, eps)
    _count()
    return dx, dw


def glu_fwd(h, kind: str = "swish", row_scale=None, limit: float = 0.0, up_offset: float = 0.0):
    out = _out(*h.shape[:-1], h.shape[-1] // 2, dtype=h.dtype, device=h.device, op="glu_fwd")
    ops().glu_fwd(h, out, row_scale, ACT_KINDS[kind], limit or 0.0, up_offset)
    _count()
    return out


def glu_bwd(h, dout, kind: str = "swish", row_scale=None, limit: float = 0.0, up_offset: float = 0.0):
    dh = _out(h.shape, dtype=h.dtype, device=h.device, op="glu_bwd dh")
    drs = (_out(row_scale.shape, dtype=row_scale.dtype, device=h.device, op="glu_bwd d_row_scale", fill=0.0)
           if row_scale is not None else None)
    ops().glu_bwd(h, dout, dh, row_scale, drs, ACT_KINDS[kind], limit or 0.0, up_offset)
    _count()
    return dh, drs


def glu_bwd_into(h, dout, kind: str, row_scale, d_row_scale, limit: float = 0.0, up_offset: float = 0.0):
    """`glu_bwd` whose per-row gradient of `row_scale` lands in the caller's fp32 buffer
    (cleared here first: the kernel adds into it). Returns dh."""
    dh = _out(h.shape, dtype=h.dtype, device=h.device, op="glu_bwd dh")
    d_row_scale.zero_()
    ops().glu_bwd(h, dout, dh, row_scale, d_row_scale, ACT_KINDS[kind], limit or 0.0, up_offset)
    _count()
    return dh


# ------------------------------------------------------------------ loss / optimiser / rows
def ce_fwd_bwd(logits, targets, mask, grad_scale: float, z_weight: float = 0.0, softcap: float = 0.0):
    """In place: logits become dlogits. Returns per-row loss (fp32)."""
    loss = _out(logits.shape[0], dtype=torch.float32, device=logits.device, op="ce_fwd_bwd loss")
    ops().ce_fwd_bwd(logits, targets, mask, loss, None, grad_scale, z_weight, softcap or 0.0)
    _count()
    return loss


def adamw(p, g, m, v, *, lr, b1, b2, eps, wd, step: int, m_sf=None, v_sf=None, shadow=None,
          grad_scale: Optional[torch.Tensor] = None, grad_scale_const: float = 1.0) -> None:
    ops().adamw(p, g, m, v, m_sf, v_sf, shadow, grad_scale, lr, b1, b2, eps, wd,
                1.0 - b1 ** step, 1.0 - b2 ** step, grad_scale_const)
    _count()


def sumsq(g, out) -> None:
    ops().sumsq(g, out)
    _count()


def topk_rows(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices [..., k] (int64) of the k largest entries along the last dimension of fp32
    scores (at most 512 wide), in descending order of value; ties go to the lower index."""
    flat = scores.reshape(-1, scores.shape[-1]).contiguous()
    idx = _out(flat.shape[0], k, dtype=torch.int64, device=scores.device, op="topk_rows")
    ops().topk_rows(flat, idx)
    _count()
    return idx.view(*scores.shape[:-1], k)


def gather_rows(x, index, rows: int):
    out = _out(rows, x.shape[-1], dtype=x.dtype, device=x.device, op="gather_rows")
    ops().gather_rows(x, index, out)
    _count()
    return out


def combine_bwd(y, dout, pos, w, rows: int):
    """Backward of `combine_rows`: dy [rows, d] (pad rows zero) and dw [T, k] (None
    without y)."""
    dy = torch.zeros(rows, dout.shape[-1], dtype=dout.dtype, device=dout.device)
    dw = torch.empty(pos.shape, dtype=torch.float32, device=dout.device) if y is not None else None
    ops().combine_bwd(y, dout, pos, w, dy, dw)
    _count()
    return dy, dw


def combine_dots(y, dout, pos):
    """dw [T, k] of `combine_rows` alone: <y[pos[t, j]], dout[t]> (0 for dropped picks)."""
    dw = torch.empty(pos.shape, dtype=torch.float32, device=dout.device)
    ops().combine_bwd(y, dout, pos, None, None, dw)
    _count()
    return dw


def combine_rows(y, pos, w, tokens: int):
    out = _out(tokens, y.shape[-1], dtype=y.dtype, device=y.device, op="combine_rows")
    ops().combine_rows(y, pos, w, out)
    _count()
    return out


def combine_rows_into(y, pos, w, out) -> None:
    """out[t] = Σ_j w[t,j] · y[pos[t,j]] (w None: a plain sum) into a contiguous `out` [T, d]."""
    assert out.is_contiguous()
    ops().combine_rows(y, pos, w, out)
    _count()


# ------------------------------------------------------------------ attention
def document_bounds(segments: torch.Tensor):
    """(row_lo, key_hi) int32 [B, T] of packed rows from their document ids (non-decreasing
    along a row): the first position of each position's document, and its last."""
    seg = segments.contiguous()
    row_lo = torch.searchsorted(seg, seg, right=False).to(torch.int32)
    key_hi = (torch.searchsorted(seg, seg, right=True) - 1).to(torch.int32)
    return row_lo.contiguous(), key_hi.contiguous()


def attn_fwd(q, k, v, *, causal=True, window=0, sinks=None, scale=None, row_lo=None):
    b, t, h, d = q.shape
    o = _out(q.shape, dtype=q.dtype, device=q.device, op="attn_fwd o")
    lse = _out(b, h, t, dtype=torch.float32, device=q.device, op="attn_fwd lse")
    ops().attn_fwd(q, k, v, o, lse, sinks, status_word(q.device), scale if scale is not None else d ** -0.5,
                   causal, window or 0, row_lo)
    _count()
    return o, lse


def attn_bwd(q, k, v, o, do, lse, *, causal=True, window=0, sinks=None, scale=None, row_lo=None, key_hi=None,
             phase_cycles=None):
    """(dq fp32, dk, dv, dsinks). `phase_cycles` (int32[32] on the device, optional): the CTA of the
    first key tile adds the cycles its softmax warp 0 (slots 0-13) and its MMA issuer (16-23) spent
    in each phase of the schedule."""
    b, t, h, d = q.shape
    dq = _out(b, t, h, d, dtype=torch.float32, device=q.device, op="attn_bwd dq", fill=0.0)
    dk = _out(k.shape, dtype=k.dtype, device=k.device, op="attn_bwd dk")
    dv = _out(v.shape, dtype=v.dtype, device=v.device, op="attn_bwd dv")
    delta = _out(b, h, t, dtype=torch.float32, device=q.device, op="attn_bwd delta")
    dsinks = torch.zeros_like(sinks) if sinks is not None else None
    ops().attn_bwd(q, k, v, o, do, lse, dq, dk, dv, delta, sinks, dsinks, status_word(q.device),
                   scale if scale is not None else d ** -0.5, causal, window or 0, row_lo, key_hi, phase_cycles)
    _count(2)
    return dq, dk, dv, dsinks


# ------------------------------------------------------------------ expert-parallel exchange
def ep_push_rows(x, src_token, dst_rank, dst_row, peer_base, row_scale=None, sms: int = 0, peer_scale=None) -> None:
    """Row i of the picks (x[src_token[i]]) → row dst_row[i] of rank dst_rank[i]'s buffer.
    With `row_scale` the row is multiplied on the way; with `peer_scale` as well (the peers'
    fp32 [rows] buffers) it travels unscaled and the scale is stored beside it instead."""
    ops().ep_push_rows(x, src_token, dst_rank, dst_row, row_scale, peer_base, sms, peer_scale)
    _count()


def ep_push_rows_mx(x, rank_of, row_of, peer_q, peer_sf, weights=None, peer_scale=None, sms: int = 0) -> None:
    """Token t's row → row `row_of[t, j]` of rank `rank_of[t, j]`'s buffers for each of its picks,
    read and quantised once (MXFP8 along the row): e4m3 bytes into the peers' [cap, d] byte buffers,
    E8M0 scales row-major into their [cap, d/32] byte buffers (`sf_rows_to_tiles` makes the GEMM's
    tiles of them on the owner); `weights[t, j]` (a pick's router weight, fp32) is stored
    beside the row in the peers' fp32 `peer_scale` buffers, not applied."""
    ops().ep_push_rows_mx(x, rank_of, row_of, weights, peer_q, peer_sf, peer_scale, sms)
    _count()


def causal_conv(x: torch.Tensor, w: torch.Tensor, bias=None, position=None, bwd: bool = False) -> torch.Tensor:
    """y[b,t,c] = Σ_j w[c,j] x[b,t-j,c] (+ bias) over [B, T, C] bf16 rows, w fp32 [C, taps <= 8]; a tap
    is dropped where `position` (int32 [B, T], the position inside its document; None: whole rows)
    is smaller than j. With `bwd` the same taps run forwards in time: the gradient by x of dy."""
    out = _out(x.shape, dtype=x.dtype, device=x.device, op="causal_conv")
    ops().causal_conv(bwd, x, w, bias, position, out)
    _count()
    return out


def causal_conv_wgrad(x, dy, taps: int, position=None, bias: bool = False):
    """(dw fp32 [C, taps], db fp32 [C] or None) of `causal_conv`."""
    c = x.shape[-1]
    dw = torch.zeros(c, taps, dtype=torch.float32, device=x.device)
    db = torch.zeros(c, dtype=torch.float32, device=x.device) if bias else None
    ops().causal_conv_wgrad(x, dy, position, dw, db)
    _count()
    return dw, db


def sf_rows_to_tiles(src: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Row-major E8M0 scales [rows, cols/32] → the scale tiles a block-scaled GEMM reads."""
    rows, sf_cols = src.shape
    if out is None:
        out = _out(sf_bytes(rows, sf_cols * 32), dtype=torch.uint8, device=src.device, op="sf_rows_to_tiles")
    ops().sf_rows_to_tiles(src, out)
    _count()
    return out


def requant_mxfp8_cols(q: torch.Tensor, sf: torch.Tensor, rows: int, cols: int):
    """(q_col [cols, rows padded to 128], sf_col): the transposed MXFP8 copy, quantised along the
    rows, of a matrix that is MXFP8 along its columns already (e4m3 bytes [rows, cols] + scale
    tiles). Same values as quantising the dequantised matrix column-wise."""
    r_pad = -(-rows // 128) * 128
    q_col = _out(cols, r_pad, dtype=torch.float8_e4m3fn, device=q.device, op="requant_mxfp8_cols q_col")
    sf_col = _out(sf_bytes(cols, r_pad), dtype=torch.uint8, device=q.device, op="requant_mxfp8_cols sf_col")
    ops().requant_mxfp8_cols(q.view(torch.uint8), sf, q_col.view(torch.uint8), sf_col, rows, cols, r_pad)
    _count()
    return q_col, sf_col


def ep_signal(peer_flags, channel: int, world: int, my_rank: int, epoch: int) -> None:
    ops().ep_signal(peer_flags, channel, world, my_rank, epoch)
    _count()


def ep_pull_combine(peer_base, rank_of, row_of, w, tokens: int, d: int, dtype, flags=None, epoch: int = 0,
                    limit_s: float = 5.0, out=None):
    """out[t] = Σ_j w[t,j] · rows of the peers' buffers (w None: a plain sum), into `out` when given."""
    if out is None:
        out = torch.empty(tokens, d, dtype=dtype, device=rank_of.device)
    assert out.is_contiguous() and out.shape == (tokens, d)
    ops().ep_pull_combine(peer_base, rank_of, row_of, w, out, flags, epoch, status_word(rank_of.device), limit_s)
    _count()
    return out


def ep_pull_dot(peer_base, rank_of, row_of, dout):
    dw = torch.empty(row_of.shape, dtype=torch.float32, device=dout.device)
    ops().ep_pull_dot(peer_base, rank_of, row_of, dout, dw)
    _count()
    return dw


def row_dots(a, b, out=None):
    """out[r] = <a[r], b[r]> in fp32 over bf16 rows."""
    if out is None:
        out = torch.empty(a.shape[0], dtype=torch.float32, device=a.device)
    ops().row_dots(a, b, out)
    _count()
    return out


def ep_pull_scalar(peer_base, rank_of, row_of, flags=None, epoch: int = 0, limit_s: float = 5.0, out=None):
    """out[t, j] = the fp32 value at row row_of[t, j] of rank rank_of[t, j]'s buffer."""
    if out is None:
        out = torch.empty(row_of.shape, dtype=torch.float32, device=row_of.device)
    assert out.is_contiguous() and out.shape == row_of.shape and out.dtype == torch.float32
    ops().ep_pull_scalar(peer_base, rank_of, row_of, out, flags, epoch, status_word(row_of.device), limit_s)
    _count()
    return out


def set_comm_ctas_per_sm(n: int) -> None:
    """CTAs per SM the expert-exchange kernels may take (0: each kernel's own default)."""
    ops().set_comm_ctas_per_sm(int(n))


def ep_wait(flags, epoch: int, limit_s: float = 5.0) -> None:
    ops().ep_wait(flags, epoch, status_word(flags.device), limit_s)
    _count()


def tp_push_block(src, peer_base, my_rank: int, sms: int = 0) -> None:
    """This rank's rows → row block `my_rank` of every peer's gather buffer (P2P stores)."""
    ops().tp_push_block(src, peer_base, my_rank, sms)
    _count()


def tp_pull_reduce(peer_base, my_rank: int, out, residual=None, flags=None, epoch: int = 0,
                   limit_s: float = 5.0) -> None:
    """out = (residual +) Σ_peers partial_peer[row block my_rank] (P2P loads, fp32 sums)."""
    ops().tp_pull_reduce(peer_base, my_rank, out, residual, flags, epoch, status_word(out.device), limit_s)
    _count()


def zero_pad_rows(buf, offsets, counts) -> None:
    ops().zero_pad_rows(buf, offsets, counts)
    _count()
