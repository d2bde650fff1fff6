"""Composite differentiable ops: the chunked LM-head cross-entropy and the sorted
MoE expert stack (permute → grouped GLU GEMMs → weighted combine).

Reference behaviour: ``architecture/logits.py:209-353`` (logits never materialised
whole; head gradients computed in the forward) and ``architecture/experts/moe.py:634``
(`run_sorted`) with ``token_rows`` / ``token_sums`` (``:992-1071``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import reference as ref
from .functional import _K, kernels_on

CE_CHUNK_BYTES = 1 << 31  # logits held at once (bf16): fewer, larger chunks mean fewer passes over dW


# ------------------------------------------------------------------ LM head + loss
class _CEHead(torch.autograd.Function):
    """sum over kept tokens of CE(x·W^T, target). The forward walks token chunks:
    logits chunk (tcgen05 GEMM) → loss + dlogits in place (one kernel) → dX chunk and
    dW accumulation (two GEMMs). The backward only scales by the incoming gradient."""

    @staticmethod
    def forward(ctx, x, w, targets, mask, z_weight, softcap):
        K = _K()
        t, d = x.shape
        v = w.shape[0]
        rows = max(128, min(t, (CE_CHUNK_BYTES // (2 * v)) // 128 * 128))
        need_dx, need_dw = x.requires_grad, w.requires_grad
        dx = torch.empty_like(x) if need_dx else None
        main = getattr(w, "main_grad", None)
        dw = None
        if need_dw:
            dw = main if main is not None else torch.zeros(v, d, dtype=torch.float32, device=x.device)
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        tg = targets.to(torch.int32).contiguous()
        mk = None if mask is None else mask.float().contiguous()
        for s in range(0, t, rows):
            e = min(t, s + rows)
            xc = x[s:e]
            logits = K.gemm_bf16(xc, w)
            per_row = K.ce_fwd_bwd(logits, tg[s:e], None if mk is None else mk[s:e], 1.0, z_weight,
                                   softcap or 0.0)
            loss += per_row.sum()
            if need_dx:
                K.gemm_bf16(logits, w, b_mn=True, out=dx[s:e])
            if need_dw:
                K.gemm_bf16(logits, xc, a_mn=True, b_mn=True, out=dw, accumulate=True)
        ctx.save_for_backward(dx, None if main is not None else dw)
        ctx.main = main is not None
        return loss

    @staticmethod
    def backward(ctx, g):
        dx, dw = ctx.saved_tensors
        gx = None if dx is None else (dx.float() * g).to(dx.dtype)
        gw = None if dw is None else dw * g
        return gx, gw, None, None, None, None


def cross_entropy_head(x, w, targets, mask=None, *, bias=None, z_weight: float = 0.0,
                       softcap: Optional[float] = None):
    """(sum of per-token losses over kept positions, number kept). x [T,d], w [V,d]."""
    count = (torch.tensor(float(targets.numel()), device=x.device) if mask is None
             else mask.float().sum())
    native = (kernels_on(x) and bias is None and w.dtype == torch.bfloat16
              and w.shape[0] % 8 == 0 and x.shape[-1] % 8 == 0
              and getattr(w, "main_grad", None) is None)
    if native:
        return _CEHead.apply(x.contiguous(), w, targets, mask, float(z_weight), softcap), count
    # plain path, a chunk of tokens at a time so the fp32 logits stay bounded
    t = x.shape[0]
    rows = max(1, min(t, (1 << 28) // max(1, w.shape[0])))
    total = x.new_zeros((), dtype=torch.float32)
    for s in range(0, t, rows):
        logits = F.linear(x[s:s + rows], w.to(x.dtype), None if bias is None else bias.to(x.dtype))
        part, _ = ref.cross_entropy(logits, targets[s:s + rows],
                                    None if mask is None else mask[s:s + rows], z_weight, softcap)
        total = total + part
    return total, count


def _grad_dtype(w: torch.Tensor):
    """bf16 weight gradients leave the GEMM as bf16; anything else as fp32."""
    return torch.bfloat16 if w.dtype == torch.bfloat16 else torch.float32


# ------------------------------------------------------------------ sorted MoE experts
def sort_picks(experts: torch.Tensor, num_experts: int, align: int = 128):
    """Expert-sorted, `align`-padded layout of the T·k picks, with static shapes.

    Returns (row_index int32[R] = source token of each padded row or -1,
    pos int32[T,k] = padded row of each pick, offsets int32[E+1]) where
    R = T·k + E·(align-1) rounded up to `align` bounds the padded rows."""
    t, k = experts.shape
    dev = experts.device
    flat = experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + align - 1) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    offsets[1:] = padded.cumsum(0)
    starts = counts.cumsum(0) - counts  # first sorted index of each expert
    sorted_expert = flat[order]
    rank = torch.arange(t * k, device=dev) - starts[sorted_expert]
    dest = offsets[:-1][sorted_expert] + rank
    r_max = -(-(t * k + num_experts * (align - 1)) // align) * align
    row_index = torch.full((r_max,), -1, dtype=torch.int32, device=dev)
    row_index[dest] = (order // k).to(torch.int32)
    pos = torch.empty(t * k, dtype=torch.int32, device=dev)
    pos[order] = dest.to(torch.int32)
    return row_index, pos.view(t, k), offsets.to(torch.int32)


def _row_weights(wts: torch.Tensor, pos: torch.Tensor, rows: int) -> torch.Tensor:
    """fp32[rows]: the router weight of each expert-sorted row (0 for padding rows)."""
    w_row = torch.zeros(rows, dtype=torch.float32, device=wts.device)
    w_row[pos.reshape(-1).long()] = wts.reshape(-1)
    return w_row


class _SortedExperts(torch.autograd.Function):
    """out[t] = Σ_j w[t,j] · expert_{e[t,j]}(x[t]) on one GPU.

    A row's router weight multiplies its *activation* (a' = w · glu(h)), so the down
    projection already yields weighted rows and the combine is a plain sum. In the
    backward the gradient of the weights then falls out of the activation's backward
    (d w = <da', glu(h)>, one scalar per row from `glu_bwd`), and the experts' outputs are
    never needed again. Tokens are walked in `chunks` equal ranges, which bounds the
    sorted intermediates (rows × 2f and rows × d) to one range at a time; weight
    gradients accumulate over the ranges in fp32."""

    @staticmethod
    def forward(ctx, x, w_gu, w_down, weights, experts, act, limit, up_offset, mx, chunks):
        K = _K()
        t, d = x.shape
        e, f2, _ = w_gu.shape
        f = f2 // 2
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        grad = any(ctx.needs_input_grad)
        wts = weights.float().contiguous()
        chunks = chunks if chunks > 1 and t % chunks == 0 else 1
        tc = t // chunks
        out = torch.empty(t, d, dtype=x.dtype, device=x.device)
        if mx:
            # both orientations of the weights in one pass when a backward follows
            gq, gsf, gtq, gtsf = K.quant_mxfp8_batched(w_gu.detach(), rowwise=True, colwise=grad)
            dq, dsf, dtq, dtsf = K.quant_mxfp8_batched(w_down.detach(), rowwise=True, colwise=grad)
        saved = []
        for c in range(chunks):
            xc, ec, wc = x[c * tc:(c + 1) * tc], experts[c * tc:(c + 1) * tc], wts[c * tc:(c + 1) * tc]
            row_index, pos, offsets = sort_picks(ec, e)
            rows = row_index.numel()
            w_row = _row_weights(wc, pos, rows)
            xtq = xtsf = None
            if mx:
                xq, xsf, xtq, xtsf = K.quant_mxfp8(xc, row_index=row_index, rows=rows, colwise=grad)
                h = K.grouped_gemm(xq, gq, offsets, f2, d, kind=kind, asf=xsf, bsf=gsf)
                del xq, xsf
                # the weighted activation is quantised as it is computed: no bf16 copy exists
                aq, asf, _, _ = K.quant_mxfp8_glu(h, None, act, limit=limit, up_offset=up_offset, row_scale=w_row)
                y = K.grouped_gemm(aq, dq, offsets, d, f, kind=kind, asf=asf, bsf=dsf)
                del aq, asf
            else:
                xs = K.gather_rows(xc, row_index, rows)
                h = K.grouped_gemm(xs, w_gu.view(e * f2, d), offsets, f2, d)
                a = K.glu_fwd(h, act, w_row, limit, up_offset)
                y = K.grouped_gemm(a, w_down.view(e * d, f), offsets, d, f)
                del xs, a
            K.combine_rows_into(y, pos, None, out[c * tc:(c + 1) * tc])
            del y
            if grad:
                saved.append((row_index, pos, offsets, w_row, h, xtq, xtsf))
        ctx.save_for_backward(x, w_gu, w_down)
        ctx.chunks_saved = saved
        ctx.wq = (gtq, gtsf, dtq, dtsf) if mx and grad else None
        ctx.cfg = (act, limit, up_offset, mx, tc, weights.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        K = _K()
        x, w_gu, w_down = ctx.saved_tensors
        act, limit, up_offset, mx, tc, w_dtype = ctx.cfg
        saved, ctx.chunks_saved = ctx.chunks_saved, None
        t, d = x.shape
        e, f2, _ = w_gu.shape
        f = f2 // 2
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        dout = dout.contiguous()
        g_gu = getattr(w_gu, "main_grad", None)
        g_down = getattr(w_down, "main_grad", None)
        # the first range's GEMM writes the gradient in the dtype it is kept in; the GEMMs of the
        # ranges after it add into that (the sum is rounded to that dtype after each range)
        acc_gu, acc_down = g_gu, g_down
        if mx:
            gtq, gtsf, dtq, dtsf = ctx.wq
            ctx.wq = None
        dx = torch.empty_like(x)
        dwts = torch.empty(t, saved[0][1].shape[1], dtype=torch.float32, device=x.device)
        dw_gu = dw_down = None
        for c, (row_index, pos, offsets, w_row, h, xtq, xtsf) in enumerate(saved):
            saved[c] = None
            rows = row_index.numel()
            dc, xc = dout[c * tc:(c + 1) * tc], x[c * tc:(c + 1) * tc]
            if mx:
                # dy[r] = dout[token(r)]: a row gather inside the quantiser (both orientations)
                dyq, dysf, dytq, dytsf = K.quant_mxfp8(dc, rowwise=True, colwise=True, row_index=row_index, rows=rows)
                # the weighted activation is recomputed inside the quantiser (cheaper than keeping it)
                _, _, atq, atsf = K.quant_mxfp8_glu(h, None, act, rowwise=False, colwise=True, limit=limit,
                                                    up_offset=up_offset, row_scale=w_row)
                # dW_down[e] = dy_e^T · a'_e
                dw_down = K.grouped_gemm_k(dytq, atq, offsets, d, f, kind=kind, asf=dytsf, bsf=atsf, out=acc_down,
                                           accumulate=acc_down is not None, out_dtype=_grad_dtype(w_down))
                acc_down = dw_down
                del dytq, dytsf, atq, atsf
                # da' = dy · W_down (per expert, contraction over d)
                da = K.grouped_gemm(dyq, dtq, offsets, f, d, kind=kind, asf=dysf, bsf=dtsf)
                del dyq, dysf
            else:
                dy = K.gather_rows(dc, row_index, rows)
                a = K.glu_fwd(h, act, w_row, limit, up_offset)
                dw_down = K.grouped_gemm_k(dy, a, offsets, d, f, a_mn=True, b_mn=True, out=acc_down,
                                           accumulate=acc_down is not None, out_dtype=_grad_dtype(w_down))
                acc_down = dw_down
                da = K.grouped_gemm(dy, w_down.view(e * d, f), offsets, f, d, b_mn=True)
                del a, dy
            # dh, and per row <da', glu(h)> = the gradient of that row's router weight
            dh, drs = K.glu_bwd(h, da, act, w_row, limit, up_offset)
            del da, h
            dwts[c * tc:(c + 1) * tc] = drs[pos.reshape(-1).long()].view(pos.shape)
            if mx:
                hq, hsf, htq, htsf = K.quant_mxfp8(dh, rowwise=True, colwise=True)
                del dh
                dw_gu = K.grouped_gemm_k(htq, xtq, offsets, f2, d, kind=kind, asf=htsf, bsf=xtsf, out=acc_gu,
                                         accumulate=acc_gu is not None, out_dtype=_grad_dtype(w_gu))
                acc_gu = dw_gu
                del htq, htsf, xtq, xtsf
                dxs = K.grouped_gemm(hq, gtq, offsets, d, f2, kind=kind, asf=hsf, bsf=gtsf)
                del hq, hsf
            else:
                xs = K.gather_rows(xc, row_index, rows)
                dw_gu = K.grouped_gemm_k(dh, xs, offsets, f2, d, a_mn=True, b_mn=True, out=acc_gu,
                                         accumulate=acc_gu is not None, out_dtype=_grad_dtype(w_gu))
                acc_gu = dw_gu
                dxs = K.grouped_gemm(dh, w_gu.view(e * f2, d), offsets, d, f2, b_mn=True)
                del xs, dh
            K.combine_rows_into(dxs, pos, None, dx[c * tc:(c + 1) * tc])
            del dxs
        gw_gu = None if g_gu is not None else dw_gu.to(w_gu.dtype)
        gw_down = None if g_down is not None else dw_down.to(w_down.dtype)
        return dx, gw_gu, gw_down, dwts.to(w_dtype), None, None, None, None, None, None


def moe_experts(x, w_gate_up, w_down, weights, experts, *, act: str = "swish",
                limit: Optional[float] = None, up_offset: float = 0.0, fmt: str = "bf16", chunks: int = 1):
    """Routed experts on x [T,d]: out[t] = Σ_j weights[t,j] · expert_{experts[t,j]}(x[t]).
    w_gate_up [E, 2f, d] (gate rows first), w_down [E, d, f]. `chunks` walks the tokens in that
    many equal ranges (``methods(moe_chunks=...)``)."""
    e, f2, d = w_gate_up.shape
    f = f2 // 2
    mx = fmt in ("mxfp8", "mxfp8_2d")
    shapes_ok = d % 128 == 0 and f % 128 == 0 if mx else (d % 8 == 0 and f % 8 == 0)
    if (kernels_on(x) and shapes_ok and act in ("swish", "quick_gelu", "gelu_tanh", "relu2")
            and w_gate_up.dtype == torch.bfloat16):
        return _SortedExperts.apply(x.contiguous(), w_gate_up, w_down, weights, experts, act,
                                    float(limit or 0.0), float(up_offset), mx, int(chunks))
    return moe_reference(x, w_gate_up, w_down, weights, experts, act, limit, up_offset)


def moe_reference(x, w_gate_up, w_down, weights, experts, act="swish", limit=None, up_offset=0.0, row_fn=None,
                  gated: bool = True, up_softcap=None, up_bias=None, down_bias=None):
    """Differentiable plain-PyTorch experts: sort picks, one matmul pair per expert.
    `row_fn` (optional) maps the experts' output rows before the weighted sum (a norm of
    each expert's output). Without `gated` the experts are plain MLPs: `w_gate_up` is the up
    projection alone ([E, f, d]) and the activation applies to it. `up_bias` ([E, 2f] or
    [E, f]) is added to an expert's projection before the activation, `down_bias` ([E, d]) to
    its output before `row_fn` and the weighted sum."""
    t, d = x.shape
    e, f2, _ = w_gate_up.shape
    f = f2 // 2 if gated else f2
    k = experts.shape[1]
    flat = experts.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=e).tolist()
    tok = order // k
    xs = x[tok]
    outs = []
    start = 0
    for ex in range(e):
        n = counts[ex]
        if n == 0:
            continue
        seg = xs[start:start + n]
        h = seg @ w_gate_up[ex].to(seg.dtype).t()
        if up_bias is not None:
            h = h + up_bias[ex].to(h.dtype)
        # experts activate as an MLP does: the up branch clipped to +-limit, then soft-capped; a
        # gate capped from above only
        if gated:
            up = h[:, f:]
            if up_softcap is not None:
                up = up.float().clamp(-limit, limit) if limit is not None else up.float()
                up = (up_softcap * torch.tanh(up / up_softcap)).to(h.dtype)
            a = ref.glu(h[:, :f], up, act, limit, up_offset)
        else:
            up = h.float().clamp(-limit, limit) if limit is not None else h.float()
            if up_softcap is not None:
                up = up_softcap * torch.tanh(up / up_softcap)
            a = ref.activation(up, act).to(h.dtype)
        y = a @ w_down[ex].to(seg.dtype).t()
        outs.append(y if down_bias is None else y + down_bias[ex].to(y.dtype))
        start += n
    ys = torch.cat(outs) if outs else xs.new_zeros(0, d)
    if row_fn is not None and ys.shape[0]:
        ys = row_fn(ys)
    wflat = weights.reshape(-1)[order].unsqueeze(-1)
    out = torch.zeros(t, d, dtype=torch.float32, device=x.device)
    out = out.index_add(0, tok, ys.float() * wflat.float())
    return out.to(x.dtype)


# ------------------------------------------------------------------ experts on rows that are already sorted
class _ExpertsOnSorted(torch.autograd.Function):
    """The expert stack on rows that already sit in expert-sorted, 128-padded order
    (what an expert-parallel rank receives from a library all-to-all):
    y[r] = expert_{group(r)}(xs[r])."""

    @staticmethod
    def forward(ctx, xs, offsets, counts, w_gu, w_down, act, limit, up_offset, mx):
        K = _K()
        rows, d = xs.shape
        e, f2, _ = w_gu.shape
        f = f2 // 2
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        grad = any(ctx.needs_input_grad)
        if counts is not None:
            K.zero_pad_rows(xs, offsets, counts)
        wq = None
        if mx:
            xq, xsf, xtq, xtsf = K.quant_mxfp8(xs, rowwise=True, colwise=grad)
            gq, gsf, gtq, gtsf = K.quant_mxfp8_batched(w_gu.detach(), rowwise=True, colwise=grad)
            dq, dsf, dtq, dtsf = K.quant_mxfp8_batched(w_down.detach(), rowwise=True, colwise=grad)
            h = K.grouped_gemm(xq, gq, offsets, f2, d, kind=kind, asf=xsf, bsf=gsf)
            del xq, xsf, gq, gsf
            aq, asf, _, _ = K.quant_mxfp8_glu(h, None, act, limit=limit, up_offset=up_offset)
            y = K.grouped_gemm(aq, dq, offsets, d, f, kind=kind, asf=asf, bsf=dsf)
            saved_x = (xtq, xtsf)
            wq = (gtq, gtsf, dtq, dtsf)
        else:
            h = K.grouped_gemm(xs, w_gu.view(e * f2, d), offsets, f2, d)
            a = K.glu_fwd(h, act, None, limit, up_offset)
            y = K.grouped_gemm(a, w_down.view(e * d, f), offsets, d, f)
            saved_x = (xs.clone(), None)
        ctx.save_for_backward(saved_x[0], saved_x[1], offsets, counts, w_gu, w_down, h)
        ctx.wq = wq if grad else None
        ctx.cfg = (act, limit, up_offset, mx)
        return y

    @staticmethod
    def backward(ctx, dy):
        K = _K()
        xsave, xtsf, offsets, counts, w_gu, w_down, h = ctx.saved_tensors
        act, limit, up_offset, mx = ctx.cfg
        e, f2, d = w_gu.shape
        f = f2 // 2
        kind = K.KIND_MXFP8 if mx else K.KIND_BF16
        dy = dy.contiguous()
        if counts is not None:
            K.zero_pad_rows(dy, offsets, counts)
        g_gu = getattr(w_gu, "main_grad", None)
        g_down = getattr(w_down, "main_grad", None)
        if mx:
            gtq, gtsf, dtq, dtsf = ctx.wq
            ctx.wq = None
            dyq, dysf, dytq, dytsf = K.quant_mxfp8(dy, rowwise=True, colwise=True)
            _, _, atq, atsf = K.quant_mxfp8_glu(h, None, act, rowwise=False, colwise=True,
                                                limit=limit, up_offset=up_offset)
            dw_down = K.grouped_gemm_k(dytq, atq, offsets, d, f, kind=kind, asf=dytsf, bsf=atsf,
                                       out=g_down, accumulate=g_down is not None,
                                       out_dtype=_grad_dtype(w_down))
            del dytq, dytsf, atq, atsf
            da = K.grouped_gemm(dyq, dtq, offsets, f, d, kind=kind, asf=dysf, bsf=dtsf)
            del dyq, dysf
            dh, _ = K.glu_bwd(h, da, act, None, limit, up_offset)
            del da
            hq, hsf, htq, htsf = K.quant_mxfp8(dh, rowwise=True, colwise=True)
            del dh
            dw_gu = K.grouped_gemm_k(htq, xsave, offsets, f2, d, kind=kind, asf=htsf, bsf=xtsf,
                                     out=g_gu, accumulate=g_gu is not None,
                                     out_dtype=_grad_dtype(w_gu))
            del htq, htsf
            dxs = K.grouped_gemm(hq, gtq, offsets, d, f2, kind=kind, asf=hsf, bsf=gtsf)
        else:
            a = K.glu_fwd(h, act, None, limit, up_offset)
            dw_down = K.grouped_gemm_k(dy, a, offsets, d, f, a_mn=True, b_mn=True, out=g_down,
                                       accumulate=g_down is not None,
                                       out_dtype=_grad_dtype(w_down))
            da = K.grouped_gemm(dy, w_down.view(e * d, f), offsets, f, d, b_mn=True)
            del a
            dh, _ = K.glu_bwd(h, da, act, None, limit, up_offset)
            del da
            dw_gu = K.grouped_gemm_k(dh, xsave, offsets, f2, d, a_mn=True, b_mn=True, out=g_gu,
                                     accumulate=g_gu is not None,
                                     out_dtype=_grad_dtype(w_gu))
            dxs = K.grouped_gemm(dh, w_gu.view(e * f2, d), offsets, d, f2, b_mn=True)
        gw_gu = None if g_gu is not None else dw_gu.to(w_gu.dtype)
        gw_down = None if g_down is not None else dw_down.to(w_down.dtype)
        return dxs, None, None, gw_gu, gw_down, None, None, None, None


def experts_on_sorted(xs, offsets, counts, w_gate_up, w_down, *, act="swish", limit=None,
                      up_offset=0.0, fmt="bf16"):
    """Expert stack over pre-sorted rows; see `_ExpertsOnSorted`. Falls back to plain
    PyTorch (per-group matmuls) off the GPU."""
    mx = fmt in ("mxfp8", "mxfp8_2d")
    if kernels_on(xs):
        return _ExpertsOnSorted.apply(xs.contiguous(), offsets, counts, w_gate_up, w_down, act,
                                      float(limit or 0.0), float(up_offset), mx)
    f = w_gate_up.shape[1] // 2
    off = offsets.tolist()
    cnt = counts.tolist() if counts is not None else [off[g + 1] - off[g] for g in range(len(off) - 1)]
    parts, at = [], 0
    for g in range(len(off) - 1):
        if off[g] > at:
            parts.append(xs.new_zeros(off[g] - at, w_down.shape[1]))
        seg = xs[off[g]: off[g] + cnt[g]]
        hh = seg @ w_gate_up[g].to(seg.dtype).t()
        aa = ref.glu(hh[:, :f], hh[:, f:], act, limit, up_offset)
        parts.append(aa @ w_down[g].to(seg.dtype).t())
        at = off[g] + cnt[g]
    if xs.shape[0] > at:
        parts.append(xs.new_zeros(xs.shape[0] - at, w_down.shape[1]))
    return torch.cat(parts)
