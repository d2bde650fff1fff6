"""Every CUDA kernel against the plain PyTorch fp32 statement of the same op."""
import pytest
import torch

from bux_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _status(cuda):
    from bux_b200.ops import kernels as K

    yield
    torch.cuda.synchronize()
    K.check_status(cuda)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k,bn", [(256, 512, 256, 256), (304, 264, 200, 128), (1024, 768, 2048, 256)])
def test_gemm_bf16(cuda, a_mn, b_mn, m, n, k, bn):
    from bux_b200.ops import kernels as K

    torch.manual_seed(0)
    a = torch.randn(m, k, device=cuda).bfloat16()
    b = torch.randn(n, k, device=cuda).bfloat16()
    want = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    got = K.gemm_bf16(a_in, b_in, a_mn=a_mn, b_mn=b_mn, bn=bn)
    assert rel_err(got, want) < 1e-2
    acc = torch.ones(m, n, device=cuda)
    K.gemm_bf16(a_in, b_in, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True, bn=bn)
    assert rel_err(acc, want + 1) < 1e-2


def test_quant_mxfp8_matches_reference(cuda):
    from bux_b200.ops import kernels as K

    torch.manual_seed(1)
    x = (torch.randn(200, 384, device=cuda) * torch.logspace(-3, 3, 384, device=cuda)).bfloat16()
    q_row, sf_row, q_col, sf_col = K.quant_mxfp8(x, rowwise=True, colwise=True)
    rq, re = ref.quant_mxfp8(x)
    assert torch.equal(ref.unswizzle_scales(sf_row, 200, 12), re)
    assert torch.equal(q_row.view(torch.uint8), rq.view(torch.uint8))
    xt = torch.zeros(384, 256, device=cuda, dtype=torch.bfloat16)
    xt[:, :200] = x.t()
    tq, te = ref.quant_mxfp8(xt)
    # scale blocks past the last row are never written (they keep the pad byte)
    assert torch.equal(ref.unswizzle_scales(sf_col, 384, 8)[:, :7], te[:, :7])
    assert torch.equal(q_col.view(torch.uint8), tq.view(torch.uint8))


@pytest.mark.parametrize("m,n,k,bn", [(128, 128, 128, 128), (256, 384, 512, 128), (1000, 768, 2048, 128),
                                      (512, 512, 1024, 256)])
def test_gemm_mxfp8(cuda, m, n, k, bn):
    from bux_b200.ops import kernels as K

    torch.manual_seed(2)
    a = torch.randn(m, k, device=cuda).bfloat16()
    b = torch.randn(n, k, device=cuda).bfloat16()
    aq, asf, _, _ = K.quant_mxfp8(a)
    bq, bsf, _, _ = K.quant_mxfp8(b)
    want = ref.gemm_mxfp8(*ref.quant_mxfp8(a), *ref.quant_mxfp8(b))
    got = K.gemm_mxfp8(aq, asf, bq, bsf, m, n, k, bn=bn)
    assert rel_err(got, want) < 1e-2


@pytest.mark.parametrize("kind", ["bf16", "mxfp8"])
def test_grouped_gemm_rows(cuda, kind):
    from bux_b200.ops import kernels as K

    torch.manual_seed(3)
    counts = [128, 0, 384, 256]
    n, k = 256, 512
    offsets = torch.tensor([0, *torch.tensor(counts).cumsum(0).tolist()], dtype=torch.int32, device=cuda)
    rows = sum(counts)
    a = torch.randn(rows, k, device=cuda).bfloat16()
    w = torch.randn(len(counts), n, k, device=cuda).bfloat16()
    want = torch.cat([a[offsets[g]:offsets[g + 1]].float() @ w[g].float().t() for g in range(len(counts))])
    if kind == "bf16":
        got = K.grouped_gemm(a, w.view(-1, k), offsets, n, k)
        tol = 1e-2
    else:
        aq, asf, _, _ = K.quant_mxfp8(a)
        wq, wsf, _, _ = K.quant_mxfp8(w.view(-1, k))
        got = K.grouped_gemm(aq, wq, offsets, n, k, kind=K.KIND_MXFP8, asf=asf, bsf=wsf)
        tol = 6e-2
    assert rel_err(got, want) < tol


def test_grouped_gemm_contraction(cuda):
    from bux_b200.ops import kernels as K

    torch.manual_seed(4)
    counts = [128, 0, 256]
    m, n = 256, 128
    offsets = torch.tensor([0, *torch.tensor(counts).cumsum(0).tolist()], dtype=torch.int32, device=cuda)
    rows = sum(counts)
    dy = torch.randn(rows, m, device=cuda).bfloat16()
    x = torch.randn(rows, n, device=cuda).bfloat16()
    want = torch.stack([dy[offsets[g]:offsets[g + 1]].float().t() @ x[offsets[g]:offsets[g + 1]].float()
                        for g in range(len(counts))])
    got = K.grouped_gemm_k(dy, x, offsets, m, n, a_mn=True, b_mn=True)
    assert rel_err(got, want) < 1e-2
    # gradients kept in bf16: written by one call, added to by the next (the chunks of a step)
    first = K.grouped_gemm_k(dy, x, offsets, m, n, a_mn=True, b_mn=True, out_dtype=torch.bfloat16)
    assert first.dtype == torch.bfloat16 and rel_err(first, want) < 1e-2
    again = K.grouped_gemm_k(dy, x, offsets, m, n, a_mn=True, b_mn=True, out=first, accumulate=True)
    assert again is first and rel_err(first, 2 * want) < 1e-2
    assert first[1].abs().max() == 0   # the empty group stays zero


def test_rmsnorm(cuda):
    from bux_b200.ops import kernels as K

    torch.manual_seed(5)
    x = torch.randn(300, 512, device=cuda).bfloat16().requires_grad_()
    w = torch.randn(512, device=cuda).requires_grad_()
    y, rstd = K.rmsnorm_fwd(x.detach(), w.detach(), 1e-6)
    want = ref.rmsnorm(x, w, 1e-6)
    assert rel_err(y, want) < 1e-2
    dy = torch.randn_like(want)
    want.backward(dy)
    dx, dw = K.rmsnorm_bwd(x.detach(), w.detach(), dy, rstd)
    assert rel_err(dx, x.grad) < 2e-2
    assert rel_err(dw, w.grad) < 2e-2


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("norm", [True, False])
def test_norm_rope(cuda, d, norm):
    from bux_b200.ops import kernels as K

    torch.manual_seed(6)
    x = torch.randn(2, 50, 4, d, device=cuda).bfloat16().requires_grad_()
    w = torch.randn(d, device=cuda).requires_grad_() if norm else None
    pos = torch.arange(50, device=cuda).repeat(2, 1)
    cos, sin = ref.rope_tables(pos, d, 10000.0)
    want = ref.rmsnorm_rope(x, w, cos, sin, 1e-6) if norm else ref.rope(x, cos, sin)
    c2, s2 = cos.reshape(-1, d // 2).contiguous(), sin.reshape(-1, d // 2).contiguous()
    y, rstd = K.norm_rope_fwd(x.detach(), None if w is None else w.detach(), c2, s2, 1e-6)
    assert rel_err(y, want) < 1e-2
    dy = torch.randn_like(want)
    want.backward(dy)
    dx, dw = K.norm_rope_bwd(x.detach(), None if w is None else w.detach(), c2, s2, rstd, dy, 1e-6)
    assert rel_err(dx, x.grad) < 2e-2
    if norm:
        assert rel_err(dw, w.grad) < 2e-2


@pytest.mark.parametrize("kind,limit,off", [("swish", 0.0, 0.0), ("quick_gelu", 7.0, 1.0)])
def test_glu(cuda, kind, limit, off):
    from bux_b200.ops import kernels as K

    torch.manual_seed(7)
    h = (torch.randn(100, 256, device=cuda) * 4).bfloat16().requires_grad_()
    rs = torch.rand(100, device=cuda).requires_grad_()
    want = ref.glu(h[:, :128], h[:, 128:], kind, limit or None, off).float() * rs[:, None]
    got = K.glu_fwd(h.detach(), kind, rs.detach(), limit, off)
    assert rel_err(got, want) < 1e-2
    dout = torch.randn(100, 128, device=cuda).bfloat16()
    want.backward(dout.float())
    dh, drs = K.glu_bwd(h.detach(), dout, kind, rs.detach(), limit, off)
    assert rel_err(dh, h.grad) < 2e-2
    assert rel_err(drs, rs.grad) < 2e-2


def test_cross_entropy(cuda):
    from bux_b200.ops import kernels as K

    torch.manual_seed(8)
    logits = (torch.randn(64, 1000, device=cuda) * 3).bfloat16()
    tgt = torch.randint(0, 1000, (64,), device=cuda, dtype=torch.int32)
    mask = (torch.rand(64, device=cuda) > 0.2).float()
    lf = logits.float().requires_grad_()
    total, count = ref.cross_entropy(lf, tgt, mask, z_weight=1e-4)
    (total / count).backward()
    work = logits.clone()
    loss = K.ce_fwd_bwd(work, tgt, mask, 1.0 / count.item(), z_weight=1e-4)
    assert abs(loss.sum().item() - total.item()) / total.item() < 1e-3
    assert rel_err(work, lf.grad) < 2e-2


@pytest.mark.parametrize("mom", ["f32", "bf16", "fp8"])
def test_adamw(cuda, mom):
    from bux_b200.ops import kernels as K

    torch.manual_seed(9)
    n = 5000
    p = torch.randn(n, device=cuda)
    g = torch.randn(n, device=cuda).bfloat16()
    rp, rm, rv = p.clone(), torch.zeros(n, device=cuda), torch.zeros(n, device=cuda)
    if mom == "fp8":
        m = torch.zeros(n, dtype=torch.uint8, device=cuda)
        v = torch.zeros(n, dtype=torch.uint8, device=cuda)
        msf = torch.ones((n + 31) // 32, dtype=torch.uint8, device=cuda)
        vsf = torch.ones((n + 31) // 32, dtype=torch.uint8, device=cuda)
    else:
        dt = torch.float32 if mom == "f32" else torch.bfloat16
        m, v, msf, vsf = torch.zeros(n, dtype=dt, device=cuda), torch.zeros(n, dtype=dt, device=cuda), None, None
    shadow = torch.empty(n, dtype=torch.bfloat16, device=cuda)
    for step in (1, 2, 3):
        K.adamw(p, g, m, v, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, step=step, m_sf=msf, v_sf=vsf,
                shadow=shadow)
        ref.adamw_step(rp, g, rm, rv, lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, step=step)
    tol = {"f32": 1e-5, "bf16": 2e-3, "fp8": 2e-2}[mom]
    assert rel_err(p, rp) < tol
    assert rel_err(shadow, rp) < 1e-2


def test_gather_combine(cuda):
    from bux_b200.ops import kernels as K

    torch.manual_seed(10)
    x = torch.randn(40, 64, device=cuda).bfloat16()
    idx = torch.randint(-1, 40, (100,), device=cuda, dtype=torch.int32)
    got = K.gather_rows(x, idx, 100)
    want = torch.where(idx[:, None] >= 0, x[idx.clamp_min(0).long()], torch.zeros_like(x[:1]))
    assert torch.equal(got, want)
    pos = torch.randint(-1, 100, (30, 4), device=cuda, dtype=torch.int32)
    w = torch.rand(30, 4, device=cuda)
    out = K.combine_rows(got, pos, w, 30)
    gathered = torch.where(pos[..., None] >= 0, got[pos.clamp_min(0).long()].float(), torch.zeros(1, device=cuda))
    assert rel_err(out, (gathered * w[..., None]).sum(1)) < 1e-2


@pytest.mark.parametrize("d,h,g", [(128, 4, 2), (64, 8, 2)])
@pytest.mark.parametrize("t,window,sinks", [(256, 0, False), (300, 0, False), (384, 128, True)])
def test_attention_fwd(cuda, d, h, g, t, window, sinks):
    from bux_b200.ops import kernels as K

    torch.manual_seed(11)
    q = torch.randn(2, t, h, d, device=cuda).bfloat16()
    k = torch.randn(2, t, g, d, device=cuda).bfloat16()
    v = torch.randn(2, t, g, d, device=cuda).bfloat16()
    sk = torch.randn(h, device=cuda) if sinks else None
    want, want_lse = ref.attention(q, k, v, causal=True, window=window or None, sinks=sk)
    got, lse = K.attn_fwd(q, k, v, causal=True, window=window, sinks=sk)
    assert rel_err(got, want) < 2e-2
    assert rel_err(lse, want_lse) < 1e-3


@pytest.mark.parametrize("d,h,g", [(128, 4, 2), (64, 4, 1)])
@pytest.mark.parametrize("t,window,sinks", [(256, 0, False), (300, 0, False), (384, 128, True)])
def test_attention_bwd(cuda, d, h, g, t, window, sinks):
    from bux_b200.ops import kernels as K

    torch.manual_seed(12)
    q = torch.randn(2, t, h, d, device=cuda).bfloat16().requires_grad_()
    k = torch.randn(2, t, g, d, device=cuda).bfloat16().requires_grad_()
    v = torch.randn(2, t, g, d, device=cuda).bfloat16().requires_grad_()
    sk = torch.randn(h, device=cuda).requires_grad_() if sinks else None
    want, _ = ref.attention(q, k, v, causal=True, window=window or None, sinks=sk)
    do = torch.randn_like(q)
    want.backward(do)
    with torch.no_grad():
        o, lse = K.attn_fwd(q, k, v, causal=True, window=window, sinks=sk)
        dq, dk, dv, dsk = K.attn_bwd(q, k, v, o, do, lse, causal=True, window=window, sinks=sk)
    assert rel_err(dv, v.grad) < 3e-2
    assert rel_err(dk, k.grad) < 3e-2
    assert rel_err(dq, q.grad) < 3e-2
    if sinks:
        assert rel_err(dsk, sk.grad) < 3e-2


def _documents(t: int, lens, device):
    """Document ids [1, t] of a row packed with documents of the given lengths."""
    assert sum(lens) == t
    ids = torch.cat([torch.full((n,), i + 1) for i, n in enumerate(lens)])
    return ids[None].to(device)


@pytest.mark.parametrize("t,h,g,lens,window,sinks", [
    (4096, 8, 1, None, 0, False),                                             # the benchmark's shape: 8 heads per group
    (4096, 8, 1, [700, 130, 1, 255, 1000, 58, 512, 384, 999, 57], 0, False),  # ten documents, odd boundaries
    (1024, 4, 2, [300, 212, 128, 384], 256, True),                            # documents + window + sinks
    (2048, 4, 2, None, 512, False),                                           # a window far from the diagonal's tile
])
def test_attention_long_rows_documents(cuda, t, h, g, lens, window, sinks):
    """Forward and backward at the lengths the benchmark runs, with packed documents
    (every query sees only its own document), against the fp32 statement."""
    from bux_b200.ops import kernels as K

    torch.manual_seed(13)
    d = 128
    q = torch.randn(1, t, h, d, device=cuda).bfloat16().requires_grad_()
    k = torch.randn(1, t, g, d, device=cuda).bfloat16().requires_grad_()
    v = torch.randn(1, t, g, d, device=cuda).bfloat16().requires_grad_()
    sk = torch.randn(h, device=cuda).requires_grad_() if sinks else None
    seg = _documents(t, lens, cuda) if lens else None
    want, want_lse = ref.attention(q, k, v, causal=True, window=window or None, sinks=sk, segments=seg)
    do = torch.randn_like(q)
    want.backward(do)
    row_lo, key_hi = K.document_bounds(seg) if seg is not None else (None, None)
    if seg is not None:
        assert row_lo[0, 0] == 0 and key_hi[0, 0] == lens[0] - 1 and row_lo[0, -1] == t - lens[-1]
    with torch.no_grad():
        o, lse = K.attn_fwd(q, k, v, causal=True, window=window, sinks=sk, row_lo=row_lo)
        dq, dk, dv, dsk = K.attn_bwd(q, k, v, o, do, lse, causal=True, window=window, sinks=sk,
                                     row_lo=row_lo, key_hi=key_hi)
    assert rel_err(o, want) < 2e-2
    assert rel_err(lse, want_lse) < 1e-3
    assert rel_err(dv, v.grad) < 3e-2
    assert rel_err(dk, k.grad) < 3e-2
    assert rel_err(dq, q.grad) < 3e-2
    if sinks:
        assert rel_err(dsk, sk.grad) < 3e-2


def test_attention_layer_takes_the_kernels_for_packed_rows(cuda):
    """`functional.attention` with segments runs the kernels (not the quadratic statement)."""
    from bux_b200.ops import functional as OF
    from bux_b200.ops import kernels as K

    torch.manual_seed(14)
    q = torch.randn(2, 512, 4, 64, device=cuda).bfloat16().requires_grad_()
    k = torch.randn(2, 512, 2, 64, device=cuda).bfloat16().requires_grad_()
    v = torch.randn(2, 512, 2, 64, device=cuda).bfloat16().requires_grad_()
    seg = torch.cat([_documents(512, [100, 156, 256], cuda), _documents(512, [512], cuda)])
    before = K.launches
    out = OF.attention(q, k, v, causal=True, segments=seg)
    out.backward(torch.ones_like(out))
    assert K.launches - before == 3  # forward, delta, backward
    want, _ = ref.attention(q.detach(), k.detach(), v.detach(), causal=True, segments=seg)
    assert rel_err(out, want) < 2e-2


@pytest.mark.parametrize("kind,limit,up_offset", [("swish", 0.0, 0.0), ("quick_gelu", 7.0, 1.0)])
def test_quantiser_that_computes_the_gated_activation_matches_two_passes(kind, limit, up_offset):
    """glu (and its gradient) computed inside the MXFP8 quantiser gives the bytes that the
    separate activation kernel followed by the quantiser gives."""
    from bux_b200.ops import kernels as K

    torch.manual_seed(0)
    rows, f = 1000, 256  # a ragged last row tile
    h = (torch.randn(rows, 2 * f, device="cuda") * 3).bfloat16()
    da = torch.randn(rows, f, device="cuda").bfloat16()
    a = K.glu_fwd(h, kind, None, limit, up_offset)
    want = K.quant_mxfp8(a, rowwise=True, colwise=True)
    got = K.quant_mxfp8_glu(h, None, kind, rowwise=True, colwise=True, limit=limit, up_offset=up_offset)
    for w, g in zip(want, got):
        assert torch.equal(w.view(torch.uint8), g.view(torch.uint8))
    dh, _ = K.glu_bwd(h, da, kind, None, limit, up_offset)
    want = K.quant_mxfp8(dh, rowwise=True, colwise=True)
    got = K.quant_mxfp8_glu(h, da, kind, rowwise=True, colwise=True, limit=limit, up_offset=up_offset)
    for w, g in zip(want, got):
        assert torch.equal(w.view(torch.uint8), g.view(torch.uint8))
    # and against the fp32 statement of the op: the dequantised copy is close to glu(h)
    ref_a = ref.glu(h[:, :f].float(), h[:, f:].float(), kind, limit or None, up_offset)
    aq, asf, _, _ = K.quant_mxfp8_glu(h, None, kind, limit=limit, up_offset=up_offset)
    back = ref.dequant_mxfp8(aq, ref.unswizzle_scales(asf, rows, f // 32))
    assert rel_err(back, ref_a) < 0.04


@pytest.mark.parametrize("n,k", [(128, 8), (32, 4), (200, 6), (512, 32)])
def test_topk_rows_matches_torch(n, k):
    from bux_b200.ops import kernels as K

    torch.manual_seed(0)
    scores = torch.randn(1000, n, device="cuda")
    scores[3, :5] = float("-inf")          # group-limited routing masks entries out
    got = K.topk_rows(scores, k)
    want = scores.topk(k, dim=-1)
    assert torch.equal(scores.gather(-1, got), want.values)   # same values in the same order
    assert torch.equal(got, want.indices)                      # distinct random values: same indices
    ties = torch.zeros(4, n, device="cuda")
    assert torch.equal(K.topk_rows(ties, k), torch.arange(k, device="cuda").expand(4, k))


def test_nvfp4_quantiser_matches_the_recipe(cuda):
    """The CUDA quantiser (hardware E2M1 conversion) writes the bytes the PyTorch statement
    of the recipe packs."""
    from bux_b200.ops import kernels as K
    from bux_b200.ops import nvfp4 as N

    torch.manual_seed(21)
    x = (torch.randn(300, 512, device=cuda) * torch.logspace(-2, 2, 512, device=cuda)).bfloat16()
    packed, scales, ts = K.quant_nvfp4(x)
    want = N.quantize(x.float())
    wp, ws = N.pack(want)
    assert torch.allclose(ts, want.tensor_scale.reshape(1))
    assert torch.equal(scales, ws)
    mism = (packed != wp).float().mean().item()
    assert mism < 1e-3, mism   # ties at a grid midpoint may round differently after the division


@pytest.mark.parametrize("taps,bias,packed", [(4, False, False), (3, True, True), (8, True, False), (1, False, True)])
def test_causal_conv_matches_the_shifted_sums(cuda, taps, bias, packed):
    """The causal depthwise convolution kernels (forward, dx, dw, db) against the PyTorch sum of
    shifted rows in fp32, with and without document starts inside the rows."""
    from bux_b200 import ops

    torch.manual_seed(0)
    b, t, c = 3, 200, 264
    x = torch.randn(b, t, c, device=cuda).bfloat16().requires_grad_()
    w = (torch.randn(c, taps, device=cuda) * 0.5).bfloat16().requires_grad_()
    bb = torch.randn(c, device=cuda).bfloat16().requires_grad_() if bias else None
    pos = None
    if packed:
        pos = torch.arange(t, device=cuda).repeat(b, 1)
        pos[0, 70:] -= 70
        pos[1, 5:] -= 5
        pos[1, 131:] -= 126
    dy = torch.randn(b, t, c, device=cuda).bfloat16()
    y = ops.causal_conv(x, w, bb, pos)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    br = bb.detach().float().requires_grad_() if bias else None
    yr = xr * wr[:, 0]
    for j in range(1, taps):
        shifted = torch.nn.functional.pad(xr[:, : t - j], (0, 0, j, 0))
        if pos is not None:
            shifted = shifted * (pos >= j).unsqueeze(-1).float()
        yr = yr + shifted * wr[:, j]
    if bias:
        yr = yr + br
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xr.grad) < 1e-2
    assert rel_err(w.grad, wr.grad) < 1e-2
    if bias:
        assert rel_err(bb.grad, br.grad) < 1e-2
