"""The sanitizer-free kernel checks: guard regions around outputs, ragged group edges,
run-twice determinism."""
import pytest
import torch

from bux_b200.ops import checks
from bux_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture
def guarded(cuda):
    was = checks.enabled()
    checks.enable(True)
    yield cuda
    checks.enable(was)


def test_guard_regions_hold_after_every_kernel_family(guarded):
    """Each kernel writes between its guards: odd sizes included, where a tile overhangs."""
    from bux_b200.ops import kernels as K

    dev = guarded
    torch.manual_seed(0)
    a = torch.randn(304, 200, device=dev).bfloat16()
    b = torch.randn(264, 200, device=dev).bfloat16()
    K.gemm_bf16(a, b, bn=128)
    x = torch.randn(200, 384, device=dev).bfloat16()
    q_row, sf_row, q_col, sf_col = K.quant_mxfp8(x, rowwise=True, colwise=True)
    K.requant_mxfp8_cols(q_row, sf_row, 200, 384)
    w = torch.randn(384, device=dev)
    y, rstd = K.rmsnorm_fwd(x, w, 1e-6)
    K.rmsnorm_bwd(x, w, y, rstd)
    h = torch.randn(130, 512, device=dev).bfloat16()
    rs = torch.rand(130, device=dev)
    K.glu_fwd(h, "swish", rs)
    K.glu_bwd(h, torch.randn(130, 256, device=dev).bfloat16(), "swish", rs)
    K.quant_mxfp8_glu(h, None, "swish", rowwise=True, colwise=True, row_scale=rs)
    qq = torch.randn(2, 300, 4, 128, device=dev).bfloat16()
    kk = torch.randn(2, 300, 2, 128, device=dev).bfloat16()
    vv = torch.randn(2, 300, 2, 128, device=dev).bfloat16()
    o, lse = K.attn_fwd(qq, kk, vv, causal=True)
    K.attn_bwd(qq, kk, vv, o, torch.randn_like(qq), lse, causal=True)
    K.topk_rows(torch.randn(77, 128, device=dev), 8)
    logits = torch.randn(37, 1000, device=dev).bfloat16()
    K.ce_fwd_bwd(logits, torch.randint(0, 1000, (37,), device=dev, dtype=torch.int32), None, 1.0)
    torch.cuda.synchronize()
    K.check_status(dev)
    checks.verify()


def test_verify_names_the_op_whose_guard_was_overwritten(guarded):
    """A write past an output's end lands in its guard and is reported with the op's name.
    (The stray write is made by a host-side copy through a longer view, not by a kernel.)"""
    out = checks.guarded_empty((16, 8), torch.float32, guarded, "made_up_op")
    longer = out.as_strided((16 * 8 + 4,), (1,))
    longer[-4:] = 1.0
    torch.cuda.synchronize()
    with pytest.raises(AssertionError, match="made_up_op: 16 bytes after"):
        checks.verify()
    checks.verify()  # cleared


@pytest.mark.parametrize("kind", ["bf16", "mxfp8"])
def test_grouped_gemm_ragged_group_edges(guarded, kind):
    """Groups of 0, 1, 127, 128 and 129 real rows (each padded to 128) against fp32."""
    from bux_b200.ops import kernels as K

    dev = guarded
    torch.manual_seed(1)
    counts = [0, 1, 127, 128, 129, 0, 5]
    padded = [-(-c // 128) * 128 for c in counts]
    offsets = torch.tensor([0] + list(torch.tensor(padded).cumsum(0)), dtype=torch.int32, device=dev)
    rows, k, n = int(offsets[-1]), 256, 384
    x = torch.zeros(rows, k, device=dev)
    for g, c in enumerate(counts):
        x[int(offsets[g]): int(offsets[g]) + c] = torch.randn(c, k, device=dev)
    x = x.bfloat16()
    w = (torch.randn(len(counts), n, k, device=dev) * 0.1).bfloat16()
    want = torch.zeros(rows, n, device=dev)
    for g in range(len(counts)):
        s, e = int(offsets[g]), int(offsets[g + 1])
        want[s:e] = x[s:e].float() @ w[g].float().t()
    if kind == "bf16":
        got = K.grouped_gemm(x, w.view(-1, k), offsets, n, k)
        tol = 1e-2
    else:
        xq, xsf, _, _ = K.quant_mxfp8(x, rowwise=True)
        wq, wsf, _, _ = K.quant_mxfp8_batched(w, rowwise=True)
        got = K.grouped_gemm(xq, wq, offsets, n, k, kind=K.KIND_MXFP8, asf=xsf, bsf=wsf)
        tol = 5e-2
    torch.cuda.synchronize()
    K.check_status(dev)
    checks.verify()
    assert rel_err(got, want) < tol
    # the weight-gradient form over the same ragged groups
    dy = torch.randn(rows, n, device=dev).bfloat16()
    want_dw = torch.stack([dy[int(offsets[g]):int(offsets[g + 1])].float().t() @ x[int(offsets[g]):int(offsets[g + 1])].float()
                           for g in range(len(counts))])
    got_dw = K.grouped_gemm_k(dy, x, offsets, n, k, a_mn=True, b_mn=True)
    torch.cuda.synchronize()
    checks.verify()
    live = [g for g, c in enumerate(counts) if c > 0]
    assert rel_err(got_dw[live], want_dw[live]) < 1e-2
    empty = [g for g, c in enumerate(counts) if c == 0]
    assert got_dw[empty].abs().max() == 0


def test_kernels_give_the_same_bits_twice(cuda):
    """Run-twice determinism of the kernels whose outputs are written without atomics."""
    from bux_b200.ops import kernels as K

    torch.manual_seed(2)
    q = torch.randn(2, 640, 8, 128, device=cuda).bfloat16()
    k = torch.randn(2, 640, 2, 128, device=cuda).bfloat16()
    v = torch.randn(2, 640, 2, 128, device=cuda).bfloat16()
    do = torch.randn_like(q)
    x = torch.randn(1000, 512, device=cuda).bfloat16()
    w = torch.randn(768, 512, device=cuda).bfloat16()

    def run():
        o, lse = K.attn_fwd(q, k, v, causal=True)
        dq, dk, dv, _ = K.attn_bwd(q, k, v, o, do, lse, causal=True)
        xq, xsf, xtq, xtsf = K.quant_mxfp8(x, rowwise=True, colwise=True)
        wq, wsf, _, _ = K.quant_mxfp8(w, rowwise=True)
        return {"o": o, "lse": lse, "dk": dk, "dv": dv, "xq": xq.view(torch.uint8), "xtq": xtq.view(torch.uint8),
                "gemm": K.gemm_bf16(x, w), "gemm_mx": K.gemm_mxfp8(xq, xsf, wq, wsf, 1000, 768, 512)}

    assert checks.same_twice(run) == []
