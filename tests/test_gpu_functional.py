"""Differentiable CUDA ops (kernels behind autograd) against plain PyTorch in fp32."""
import pytest
import torch

from bux_b200 import ops
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


@pytest.mark.parametrize("fmt,tol", [("bf16", 2e-2), ("mxfp8", 8e-2)])
def test_linear(cuda, fmt, tol):
    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device=cuda).bfloat16().requires_grad_()
    w = (torch.randn(384, 256, device=cuda) * 0.05).bfloat16().requires_grad_()
    y = ops.linear(x, w, fmt=fmt)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    assert rel_err(y, yr) < tol
    assert rel_err(x.grad, xr.grad) < tol
    assert rel_err(w.grad, wr.grad) < tol


@pytest.mark.parametrize("passes", [("fprop",), ("dgrad", "wgrad"), ("fprop", "wgrad"), ("dgrad",)])
def test_linear_mxfp8_in_some_passes_only(cuda, passes):
    """The GEMMs that `passes` lists multiply in MXFP8, the others exactly as the bf16 linear does."""
    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device=cuda).bfloat16()
    w = (torch.randn(384, 256, device=cuda) * 0.05).bfloat16()
    dy = torch.randn(4, 96, 384, device=cuda).bfloat16()

    def run(fmt, only):
        xi, wi = x.clone().requires_grad_(), w.clone().requires_grad_()
        y = ops.linear(xi, wi, fmt=fmt, passes=only)
        y.backward(dy)
        return {"fprop": y.detach(), "dgrad": xi.grad, "wgrad": wi.grad}

    plain = run("bf16", ("fprop", "dgrad", "wgrad"))
    low = run("mxfp8", ("fprop", "dgrad", "wgrad"))
    got = run("mxfp8", passes)
    for name in ("fprop", "dgrad", "wgrad"):
        want = low if name in passes else plain
        assert torch.equal(got[name], want[name]), name
        assert rel_err(got[name], plain[name]) < 8e-2


def test_cross_entropy_head(cuda):
    torch.manual_seed(1)
    x = torch.randn(300, 128, device=cuda).bfloat16().requires_grad_()
    w = (torch.randn(1000, 128, device=cuda) * 0.1).bfloat16().requires_grad_()
    tgt = torch.randint(0, 1000, (300,), device=cuda)
    mask = (torch.rand(300, device=cuda) > 0.1).float()
    total, count = ops.cross_entropy_head(x, w, tgt, mask, z_weight=1e-4)
    (total / count).backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    tr, cr = ref.cross_entropy(xr @ wr.t(), tgt, mask, 1e-4)
    (tr / cr).backward()
    assert abs(total.item() - tr.item()) / tr.item() < 5e-3
    assert rel_err(x.grad, xr.grad) < 3e-2
    assert rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("fmt,tol", [("bf16", 3e-2), ("mxfp8", 1e-1)])
def test_moe_experts(cuda, fmt, tol):
    torch.manual_seed(2)
    t, d, f, e, k = 512, 256, 128, 8, 2
    x = torch.randn(t, d, device=cuda).bfloat16().requires_grad_()
    wgu = (torch.randn(e, 2 * f, d, device=cuda) * 0.06).bfloat16().requires_grad_()
    wd = (torch.randn(e, d, f, device=cuda) * 0.06).bfloat16().requires_grad_()
    logits = torch.randn(t, e, device=cuda)
    logits[:, 3] = -100.0  # an expert nobody picks
    wts, idx, _ = ref.router_topk(logits, k)
    wts = wts.requires_grad_()
    out = ops.moe_experts(x, wgu, wd, wts, idx, fmt=fmt)
    dout = torch.randn_like(out)
    out.backward(dout)
    xr = x.detach().float().requires_grad_()
    gr = wgu.detach().float().requires_grad_()
    dr = wd.detach().float().requires_grad_()
    wr = wts.detach().clone().requires_grad_()
    want = ops.moe_reference(xr, gr, dr, wr, idx)
    want.backward(dout.float())
    assert rel_err(out, want) < tol
    assert rel_err(x.grad, xr.grad) < tol
    assert rel_err(wgu.grad, gr.grad) < tol
    assert rel_err(wd.grad, dr.grad) < tol
    assert rel_err(wts.grad, wr.grad) < tol


def test_norm_glu_attention_autograd(cuda):
    torch.manual_seed(3)
    x = torch.randn(2, 64, 256, device=cuda).bfloat16().requires_grad_()
    w = torch.ones(256, device=cuda).requires_grad_()
    y = ops.rmsnorm(x, w, 1e-6)
    h = ops.glu(y.view(2, 64, 256))
    h.sum().backward()
    assert torch.isfinite(x.grad).all() and torch.isfinite(w.grad).all()
    q = torch.randn(1, 256, 4, 64, device=cuda).bfloat16().requires_grad_()
    k = torch.randn(1, 256, 2, 64, device=cuda).bfloat16().requires_grad_()
    v = torch.randn(1, 256, 2, 64, device=cuda).bfloat16().requires_grad_()
    o = ops.attention(q, k, v)
    o.float().square().sum().backward()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf, _ = ref.attention(qr, kr, vr)
    orf.square().sum().backward()
    assert rel_err(q.grad, qr.grad) < 4e-2 and rel_err(k.grad, kr.grad) < 4e-2


@pytest.mark.gpu
def test_linear_f32_matches_fp32_matmul():
    from bux_b200.ops import functional as F_

    torch.manual_seed(0)
    x = torch.randn(512, 256, device="cuda").bfloat16().requires_grad_(True)
    for dtype in (torch.float32, torch.bfloat16):
        w = (torch.randn(128, 256, device="cuda") * 0.05).to(dtype).requires_grad_(True)
        y = F_.linear_f32(x, w)
        want = x.float() @ w.float().t()
        assert y.dtype == torch.float32
        assert torch.allclose(y, want, atol=2e-4 if dtype == torch.float32 else 1e-5, rtol=1e-4)
        g = torch.randn_like(y)
        dx, dw = torch.autograd.grad(y, (x, w), g)
        gb = g.bfloat16().float()
        assert torch.allclose(dx.float(), (gb @ w.float()), atol=2e-2, rtol=2e-2)
        assert torch.allclose(dw.float(), gb.t() @ x.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_remat_that_keeps_attention_outputs_matches_plain_remat():
    from bux_b200.lang import compile_runs
    from bux_b200.ops import kernels as K
    from bux_b200.train.trainer import Trainer

    src = """
d_model=256
vocab_size=512
n = rmsnorm
block = [n gqa(num_heads=4, num_kv_heads=2, head_dim=64, rope=rope())] [n gated_mlp(intermediate_size=512, activation=swish)]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-3)
seq_len = 256
batch = 4
steps = 4
precision = precision(compute=bfloat16)
"""
    run = compile_runs(src, filename="k.bux")[0]
    out = []
    for keep, offload in ((False, False), (True, False), (1, True)):
        tr = Trainer(run, device="cuda")
        tr.model.set_remat(True, offload=offload, keep_attention=keep)
        feed = iter(tr.batches())
        before = K.launches
        losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
        out.append((losses, K.launches - before, {n: p.detach().float().clone() for n, p in tr.model.named_parameters()}))
    (l0, n0, s0), (l1, n1, s1), (l2, n2, s2) = out
    assert l0 == pytest.approx(l1, abs=1e-3) and l0 == pytest.approx(l2, abs=1e-3)
    assert n1 == n0 - 2 * 2              # one attention forward less per block and step
    assert n2 == n0 - 2 * 1              # a count keeps the last so many blocks only (inputs on the host)
    assert all(torch.allclose(s0[k], s2[k], atol=2e-3, rtol=2e-2) for k in s0)
    # dQ is summed by fp32 reductions whose order varies from run to run: close, not bit-equal
    assert all(torch.allclose(s0[k], s1[k], atol=2e-3, rtol=2e-2) for k in s0)


@pytest.mark.parametrize("shape", [(512, 2048), (2048, 768), (3, 256, 512)])
def test_newton_schulz_on_the_tcgen05_gemm_matches_fp32(shape):
    """Muon's orthogonalisation through the framework's GEMM against the same iteration in
    fp32 PyTorch; the result is close to an orthogonal factor (singular values near 1)."""
    from bux_b200.ops import kernels as K
    from bux_b200.train import optim

    torch.manual_seed(0)
    g = torch.randn(*shape, device="cuda")
    before = K.launches
    got = optim.newton_schulz(g, steps=5, dtype=torch.bfloat16).float()
    want = optim.newton_schulz(g, steps=5, dtype=torch.float32)
    assert got.shape == want.shape
    assert (got - want).norm() / want.norm() < 0.06
    s = torch.linalg.svdvals(got.reshape(-1, *shape[-2:])[0])
    assert 0.5 < s.min() and s.max() < 1.3
    assert K.launches >= before + 15  # three GEMMs per step, per matrix


def test_interleaved_microbatches_match_a_plain_accumulation_on_two_streams(cuda):
    """``methods(interleave=true)`` on the GPU: every microbatch's forward is issued on one of two
    streams by its parity, beside the backward of the one before on the other. A mixture of
    experts, a value residual that crosses blocks and ``remat=full``: the parameters after two
    steps are those of the microbatches run one after another."""
    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    src = """
d_model=256
vocab_size=512
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, head_dim=64, rope=rope(), value_residual=learned)
e = moe(num_experts=8, top_k=2, expert=gated_mlp(intermediate_size=128, activation=swish))
first = [n a(v=@v)] [n e]
rest = [n a(v=$v)] [n e]
model = embed first rest^3 n head
data = synthetic
optimizer = adamw(lr=1e-3, eps=1.0)
seq_len = 256
batch = 8
steps = 4
precision = precision(compute=bfloat16)
methods = methods(microbatches=4, remat=full{more})
"""
    out = {}
    for name, more in (("plain", ""), ("interleaved", ", interleave=true")):
        tr = Trainer(compile_runs(src.format(more=more), filename="g.bux")[0], device=cuda)
        feed = iter(tr.batches())
        losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
        torch.cuda.synchronize()
        out[name] = (losses, {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}, tr._interleave)
    assert out["interleaved"][2] and out["interleaved"][2].ticks == 2 * 3 * 6      # two steps, three pairs, six pieces
    assert out["plain"][0] == pytest.approx(out["interleaved"][0], abs=1e-3)
    for name, p in out["plain"][1].items():
        assert rel_err(out["interleaved"][1][name], p) < 1e-3, name
