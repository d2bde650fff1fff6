"""The chunkwise-recurrence kernel against the PyTorch statements of the same recurrence."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _loop(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0):
    """X = P S + W V; O = Qd S + Mqk V + Mqb X; S' = lam S + Kd^T V + Bd^T X, chunk by chunk, fp32."""
    b, h, n = V.shape[:3]
    S = S0.clone() if S0 is not None else torch.zeros(b, h, Qd.shape[-1], V.shape[-1], device=V.device)
    outs = []
    for i in range(n):
        o = Qd[:, :, i] @ S + Mqk[:, :, i] @ V[:, :, i]
        new = lam[:, :, i].unsqueeze(-1) * S + Kd[:, :, i].transpose(-1, -2) @ V[:, :, i]
        if P is not None:
            X = P[:, :, i] @ S + W[:, :, i] @ V[:, :, i]
            o = o + Mqb[:, :, i] @ X
            new = new + Bd[:, :, i].transpose(-1, -2) @ X
        S = new
        outs.append(o)
    return torch.stack(outs, 2), S


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("rank1", [True, False])
@pytest.mark.parametrize("dk,dv,with_state", [(128, 128, False), (64, 128, True), (128, 64, True)])
def test_chunk_scan_matches_the_chunk_loop(cuda, rank1, dk, dv, with_state):
    from bux_b200.ops import scan

    torch.manual_seed(0)
    b, h, n = 2, 3, 5
    dev = "cuda"

    def rnd(*shape, scale=1.0):
        # values a bf16 operand holds exactly, so that the comparison sees the arithmetic only
        return (torch.randn(*shape, device=dev) * scale).bfloat16().float().requires_grad_()

    Qd, Kd, V = rnd(b, h, n, 64, dk, scale=0.3), rnd(b, h, n, 64, dk, scale=0.3), rnd(b, h, n, 64, dv)
    Mqk = rnd(b, h, n, 64, 64, scale=0.2)
    lam = torch.rand(b, h, n, dk, device=dev).mul(0.5).add(0.5).requires_grad_()
    S0 = rnd(b, h, dk, dv, scale=0.5) if with_state else None
    P = W = Mqb = Bd = None
    if rank1:
        P, Bd = rnd(b, h, n, 64, dk, scale=0.1), rnd(b, h, n, 64, dk, scale=0.1)
        W, Mqb = rnd(b, h, n, 64, 64, scale=0.1), rnd(b, h, n, 64, 64, scale=0.2)
    leaves = [t for t in (P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0) if t is not None]
    go, gs = torch.randn(b, h, n, 64, dv, device=dev), torch.randn(b, h, dk, dv, device=dev) * 0.1

    want_o, want_s = _loop(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)
    ((want_o * go).sum() + (want_s * gs).sum()).backward()
    want_g = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    got_o, got_s = scan.chunk_scan(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)
    ((got_o * go).sum() + (got_s * gs).sum()).backward()
    assert _rel(got_o, want_o) < 2e-2 and _rel(got_s, want_s) < 2e-2
    for t, w in zip(leaves, want_g):
        assert _rel(t.grad, w) < 3e-2


@pytest.mark.parametrize("kind", ["gated_delta", "decayed"])
def test_scan_on_the_kernel_matches_the_stepwise_recurrence(cuda, kind):
    """`scan` (bf16 on the GPU: the serial part on the kernel) against one position at a time in fp32."""
    from bux_b200.models.layers import recurrent as R

    torch.manual_seed(1)
    b, t, h, dk, dv = 2, 200, 2, 64, 64
    dev = "cuda"
    q = torch.nn.functional.normalize(torch.randn(b, t, h, dk, device=dev), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(b, t, h, dk, device=dev), dim=-1)
    v = torch.randn(b, t, h, dv, device=dev)
    starts = torch.zeros(b, t, dtype=torch.bool, device=dev)
    starts[:, 0] = True
    starts[0, 77] = True
    if kind == "gated_delta":
        g = -torch.rand(b, t, h, 1, device=dev) * 0.1
        beta = torch.rand(b, t, h, device=dev)
        step = beta.unsqueeze(-1) * k
        args = (q, step, v, g, -g.exp() * k, step)
    else:
        g = -torch.rand(b, t, h, dk, device=dev) * 0.1
        args = (q, k, v, g, None, None)
    want, want_s = R.scan_steps(*[x.cpu() if x is not None else None for x in args], starts.cpu())
    half = [x.bfloat16() if x is not None else None for x in args]
    got, got_s = R.scan(*half, starts)
    assert got.dtype == torch.bfloat16
    assert _rel(got.cpu(), want) < 3e-2 and _rel(got_s.cpu(), want_s) < 3e-2
