"""The chunk-scan op's packing and backward formulas, with the kernel replaced by its statement in PyTorch."""

import torch

from bux_b200.ops import scan


def _kernel_statement(a1, aux1, aux3, a4, v, lam, s0, *, want_out, reverse):
    """What `chunk_scan_kernel` computes, in fp32 on the host."""
    b, h, n = v.shape[:3]
    a1, aux1, a4, v = a1.float(), aux1.float(), a4.float(), v.float()
    S = s0.clone() if s0 is not None else torch.zeros(b, h, 128, 128)
    out = torch.zeros(b, h, n, 64, 128)
    x_out = torch.zeros(b, h, n, 64, 128)
    states = torch.zeros(b, h, n, 128, 128)
    for i in (range(n - 1, -1, -1) if reverse else range(n)):
        states[:, :, i] = S
        Y = a1[:, :, i] @ S + aux1[:, :, i] @ v[:, :, i]
        X = Y[:, :, :64]
        x_out[:, :, i] = X
        if want_out:
            out[:, :, i] = Y[:, :, 64:] + aux3[:, :, i].float() @ X
        S = lam[:, :, i].unsqueeze(-1) * S + a4[:, :, i].transpose(-1, -2) @ torch.cat([v[:, :, i], X], dim=-2)
    return (out if want_out else None), x_out, states, S


def _loop(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0):
    b, h, n = V.shape[:3]
    S = S0.clone() if S0 is not None else torch.zeros(b, h, Qd.shape[-1], V.shape[-1])
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


def _case(rank1, dk, dv, with_state, monkeypatch):
    monkeypatch.setattr(scan, "_run", _kernel_statement)
    torch.manual_seed(0)
    b, h, n = 1, 2, 3

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape) * scale).bfloat16().float().requires_grad_()

    Qd, Kd, V = rnd(b, h, n, 64, dk, scale=0.3), rnd(b, h, n, 64, dk, scale=0.3), rnd(b, h, n, 64, dv)
    Mqk = rnd(b, h, n, 64, 64, scale=0.2)
    lam = torch.rand(b, h, n, dk).mul(0.5).add(0.5).requires_grad_()
    S0 = rnd(b, h, dk, dv, scale=0.5) if with_state else None
    P = W = Mqb = Bd = None
    if rank1:
        P, Bd = rnd(b, h, n, 64, dk, scale=0.1), rnd(b, h, n, 64, dk, scale=0.1)
        W, Mqb = rnd(b, h, n, 64, 64, scale=0.1), rnd(b, h, n, 64, 64, scale=0.2)
    leaves = [t for t in (P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0) if t is not None]
    go, gs = torch.randn(b, h, n, 64, dv), torch.randn(b, h, dk, dv) * 0.1
    want_o, want_s = _loop(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)
    ((want_o * go).sum() + (want_s * gs).sum()).backward()
    want_g = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    got_o, got_s = scan.chunk_scan(P, Qd, W, Mqk, Mqb, Kd, Bd, V, lam, S0)
    ((got_o * go).sum() + (got_s * gs).sum()).backward()
    assert torch.allclose(got_o, want_o, atol=1e-4) and torch.allclose(got_s, want_s, atol=1e-4)
    for t, w in zip(leaves, want_g):
        # the backward hands dO to the reverse walk in bf16
        assert (t.grad - w).norm() / w.norm() < 1e-2


def test_rank_one_recurrence(monkeypatch):
    _case(True, 128, 128, False, monkeypatch)


def test_rank_one_recurrence_with_padded_dims_and_a_state(monkeypatch):
    _case(True, 64, 96, True, monkeypatch)


def test_decayed_recurrence(monkeypatch):
    _case(False, 32, 128, True, monkeypatch)
