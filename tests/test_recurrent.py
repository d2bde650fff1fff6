"""Recurrent mixers: the chunked scan against the position-by-position recurrence, and
every layer type of the family training on CPU."""
import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.models.layers import recurrent as R
from bux_b200.train.trainer import Trainer


def _inputs(t=150, dk=8, dv=12, per_channel=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    b, h = 2, 3
    q, k = torch.randn(b, t, h, dk, generator=g), torch.randn(b, t, h, dk, generator=g)
    v = torch.randn(b, t, h, dv, generator=g)
    gd = -torch.rand(b, t, h, dk if per_channel else 1, generator=g) * 0.3
    return q, R.l2norm(k), v, gd


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("rank_one", [False, True])
@pytest.mark.parametrize("docs", [False, True])
def test_chunked_scan_matches_the_recurrence(per_channel, rank_one, docs):
    q, k, v, g = _inputs(per_channel=per_channel)
    a = b = None
    if rank_one:
        gen = torch.Generator().manual_seed(1)
        kk = R.l2norm(torch.randn(k.shape, generator=gen))
        a, b = -kk, kk * torch.rand(k.shape, generator=gen)
    starts = None
    if docs:
        starts = torch.zeros(2, q.shape[1], dtype=torch.bool)
        starts[0, 70] = starts[1, 3] = starts[1, 129] = True
    want, s_want = R.scan_steps(q, k, v, g, a, b, starts)
    got, s_got = R.scan(q, k, v, g, a, b, starts)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)
    assert torch.allclose(s_got, s_want, atol=2e-4, rtol=1e-4)


def test_delta_rule_is_the_rank_one_recurrence():
    q, k, v, g = _inputs(t=100)
    beta = torch.rand(2, 100, 3)
    got, _ = R.delta_rule(q, k, v, g, beta)
    # S_t = (I - beta k k^T) diag(w) S_{t-1} + beta k v^T, position by position
    S = torch.zeros(2, 3, 8, 12)
    outs = []
    for i in range(100):
        S = g[:, i].exp().unsqueeze(-1) * S
        kt, bt = k[:, i], beta[:, i].unsqueeze(-1)
        S = S - (bt * kt).unsqueeze(-1) * torch.einsum("bhk,bhkv->bhv", kt, S).unsqueeze(-2) \
            + (bt * kt).unsqueeze(-1) * v[:, i].unsqueeze(-2)
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, i], S))
    assert torch.allclose(got, torch.stack(outs, 1), atol=2e-4, rtol=1e-4)


def test_mamba_scan_resets_at_document_starts():
    torch.manual_seed(0)
    x, dt = torch.randn(1, 12, 4), torch.rand(1, 12, 4) * 0.1
    A, B, C = -torch.rand(4, 3), torch.randn(1, 12, 3), torch.randn(1, 12, 3)
    starts = torch.zeros(1, 12, dtype=torch.bool)
    starts[0, 5] = True
    whole = R.mamba_scan(x, dt, A, B, C, starts)
    tail = R.mamba_scan(x[:, 5:], dt[:, 5:], A, B[:, 5:], C[:, 5:])
    assert torch.allclose(whole[:, 5:], tail, atol=1e-6)


SRC = """
d_model=32
vocab_size=64
n = rmsnorm
mixer = {mixer}
m = gated_mlp(intermediate_size=48, activation=swish)
block = [n mixer] [n m]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 80
batch = 2
steps = 3
precision = precision(compute=float32)
"""

MIXERS = [
    "deltanet(num_heads=2, head_dim=8)",
    "gdn(num_heads=2, head_dim=8, num_v_heads=4, v_head_dim=8)",
    "kda(num_heads=2, head_dim=8)",
    "kda(num_heads=2, head_dim=8, gate_lower_bound=-5.0)",
    "gdn2(num_heads=2, head_dim=8)",
    "gla(num_heads=2, head_dim=8)",
    "lightning(num_heads=2, head_dim=8)",
    "rwkv7(num_heads=2, head_dim=8, decay_rank=4, a_rank=4, v_rank=4, gate_rank=4)",
    "mamba(state_size=4, conv_size=3)",
    "mamba2(state_size=8, head_dim=8, conv_size=3)",
    "short_conv()",
]


@pytest.mark.parametrize("mixer", MIXERS)
def test_mixer_trains(mixer):
    run = compile_runs(SRC.format(mixer=mixer), filename="m.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]
