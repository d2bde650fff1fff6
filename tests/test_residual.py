"""Residual algebras: each starts as the plain pre-norm residual model (or its stated
equivalent), trains, and keeps the state layout the reference documents."""
import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.models import Model, residual as R
from bux_b200.train.trainer import Trainer

BASE = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope())
m = gated_mlp(intermediate_size=48, activation=swish)
block = [n a] [n m]
model = embed block^2 {tail}
{residual}
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 16
batch = 4
steps = 3
precision = precision(compute=float32)
"""


def _run(residual="", tail="n head"):
    src = BASE.format(residual=residual, tail=tail)
    return compile_runs(src, filename="r.bux")[0]


def _logits(run, ids):
    torch.manual_seed(0)
    model = Model(run.arch, dtype=torch.float32, seed=0)
    pos = torch.arange(ids.shape[1]).expand_as(ids)
    ctx = model(ids, pos, None, training=False)
    return model, ctx.heads[0].logits if hasattr(ctx.heads[0], "logits") else ctx.heads[0]


def test_sinkhorn_is_doubly_stochastic():
    m = R.sinkhorn(torch.randn(3, 5, 4, 4), 20)
    assert torch.allclose(m.sum(-2), torch.ones(3, 5, 4), atol=1e-3)
    assert torch.allclose(m.sum(-1), torch.ones(3, 5, 4), atol=1e-2)


def test_attnres_sources_by_blocks():
    state = torch.arange(1 * 1 * 6 * 2, dtype=torch.float32).view(1, 1, 6, 2)
    got = R.sources(state, 2)  # embedding, (o1+o2), (o3+o4), o5
    assert got.shape == (1, 1, 4, 2)
    assert torch.equal(got[0, 0, 1], state[0, 0, 1] + state[0, 0, 2])
    assert torch.equal(got[0, 0, 3], state[0, 0, 5])


def test_msar_layout_counts():
    # embedding + 3 expansions, then one finished block of 2 outputs + 3 expansions, 1 under way, head read
    assert R._msar_layout(1, 2, 3) is None
    assert R._msar_layout(1 + 3 + 1 + 1, 2, 3) == (0, 1)
    assert R._msar_layout(1 + 3 + (2 + 3) + 1 + 1, 2, 3) == (1, 1)
    with pytest.raises(ValueError):
        R._msar_layout(4, 2, 3)


@pytest.mark.parametrize("residual,tail", [
    ("residual = hc(expansion=2)", "merge n head"),
    ("residual = hc(expansion=2, single_pass=true)", "merge n head"),
    ("residual = mhc(expansion=2, sinkhorn_iters=3)", "merge n head"),
    ("residual = gr(rank=4, expansion=2)", "merge head"),
    ("residual = attnres()", "merge n head"),
    ("residual = attnres(block_size=2)", "merge n head"),
    ("residual = msar(kernel_sizes=[2, 3], block_size=2)", "merge n head"),
    ("residual = vpgate()", "n head"),
])
def test_algebra_trains(residual, tail):
    run = _run(residual, tail)
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]  # the same rows: the loss must fall
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0]
    names = [n for n, _ in tr.model.named_parameters()]
    assert any("algebra" in n for n in names)


def test_hc_starts_as_the_plain_residual_model():
    """Static hc with A_m = e_k, A_r = I, B = 1 and a summing merge: with n copies of the
    embedding, reading stream k gives what the plain model reads only while the streams
    are equal, so compare vpgate-free hc against a hand-rolled two-stream run instead:
    the merge (sum of n equal-start streams) equals n·embedding + n·(sum of outputs)
    when every branch writes to every stream."""
    run = _run("residual = hc(expansion=2, dynamic=false)", "merge n head")
    model = Model(run.arch, dtype=torch.float32, seed=0)
    alg = [m for m in model.modules() if isinstance(m, R.HyperConnections)]
    assert len(alg) == 5  # four branches and the merge's reader
    assert torch.equal(alg[0].static_alpha[:, 0], torch.tensor([1.0, 0.0]))
    assert torch.equal(alg[1].static_alpha[:, 0], torch.tensor([0.0, 1.0]))
    assert torch.equal(alg[0].static_alpha[:, 1:], torch.eye(2))
    assert getattr(alg[0].static_alpha, "no_weight_decay", False)


def test_vpgate_initial_weights():
    g = R.ResidualGate(R.L.ResidualGateConfig(), 8, index=2)
    a, b = g.weights()
    assert torch.allclose(b, torch.full((8,), 0.5), atol=1e-6)       # 1/sqrt(4)
    assert torch.allclose(a * a + b * b, torch.ones(8), atol=1e-5)  # variance preserving
