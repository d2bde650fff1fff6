"""The copy pointer of a head (CPLM) on CPU."""
import math

import torch

from bux_b200.lang import compile_runs
from bux_b200.models.layers import pointer as P
from bux_b200.train.trainer import Trainer

SRC = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope())
m = gated_mlp(intermediate_size=48, activation=swish)
block = [n a] [n m]
model = embed block^2 n head(pointer=copy_pointer(dim=16{options}))
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 32
batch = 2
steps = 3
precision = precision(compute=float32)
"""


def test_head_with_a_pointer_trains():
    for options in ("", ", window=8, token=63"):
        run = compile_runs(SRC.format(options=options), filename="x.bux")[0]
        tr = Trainer(run, device="cpu")
        batch = next(iter(tr.batches()))
        losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
        assert all(math.isfinite(x) for x in losses) and losses[-1] < losses[0]
        names = [n for n, _ in tr.model.named_parameters()]
        assert any("pointer.sink" in n for n in names) and any("pointer.gain" in n for n in names)


def test_mixture_is_a_probability_distribution():
    """Σ_y p(y) over the tokens (the <copy> row left out) is 1 at every position."""
    torch.manual_seed(0)
    b, t, c, vocab, copy = 1, 6, 4, 9, 8
    tokens = torch.tensor([[1, 2, 1, 3, 2, 1]])
    view = P.PointerView(torch.randn(b, t, c), torch.randn(b, t, c), torch.randn(b, t), tokens,
                         torch.ones(b, t, dtype=torch.long), copy, None)
    logits = torch.randn(t, vocab)
    total = torch.zeros(t)
    for y in range(vocab - 1):
        tg = torch.full((b, t), y)
        log_copy, log_sink = view.logs(tg)
        nll, _ = P.mixture_nll(logits, tg.reshape(-1), copy, log_copy.reshape(-1), log_sink.reshape(-1))
        total += torch.exp(-nll)
    assert torch.allclose(total, torch.ones(t), atol=1e-5)


def test_pointer_by_hand():
    """One earlier position holds the target: p_copy is its share of the attention."""
    q = torch.tensor([[[0.0, 0.0], [2.0, 0.0], [2.0, 0.0]]])
    k = torch.tensor([[[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]])
    sink = torch.zeros(1, 3)
    tokens = torch.tensor([[5, 6, 7]])
    view = P.PointerView(q, k, sink, tokens, torch.ones(1, 3, dtype=torch.long), 9, None)
    log_copy, log_sink = view.logs(torch.tensor([[5, 5, 5]]))
    assert log_copy[0, 0] == float("-inf")                       # nothing before the first position
    s = 2.0 / math.sqrt(2)                                       # score of position 0 for queries 1 and 2
    assert math.isclose(log_copy[0, 1].exp().item(), math.exp(s) / (math.exp(s) + 1), rel_tol=1e-5)
    assert math.isclose(log_copy[0, 2].exp().item(), math.exp(s) / (math.exp(s) + 2), rel_tol=1e-5)
    assert math.isclose(log_sink[0, 2].exp().item(), 1 / (math.exp(s) + 2), rel_tol=1e-5)
    # a window of one position hides position 0 from the last query
    view.window = 1
    log_copy, _ = view.logs(torch.tensor([[5, 5, 5]]))
    assert log_copy[0, 2] == float("-inf") and log_copy[0, 1] > float("-inf")


def test_without_gate_mass_the_loss_is_cross_entropy_over_the_other_rows():
    logits = torch.randn(5, 8)
    logits[:, 7] = -1e4  # <copy> gets no mass
    targets = torch.tensor([0, 1, 2, 3, 4])
    nll, _ = P.mixture_nll(logits, targets, 7, torch.full((5,), float("-inf")), torch.zeros(5))
    want = torch.nn.functional.cross_entropy(logits[:, :7], targets, reduction="none")
    assert torch.allclose(nll, want, atol=1e-5)
