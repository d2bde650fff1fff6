"""NVFP4: the quantiser's recipe and a linear layer trained with it (CPU)."""
import torch

from bux_b200.lang import compile_runs
from bux_b200.ops import nvfp4 as N


def test_values_lie_on_the_e2m1_grid_and_scales_on_e4m3():
    torch.manual_seed(0)
    x = torch.randn(32, 64) * torch.logspace(-2, 2, 64)
    b = N.quantize(x)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    assert torch.isin(b.values.abs(), grid).all()
    assert torch.equal(b.scales, b.scales.to(torch.float8_e4m3fn).float())
    # the largest magnitude maps to 6 x 448 tensor scales: nothing saturates
    assert ((b.dequantized() - x).abs() <= 0.26 * x.abs().view(32, 4, 16).amax(-1).repeat_interleave(16, 1) + 1e-6).all()


def test_round_to_nearest_even_on_the_grid():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -2.5])
    assert N.round_e2m1(x).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0, -2.0]


def test_weight_tiles_give_the_transpose_the_same_values():
    torch.manual_seed(1)
    w = torch.randn(48, 32)
    a, b = N.quantize(w, tiles=True), N.quantize(w.t().contiguous(), tiles=True)
    assert torch.equal(a.dequantized(), b.dequantized().t())


def test_stochastic_rounding_is_unbiased_and_hadamard_cancels():
    torch.manual_seed(2)
    x = torch.randn(16, 64)
    mean = sum(N.quantize(x, stochastic=True, seed=s).dequantized() for s in range(300)) / 300
    assert ((mean - x).norm() / x.norm()).item() < 0.02
    y = torch.randn(24, 64)
    assert torch.allclose(N.hadamard_rows(x) @ N.hadamard_rows(y).t(), x @ y.t(), atol=1e-4)


def test_pack_two_codes_per_byte():
    b = N.quantize(torch.tensor([[0.5, -1.0, 6.0, -6.0] * 4]))
    packed, scales = N.pack(b)
    assert packed.shape == (1, 8) and scales.shape == (1, 1)
    lo, hi = packed & 0xF, packed >> 4
    codes = torch.stack([lo, hi], -1).view(1, 16)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    back = grid[(codes & 7).long()] * torch.where(codes & 8 > 0, -1.0, 1.0)
    assert torch.equal(back, b.values)


def test_a_model_trains_with_nvfp4_matmuls():
    """A few steps with every matmul in NVFP4 stay close to the same steps in fp32, and the
    first step's gradients point the same way."""
    from bux_b200.train.trainer import Trainer

    src = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope())
m = gated_mlp(intermediate_size=64, activation=swish)
model = embed ([n a] [n m])^2 n head
data = synthetic
optimizer = adamw(lr=3e-3)
seq_len = 32
batch = 8
steps = 6
precision = precision(compute=float32, matmuls={fmt})
"""
    runs = {fmt: compile_runs(src.format(fmt=fmt), filename="n.bux")[0] for fmt in ("compute", "nvfp4")}
    losses, grads = {}, {}
    for fmt, run in runs.items():
        tr = Trainer(run, device="cpu")
        feed = iter(tr.batches())
        batch = next(feed)
        loss, _ = tr.forward_loss(tr.to_device(batch), torch.tensor(1.0 / (8 * 31)), 1, 1)
        loss.backward()
        grads[fmt] = torch.cat([p.grad.reshape(-1) for p in tr.model.parameters() if p.grad is not None])
        tr.model.zero_grad()
        losses[fmt] = [tr.train_step(b)["loss"].item() for b, _ in zip(feed, range(5))]
    assert all(abs(a - b) < 0.05 for a, b in zip(losses["nvfp4"], losses["compute"]))
    cos = torch.nn.functional.cosine_similarity(grads["nvfp4"], grads["compute"], dim=0).item()
    assert cos > 0.9, cos
