"""gqa's less common settings on CPU: each trains, and what it computes is checked by hand."""
import math

import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.models.layers import attention as A
from bux_b200.models.registry import Context
from bux_b200.train.trainer import Trainer

SRC = """
d_model=32
vocab_size=64
n = rmsnorm
a = {attn}
m = gated_mlp(intermediate_size=48, activation=swish)
block = [n a] [n m]
model = {model}
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 32
batch = 2
steps = 3
precision = precision(compute=float32)
"""


def _train(attn: str, model: str = "embed block^2 n head"):
    run = compile_runs(SRC.format(attn=attn, model=model), filename="x.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]
    return tr


def _layers(tr):
    return [m for m in tr.model.modules() if isinstance(m, A.GQA)]


def _ctx(b=2, t=32):
    return Context(torch.zeros(b, t, dtype=torch.long))


@pytest.mark.parametrize("options", [
    "power_scale=0.5, power_scale_length=16",
    "rope=rope(), log_scale=0.2, log_scale_floor=8",
    "rope=rope(), kv_conv_size=3",
    "rope=rope(), k_eq_v=true, qk_norm=rmsnorm",
    "rope=rope(), differential=true, sinks=true",
    "rope=rope(), exclusive=true",
    "rope=rope(), exclusive=learned",
    "rope=rope(), relative_bias=relbias(rank=4, extent=8), log_scale=0.1, log_scale_floor=4, softcap=20.0",
    "rope=rope(), attention_dropout=0.1",
    "rope=rope(), gated=true, gate_head_bias=true, gate_input_rank=4, gate_output_rank=4, gate_cross_head=true",
    "rope=rope(), gated=true, gate_per_head=true, gate_activation=softplus",
])
def test_setting_trains(options):
    _train(f"gqa(num_heads=4, num_kv_heads=2, {options})")


def test_scales_by_hand():
    pos = torch.tensor([0, 15, 31])
    assert torch.allclose(A.power_scale(pos, 0.5, 16), torch.tensor([(1 + 1 / 16) ** 0.5, 2 ** 0.5, 3 ** 0.5]))
    want = torch.tensor([1.0, 1 + 0.2 * math.log(2.0), 1 + 0.2 * math.log(4.0)])
    assert torch.allclose(A.length_scale(pos, 0.2, 8), want)


def test_length_scale_on_the_query_is_the_scale_on_the_logits():
    """Without a bias the two routes (scaled queries into the attention kernel, scaled
    logits in the full-logits path) give the same output."""
    tr = _train("gqa(num_heads=4, num_kv_heads=2, rope=rope(), log_scale=0.5, log_scale_floor=4, sinks=true)")
    layer = _layers(tr)[0]
    x = torch.randn(2, 32, 32)
    with torch.no_grad():
        layer.sinks.copy_(torch.randn(4))
        fast = layer(x, _ctx())
        layer.c = layer.c.model_copy(update={"attention_dropout": 0.5})  # takes the full-logits path
        ctx = _ctx()
        ctx.training = True
        torch.manual_seed(0)
        import torch.nn.functional as F

        keep = F.dropout
        F.dropout = lambda p, rate, *a, **k: p  # dropout off: the same function otherwise
        try:
            full = layer(x, ctx)
        finally:
            F.dropout = keep
    assert torch.allclose(fast, full, atol=1e-5)


def test_exclusive_output_is_orthogonal_to_the_tokens_own_value():
    out = torch.randn(2, 5, 4, 8)
    v = torch.randn(2, 5, 2, 8)
    y = A.exclusive(out, v)
    u = v.repeat_interleave(2, dim=2)
    assert (y * u).sum(-1).abs().max() < 1e-5
    half = A.exclusive(out, v, torch.full((4,), 0.5))
    assert torch.allclose(half, 0.5 * (out + y), atol=1e-6)


def test_relative_bias_by_hand():
    torch.manual_seed(0)
    r = torch.randn(1, 6, 2, 3)
    table = torch.randn(3, 4)
    bias = A.relative_bias(r, table, 6)
    assert bias.shape == (1, 2, 6, 6)
    for i in range(6):
        for j in range(6):
            want = r[0, i] @ table[:, i - j] if 0 <= i - j < 4 else torch.zeros(2)
            assert torch.allclose(bias[0, :, i, j], want, atol=1e-6)


def test_differential_and_k_eq_v_shapes():
    tr = _train("gqa(num_heads=4, num_kv_heads=2, rope=rope(), differential=true)")
    layer = _layers(tr)[0]
    assert layer.qkv.weight.shape[0] == (8 + 2 + 2) * 8 and layer.o.weight.shape[1] == 32
    assert layer.lambda_proj.weight.shape == (4, 32)
    tr = _train("gqa(num_heads=4, num_kv_heads=2, rope=rope(), k_eq_v=true)")
    layer = _layers(tr)[0]
    assert layer.qkv.weight.shape[0] == (4 + 2) * 8


def test_value_residual_learned_and_convex():
    for kind, shape in (("learned", (2,)), ("convex", ())):
        tr = _train(f"gqa(num_heads=4, num_kv_heads=2, rope=rope(), value_residual={kind}, v=$v)",
                    model="embed [n gqa(num_heads=4, num_kv_heads=2, rope=rope(), v=@v)] block^2 n head")
        mixes = [m.v_mix for m in _layers(tr) if hasattr(m, "v_mix")]
        assert len(mixes) == 2 and all(w.shape == shape for w in mixes)


def test_value_embedding_gate_starts_open():
    tr = _train("gqa(num_heads=4, num_kv_heads=2, rope=rope(), ve=$ve!, value_embed_gate=4)",
                model="embed (value_embed(features=16, ve=@ve) block)^2 n head")
    layer = _layers(tr)[0]
    assert layer.ve_gate.weight.shape == (2, 8)
    with torch.no_grad():
        layer.ve_gate.weight.zero_()
    v, e, x = torch.randn(2, 32, 2, 8), torch.randn(2, 32, 16), torch.randn(2, 32, 32)
    assert torch.allclose(layer._add_value_embedding(x, v, e, _ctx()), v + e.view(2, 32, 2, 8))


def test_paired_heads_share_one_softmax():
    """Paired attention is plain causal attention over the sequence with heads j and j + h/2
    interleaved: checked against a direct statement for one token pair ordering."""
    tr = _train("gqa(num_heads=4, num_kv_heads=2, rope=rope(), paired=true, sliding_window_size=16)")
    layer = _layers(tr)[0]
    torch.manual_seed(0)
    b, t, h, g, d = 1, 6, 4, 2, 8
    q, k, v = torch.randn(b, t, h, d), torch.randn(b, t, g, d), torch.randn(b, t, g, d)
    layer.c = layer.c.model_copy(update={"sliding_window_size": None})
    got = layer._attend_paired(q, k, v, _ctx(b, t))
    # by hand: query head j (j < 2) of token p sits at 2p, head j + 2 at 2p + 1; kv head m at 2p, m + 1 at 2p + 1
    for j in range(2):            # query head in the interleaved layout (2 of them), kv head 0 serves both
        for p in range(t):
            for second in (0, 1):
                head = j + 2 * second
                qq = q[0, p, head]
                keys, vals = [], []
                for s_pos in range(2 * p + second + 1):
                    tok, half = divmod(s_pos, 2)
                    keys.append(k[0, tok, half])   # one kv head per half (g / 2 = 1)
                    vals.append(v[0, tok, half])
                logits = torch.stack(keys) @ qq * d ** -0.5
                want = torch.softmax(logits, 0) @ torch.stack(vals)
                assert torch.allclose(got[0, p, head], want, atol=1e-5), (j, p, second)


def test_mimetic_vo_init_makes_self_attention_subtract_beta_of_the_stream():
    """With the mimetic V-O init and no noise, a token that attends to itself alone gets
    -beta of its own first g·dv channels back (value-output map -beta·I on them)."""
    from bux_b200.lang import compile
    from bux_b200.models import Model
    from bux_b200.models.layers.attention import GQA

    arch = compile("d_model=32\nvocab_size=16\n"
                   "model = embed [gqa(num_heads=4, num_kv_heads=2, head_dim=8, mimetic_vo=0.5, mimetic_noise=0.0, rope=none)] head\n")
    layer = [m for m in Model(arch).modules() if isinstance(m, GQA)][0]
    wv = layer.qkv.weight[layer.q_rows + layer.k_rows:]                  # [g·dv, d]
    vo = layer.o.weight.float() @ wv.float().repeat_interleave(1, 0).view(2, 8, 32).repeat_interleave(2, 0).reshape(32, 32)
    want = torch.zeros(32, 32)
    want[:16, :16] = -0.5 * torch.eye(16)
    assert torch.allclose(vo, want, atol=1e-6)
