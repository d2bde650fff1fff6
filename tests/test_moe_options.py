"""MoE variants on CPU: zero experts (LongCat-Flash), LatentMoE (Nemotron 3), expert_norm."""
import torch

from bux_b200.config import layers as L
from bux_b200.lang import compile_runs
from bux_b200.models.layers import moe as M
from bux_b200.train.trainer import Trainer

SRC = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope())
m = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish){options})
block = [n a] [n m]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 32
batch = 2
steps = 3
precision = precision(compute=float32)
"""


def _train(options: str):
    run = compile_runs(SRC.format(options=options), filename="x.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]
    return tr


def _moes(tr):
    return [m for m in tr.model.modules() if isinstance(m, M.MoE)]


def test_zero_experts_pass_tokens_through():
    tr = _train(", num_zero_experts=2, load_balancing=aux_free")
    layer = _moes(tr)[0]
    assert layer.router.weight.shape[0] == 6 and layer.router_bias.shape == (6,)
    # a router that only ever picks zero experts makes the layer the identity times the weights' sum
    with torch.no_grad():
        layer.router.weight.zero_()
        layer.router_bias.copy_(torch.tensor([0.0, 0, 0, 0, 9, 9]))
    from bux_b200.models.registry import Context

    x = torch.randn(2, 8, 32)
    ctx = Context(torch.zeros(2, 8, dtype=torch.long))
    out = layer(x, ctx)
    assert torch.allclose(out, x, atol=1e-5)  # normalised top-k weights of the two zero experts sum to 1


def test_zero_experts_balance_by_their_budget():
    c = L.MoEConfig(num_experts=4, top_k=2, num_zero_experts=4, load_balancing="aux_free",
                    expert=L.MLPConfig(type="gated_mlp", intermediate_size=8, activation="swish"))
    assert c.ffn_budget == 1.0
    scores = torch.full((1, 4, 8), 1 / 8)
    picks = torch.zeros(1, 4, 8)
    picks[:, :, :4] = 0.25  # each FFN expert a quarter of a pick per token: one FFN pick a token
    picks[:, :, 4:] = 0.25  # and one zero pick
    assert torch.allclose(M.budget_loss(scores, picks, c, False), torch.tensor(1.0))
    load = torch.tensor([10.0, 30, 20, 20, 5, 5, 5, 5])
    move = M.budget_move(load, c)
    target = 1.0 * 100 / (2 * 4)
    assert torch.allclose(move[:4], c.bias_update_rate * (1 - load[:4] / target))
    assert move[4:].abs().sum() == 0


def test_latent_moe_runs_experts_in_a_narrower_space():
    tr = _train(", latent_size=16, latent_input_norm=rmsnorm, latent_output_norm=rmsnorm, num_shared_experts=1")
    layer = _moes(tr)[0]
    assert layer.experts_gate_up.shape == (4, 32, 16) and layer.experts_down.shape == (4, 16, 16)
    assert layer.to_latent.weight.shape == (16, 32) and layer.from_latent.weight.shape == (32, 16)
    assert layer.shared.down.weight.shape[0] == 32  # shared experts see the full width


def test_expert_norm_normalises_each_experts_output():
    tr = _train(", expert_norm=rmsnorm")
    layer = _moes(tr)[0]
    assert layer.expert_norm.scale.grad is not None or layer.expert_norm.scale.requires_grad
    # with top_k = 1 and weight 1 the output rows have unit RMS (gain 1)
    from bux_b200.models.registry import Context

    c = layer.c.model_copy(update={"top_k": 1})
    layer.c = c
    with torch.no_grad():
        layer.expert_norm.scale.fill_(1.0)
        layer.experts_down.mul_(100.0)  # outputs far above the norm's eps
    x = torch.randn(2, 8, 32)
    out = layer(x, Context(torch.zeros(2, 8, dtype=torch.long)))
    assert torch.allclose(out.float().pow(2).mean(-1).sqrt(), torch.ones(2, 8), atol=1e-3)


def test_plain_mlp_experts_match_a_loop_over_the_picks_and_round_trip_through_the_export():
    """Routed experts that are plain MLPs (one projection up, relu², one down)."""
    from bux_b200.export import weights as W

    src = SRC.replace("expert=gated_mlp(intermediate_size=16, activation=swish){options}",
                      "expert=mlp(intermediate_size=16, activation=relu2)")
    run = compile_runs(src, filename="x.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
    assert losses[-1] < losses[0]
    m = _moes(tr)[0]
    assert m.experts_gate_up.shape == (4, 16, 32) and not m.gated
    from bux_b200.models.registry import Context

    x = torch.randn(1, 5, 32)
    ctx = Context(torch.zeros(1, 5, dtype=torch.long), None, None, training=False)
    idx, w, _ = m.route(x, ctx)
    want = torch.zeros(5, 32)
    for t in range(5):
        for j in range(idx.shape[-1]):
            e = int(idx[0, t, j])
            h = torch.relu(x[0, t] @ m.experts_gate_up[e].t()).square()
            want[t] += w[0, t, j] * (h @ m.experts_down[e].t())
    assert torch.allclose(m(x, ctx)[0], want, atol=1e-5)
    exported = W.tensors(tr.model)
    assert any(k.endswith("experts.up") for k in exported) and not any(k.endswith("experts.gate") for k in exported)
    back = W.fused(tr.model, exported)
    for name, p in tr.model.state_dict().items():
        assert torch.equal(back[name], p), name


def test_experts_soft_cap_their_up_branch_as_an_mlp_does():
    """An expert with ``up_softcap`` (and ``limit``): one expert with every token routed to it is
    the same function as the dense gated MLP of the same weights."""
    import torch

    from bux_b200.lang import compile
    from bux_b200.models import Model

    torch.manual_seed(0)
    src = ("d_model=16\nvocab_size=8\nf = gated_mlp(intermediate_size=24, activation=swish, limit=1.5, up_softcap=1.0, up_offset=1.0)\n"
           "e = moe(num_experts=1, top_k=1, expert=f)\nmodel = embed [{0}] head\n")
    dense = Model(compile(src.format("f"), filename="m.bux"), dtype=torch.float32).graph.items[1].body
    sparse = Model(compile(src.format("e"), filename="m.bux"), dtype=torch.float32).graph.items[1].body
    with torch.no_grad():
        sparse.experts_gate_up[0].copy_(dense.gate_up.weight)
        sparse.experts_down[0].copy_(dense.down.weight)
    x = torch.randn(2, 5, 16) * 3
    from bux_b200.models.registry import Context, Precision

    ids = torch.zeros(2, 5, dtype=torch.long)
    ctx = Context(ids, None, None, training=False, precision=Precision(compute=torch.float32))
    assert torch.allclose(sparse(x, ctx), dense(x, ctx), atol=1e-5)


def test_shared_experts_scored_by_the_router_and_the_smebu_move():
    """``shared_expert_sink``: every shared expert's hidden units are weighted by its own score,
    normalised with the picks. ``smebu``: the bias moves by the running average of the centred,
    soft-clamped shortfalls (``architecture/experts/moe.py:259-273,365-425`` there)."""
    import torch
    import torch.nn.functional as F

    from bux_b200.lang import compile
    from bux_b200.models import Model
    from bux_b200.models.registry import Context, Precision

    torch.manual_seed(0)
    arch = compile("d_model=16\nvocab_size=8\nf = gated_mlp(intermediate_size=8, activation=swish)\n"
                   "e = moe(num_experts=4, top_k=2, expert=f, num_shared_experts=2, shared_expert_sink=true, load_balancing=smebu,"
                   " bias_update_rate=0.1, bias_softclamp=2.0, bias_momentum=0.5)\nmodel = embed [e] head\n", filename="m.bux")
    layer = Model(arch, dtype=torch.float32).graph.items[1].body
    x = torch.randn(2, 5, 16)
    ctx = Context(torch.zeros(2, 5, dtype=torch.long), None, None, training=True, precision=Precision(compute=torch.float32))
    idx, weights, sinks = layer.route(x, ctx)
    assert sinks.shape[-1] == 2 and torch.allclose(weights.sum(-1) + sinks.sum(-1), torch.ones(2, 5), atol=1e-5)
    h = x @ layer.shared.gate_up.weight.t()
    hidden = F.silu(h[..., :16]) * h[..., 16:]
    want_shared = (hidden * sinks.repeat_interleave(8, dim=-1)) @ layer.shared.down.weight.t()
    got = layer(x, ctx)
    from bux_b200 import ops

    routed = ops.moe_reference(x.reshape(10, 16), layer.experts_gate_up, layer.experts_down, weights.reshape(10, 2), idx.reshape(10, 2)).view(2, 5, 16)
    assert torch.allclose(got, routed + want_shared, atol=1e-5)
    load = layer.router_load.clone()
    mean = load.mean()
    move = 0.1 * torch.tanh(2.0 * (mean - load) / mean)
    move = move - move.mean()
    layer.step_end_update()
    assert torch.allclose(layer.router_bias[:4], 0.5 * move[:4] if move.numel() > 4 else 0.5 * move, atol=1e-6)
    assert float(layer.router_load.sum()) == 0


def test_experts_with_biases_are_the_dense_mlp_and_skip_weight_decay():
    """``expert=gated_mlp(bias=true)``: one expert with every token routed to it is the dense
    gated MLP with the same weights and biases; the bias stacks are 2-D but weight decay skips
    them (reference: ``architecture/experts/moe.py:139,608-622``)."""
    from bux_b200.lang import compile
    from bux_b200.models import Model
    from bux_b200.models.registry import Context, Precision
    from bux_b200.train import optim

    torch.manual_seed(0)
    src = ("d_model=16\nvocab_size=8\nf = gated_mlp(intermediate_size=24, activation=swish, bias=true)\n"
           "e = moe(num_experts=1, top_k=1, expert=f)\nmodel = embed [{0}] head\n")
    dense = Model(compile(src.format("f"), filename="m.bux"), dtype=torch.float32).graph.items[1].body
    model = Model(compile(src.format("e"), filename="m.bux"), dtype=torch.float32)
    sparse = model.graph.items[1].body
    with torch.no_grad():
        dense.gate_up.bias.normal_()
        dense.down.bias.normal_()
        sparse.experts_gate_up[0].copy_(dense.gate_up.weight)
        sparse.experts_down[0].copy_(dense.down.weight)
        sparse.up_bias[0].copy_(dense.gate_up.bias)
        sparse.down_bias[0].copy_(dense.down.bias)
    x = torch.randn(2, 5, 16)
    ctx = Context(torch.zeros(2, 5, dtype=torch.long), None, None, training=False,
                  precision=Precision(compute=torch.float32))
    assert torch.allclose(sparse(x, ctx), dense(x, ctx), atol=1e-5)
    named = dict(model.named_parameters())
    for name, p in named.items():
        if name.endswith(("up_bias", "down_bias")):
            assert p.ndim == 2 and not optim.weight_decay_mask(name, p)
        if name.endswith("experts_gate_up"):
            assert optim.weight_decay_mask(name, p) and optim.muon_eligible(name, p)
