"""mla, value_embed, nextn, engram, doc_copy on CPU."""
import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.models.layers import extra as X
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
{extra}
"""
GQA = "gqa(num_heads=2, num_kv_heads=1, rope=rope())"


def _train(attn=GQA, model="embed block^2 n head", extra=""):
    run = compile_runs(SRC.format(attn=attn, model=model, extra=extra), filename="x.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(4)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]
    return tr


def test_mla_trains():
    _train("mla(num_heads=2, kv_lora_rank=8, q_lora_rank=8, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8)")


def test_value_embeddings_reach_the_attention_values():
    tr = _train("gqa(num_heads=2, num_kv_heads=1, rope=rope(), ve=$ve!)",
                model="embed (value_embed(features=16, ve=@ve) block)^2 n head")
    assert any("table" in n for n, _ in tr.model.named_parameters())


def test_nextn_adds_a_second_head():
    tr = _train(model="embed block @h n head $h nextn block n head", extra="loss = loss(mtp=0.3)")
    ids = torch.randint(0, 64, (2, 32))
    ctx = tr.model(ids, torch.arange(32).expand(2, 32), None, training=False)
    assert len(ctx.heads) == 2


def test_engram_trains_and_takes_distinct_primes():
    tr = _train(model="embed engram(head_dim=4, table_size=50, num_heads=2, conv_size=2) block^2 n head")
    (e,) = [m for m in tr.model.modules() if isinstance(m, X.Engram)]
    primes = e.primes.flatten().tolist()
    assert len(set(primes)) == len(primes) == 4 and all(X._is_prime(p) and p >= 50 for p in primes)


def test_copy_candidates_by_hand():
    #          0  1  2  3  4  5  6  7
    tokens = torch.tensor([[5, 6, 7, 5, 6, 9, 5, 6]])
    within = torch.arange(8).unsqueeze(0)
    doc = torch.zeros(1, 8, dtype=torch.long)
    cand, bucket = X.copy_candidates(tokens, within, doc, [1, 2], counts=3)
    # position 4 ends "5 6", seen ending at 1 → candidate is token 2 (7); length rank 2, once
    assert cand[0, 4].item() == 7 and bucket[0, 4].item() == (2 - 1) * 3 + 1
    # position 7 ends "5 6" again: latest earlier occurrence ended at 4 → candidate 9, twice
    assert cand[0, 7].item() == 9 and bucket[0, 7].item() == (2 - 1) * 3 + 2
    # position 3 ends "5" (seen at 0) but "7 5" never: length 1, candidate 6
    assert cand[0, 3].item() == 6 and bucket[0, 3].item() == 1
    assert cand[0, 0].item() == 0 and bucket[0, 0].item() == 0
    # a document boundary hides earlier occurrences
    doc2 = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 1]])
    within2 = torch.tensor([[0, 1, 2, 0, 1, 2, 3, 4]])
    cand2, _ = X.copy_candidates(tokens, within2, doc2, [1, 2], counts=3)
    assert cand2[0, 4].item() == 0 and cand2[0, 7].item() == 9


def test_doc_copy_trains():
    _train(model="embed doc_copy(lengths=[1, 2, 3]) block^2 n head")


def test_sparse_attention_with_an_indexer():
    from bux_b200.models.layers import sparse as S

    # top_mask keeps the k best of the seen keys, the first of equal ones
    sc = torch.tensor([[[3.0, 1.0, 3.0, 2.0]]])
    seen = torch.tensor([[[True, True, True, False]]])
    assert S.top_mask(sc, seen, 2).tolist() == [[[True, False, True, False]]]
    # with every key kept the sparse path is plain causal attention, and the loss is finite
    attn = "gqa(num_heads=2, num_kv_heads=1, rope=rope(), indexer=indexer(num_heads=2, head_dim=8, top_k=8))"
    tr = _train(attn)
    assert any("indexer" in n for n, _ in tr.model.named_parameters())
    ids = torch.randint(0, 64, (2, 32))
    ctx = tr.model(ids, torch.arange(32).expand(2, 32), None, training=True)
    assert "indexer_loss" in ctx.losses and torch.isfinite(ctx.losses["indexer_loss"])
    # the loss trains the indexer only
    loss = ctx.losses["indexer_loss"]
    grads = torch.autograd.grad(loss, [p for p in tr.model.parameters()], allow_unused=True)
    touched = {n for (n, _), g in zip(tr.model.named_parameters(), grads) if g is not None and g.abs().sum() > 0}
    assert touched and all("indexer" in n for n in touched)


def test_index_port_shares_the_picks():
    first = "gqa(num_heads=2, num_kv_heads=1, rope=rope(), indexer=indexer(num_heads=2, head_dim=8, top_k=4), index=@picks)"
    model = "embed [n a] [n m] [n gqa(num_heads=2, num_kv_heads=1, rope=rope(), indexer=indexer(num_heads=2, head_dim=8, top_k=4), index=$picks!)] n head"
    tr = _train(first, model=model)
    names = [n for n, _ in tr.model.named_parameters() if "indexer" in n]
    assert names and all(".items.1." in n for n in names)   # only the first layer owns an indexer


def test_mla_with_an_indexer():
    """With every key kept the sparse MLA is the dense one; the indexer gets its own loss."""
    base = "mla(num_heads=2, kv_lora_rank=8, q_lora_rank=8, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8{more})"
    tr = _train(base.format(more=", indexer=indexer(num_heads=2, head_dim=8, top_k=4)"))
    assert any("indexer" in n for n, _ in tr.model.named_parameters())
    ids = torch.randint(0, 64, (2, 32))
    ctx = tr.model(ids, torch.arange(32).expand(2, 32), None, training=True)
    assert "indexer_loss" in ctx.losses and torch.isfinite(ctx.losses["indexer_loss"])
    (layer,) = [m for m in tr.model.modules() if isinstance(m, X.MLA)][:1]
    x = torch.randn(2, 32, 32)
    from bux_b200.models.registry import Context

    def run(top_k):
        layer.c = layer.c.model_copy(update={"indexer": layer.c.indexer.model_copy(update={"top_k": top_k})})
        return layer(x, Context(torch.zeros(2, 32, dtype=torch.long)))

    with torch.no_grad():
        everything = run(32)
        layer_dense_cfg = layer.c.model_copy(update={"indexer": None})
        sparse_cfg, layer.c = layer.c, layer_dense_cfg
        dense = layer(x, Context(torch.zeros(2, 32, dtype=torch.long)))
        layer.c = sparse_cfg
        few = run(2)
    assert torch.allclose(everything, dense, atol=1e-5)
    assert not torch.allclose(few, dense, atol=1e-3)


CSA_SRC = """
d_model=32
vocab_size=64
n = rmsnorm
a = csa(num_heads=2, head_dim=16, q_lora_rank=16, o_lora_rank=8, o_groups=2, sliding_window_size=8,
        sinks=true, compress_ratio=4, rope=rope(fraction=0.5, layout=interleaved))
w = csa(num_heads=2, head_dim=16, sliding_window_size=8)
m = gated_mlp(intermediate_size=48, activation=swish)
model = embed [n a] [n m] [n w] [n m] n head
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 40
batch = 2
steps = 3
precision = precision(compute=float32)
"""


def test_csa_trains_is_causal_and_sees_compressed_latents_past_its_window():
    import torch

    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    run = compile_runs(CSA_SRC, filename="c.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(5)]
    assert losses[-1] < losses[0]
    model = tr.model.eval()
    ids = torch.randint(0, 64, (1, 40), generator=torch.Generator().manual_seed(0))
    base = model.logits(ids, training=False)
    later = ids.clone()
    later[0, 30] = (later[0, 30] + 1) % 64
    moved = model.logits(later, training=False)
    assert torch.allclose(base[:, :30], moved[:, :30], atol=1e-5)          # causal
    # a token 20 positions back is outside both layers' windows (8 + 8): only a compressed
    # latent can carry it to position 39
    early = ids.clone()
    early[0, 2] = (early[0, 2] + 1) % 64
    far = model.logits(early, training=False)
    assert not torch.allclose(base[:, 39], far[:, 39], atol=1e-6)


def test_csa_indexer_keeps_the_best_latents_and_its_ports_share_them():
    """A layer that compresses and indexes writes its latents and picks; the next reuses both
    (it has neither a compression nor an indexer of its own); a third re-indexes inside the
    first one's candidate pool."""
    from bux_b200.lang import compile_runs
    from bux_b200.models.layers.csa import CSA
    from bux_b200.train.trainer import Trainer

    src = CSA_SRC.replace("sinks=true, compress_ratio=4,", "sinks=true, compress_ratio=2, "
                          "indexer=indexer(num_heads=2, head_dim=8, top_k=4, candidate_block_size=2, candidate_top_k=8),")
    src = src.replace("model = embed [n a] [n m] [n w] [n m] n head",
                      "model = embed [n a(kv=@kv, index=@picks, candidates=@pool)] [n m] [n a(kv=$kv, index=$picks)] [n m] "
                      "[n a(kv=$kv, index=@again, candidates=$pool)] [n m] n head")
    run = compile_runs(src, filename="c.bux")[0]
    tr = Trainer(run, device="cpu")
    first, reuse, again = [m for m in tr.model.modules() if isinstance(m, CSA)]
    assert hasattr(first, "compress_kv") and hasattr(first.indexer, "k")
    assert not hasattr(reuse, "compress_kv") and not hasattr(reuse, "indexer")
    assert not hasattr(again, "compress_kv") and hasattr(again, "indexer") and not hasattr(again.indexer, "k")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(5)]
    assert losses[-1] < losses[0]
    ids = torch.randint(0, 64, (1, 40), generator=torch.Generator().manual_seed(0))
    ctx = tr.model(ids, torch.arange(40).unsqueeze(0), None, training=True)
    assert torch.isfinite(ctx.losses["indexer_loss"])
    kept, pool, kept_again = ctx.taps["picks"][-1], ctx.taps["pool"][-1], ctx.taps["again"][-1]
    latents, valid, index_keys = ctx.taps["kv"][-1]
    assert index_keys is not None and valid[0].tolist() == [(i + 1) % 2 == 0 for i in range(40)]
    assert kept.sum(-1).max() == 4 and not (kept & ~valid.unsqueeze(1)).any()       # top 4 of the latents it sees
    assert pool.sum(-1).max() <= 8 and not (kept_again & ~pool).any()               # picks stay inside the pool
    # the indexer's loss trains the indexers only
    grads = torch.autograd.grad(ctx.losses["indexer_loss"], list(tr.model.parameters()), allow_unused=True)
    touched = {n for (n, _), g in zip(tr.model.named_parameters(), grads) if g is not None and g.abs().sum() > 0}
    assert touched and all("indexer" in n for n in touched)


def test_csa_ports_need_compressed_latents():
    import pytest

    from bux_b200.lang import compile_runs
    from bux_b200.models import Model

    src = CSA_SRC.replace("w = csa(num_heads=2, head_dim=16, sliding_window_size=8)",
                          "w = csa(num_heads=2, head_dim=16, sliding_window_size=8, indexer=indexer(num_heads=2, top_k=4))")
    with pytest.raises(Exception, match="compress"):
        Model(compile_runs(src, filename="c.bux")[0].arch)


def _picked(indexer_cfg: str, t: int = 24, positions=None):
    """The keys a `gqa(indexer=...)` layer's indexer keeps for random inputs: (layer, picked, seen)."""
    from bux_b200.models.layers import attention as A
    from bux_b200.models.layers import sparse as S
    from bux_b200.models.registry import Context

    torch.manual_seed(0)
    attn = f"gqa(num_heads=4, num_kv_heads=2, rope=rope(), indexer={indexer_cfg})"
    tr = _train(attn)
    layer = [m for m in tr.model.modules() if isinstance(m, A.GQA)][0]
    x = torch.randn(1, t, 32)
    ids = torch.zeros(1, t, dtype=torch.long)
    if positions is None:
        ctx = Context(ids)
    else:
        pos = torch.tensor([positions])
        segments = (pos == 0).long().cumsum(-1)
        ctx = Context(ids, pos, segments)
    seen = S.seen_mask(ctx, t, None)
    with torch.no_grad():
        return layer, layer.indexer.pick(x, ctx, seen), seen, ctx


def test_indexer_blocks_are_counted_from_each_documents_first_key():
    from bux_b200.models.layers import sparse as S

    pos = torch.tensor([[0, 1, 2, 3, 4, 0, 1, 2, 3]])
    assert S.block_ids(pos, 4).tolist() == [[0, 0, 0, 0, 1, 2, 2, 2, 2]]
    values = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 9.0]]])
    assert S.per_block(values, S.block_ids(pos, 4), 3, "sum").tolist() == [[[10.0, 5.0, 30.0]]]
    assert S.per_block(values, S.block_ids(pos, 4), 3, "max").tolist() == [[[4.0, 5.0, 9.0]]]


def test_indexer_with_mean_pooled_blocks_keeps_whole_blocks_and_its_own_unfinished_one():
    """QSA: among the blocks a query sees all of it keeps the top_k // block_size best, whole;
    the keys of its own unfinished block are kept too."""
    _, picked, seen, _ = _picked("indexer(num_heads=2, head_dim=8, top_k=8, block_size=4, pool=mean)")
    kept = picked.kept[0]
    for q in range(24):
        own = q // 4
        rows = kept[q].view(6, 4)
        assert rows[own].tolist() == [k <= q % 4 for k in range(4)]         # its own block, as far as it sees
        finished = own + 1 if q % 4 == 3 else own                           # blocks the query sees all of
        whole = [b for b in range(finished) if rows[b].all()]
        partial = [b for b in range(own) if rows[b].any() and not rows[b].all()]
        assert not partial and len(whole) >= min(2, finished)               # two whole blocks of four
        assert not kept[q, q + 1:].any()
    assert picked.scores.shape[-1] == 6 and picked.block is not None        # the loss runs over blocks


def test_indexer_with_max_pooled_blocks_per_group():
    """MSA: each indexer head picks for one kv group; a block scores its best seen key; the
    query's own block is always among the top_k // block_size kept."""
    layer, picked, seen, ctx = _picked(
        "indexer(num_heads=2, head_dim=8, top_k=8, block_size=4, pool=max, per_group=true, weighted=false, relu=false)")
    kept = picked.kept[0]                                                   # [t, g, s]
    assert kept.shape == (24, 2, 24)
    for q in range(24):
        for g in range(2):
            rows = kept[q, g].view(6, 4)
            own = q // 4
            assert rows[own].tolist() == [k <= q % 4 for k in range(4)]
            others = [b for b in range(own) if rows[b].any()]
            assert all(rows[b].all() for b in others) and len(others) == min(1, own)
            if others:                                                      # the best of the other blocks
                best = picked.scores[0, q, g, : own * 4].view(own, 4).amax(-1)
                assert others[0] == int(best.argmax())
    assert not torch.equal(kept[:, 0], kept[:, 1])                          # the groups pick apart
    # attention runs per group over its own picks, and the loss is per group
    from bux_b200.models.layers import sparse as S
    q_, k_, v_ = torch.randn(1, 24, 4, 8), torch.randn(1, 24, 2, 8), torch.randn(1, 24, 2, 8)
    out, target = S.attend_kept(q_, k_, v_, picked.kept, None)
    assert target.shape == (1, 24, 2, 24) and torch.allclose(target.sum(-1), torch.full((1, 24, 2), 2.0))
    assert torch.isfinite(layer.indexer.loss(picked, target))


def test_indexer_blocks_stop_at_document_boundaries_and_train():
    positions = list(range(10)) + list(range(14))
    _, picked, seen, _ = _picked("indexer(num_heads=2, head_dim=8, top_k=8, block_size=4, pool=mean)", positions=positions)
    assert not (picked.kept & ~seen).any()
    assert not picked.kept[0, 10:, :10].any()                               # the second document sees none of the first
    for cfg in ("indexer(num_heads=2, head_dim=8, top_k=8, block_size=4, pool=mean)",
                "indexer(num_heads=1, head_dim=8, top_k=8, block_size=4, pool=max, per_group=true, weighted=false, relu=false)",
                "indexer(num_heads=1, head_dim=8, top_k=4, per_group=true, weighted=false)"):
        tr = _train(f"gqa(num_heads=2, num_kv_heads=1, rope=rope(), indexer={cfg})")
        ctx = tr.model(torch.randint(0, 64, (2, 32)), torch.arange(32).expand(2, 32), None, training=True)
        assert torch.isfinite(ctx.losses["indexer_loss"])


def test_norm_with_scale_input_puts_the_gain_before_the_statistics():
    """``rmsnorm(scale_input=true)``: norm(w * x), not norm(x) * w (reference: ``architecture/layers/norm.py:59-67``)."""
    import torch

    from bux_b200.config import layers as L
    from bux_b200.models.layers.basic import Norm

    torch.manual_seed(0)
    x = torch.randn(2, 5, 16)
    for kind in ("rmsnorm", "layernorm"):
        for zero_centered in (False, True):
            n = Norm(L.NormalizationConfig(type=kind, scale_input=True, zero_centered=zero_centered, bias=True), 16)
            with torch.no_grad():
                n.scale.copy_(torch.rand(16) + 0.5)
                n.bias.copy_(torch.randn(16))
            gain = 1 + n.scale if zero_centered else n.scale
            y = (x * gain).float()
            if kind == "layernorm":
                y = y - y.mean(-1, keepdim=True)
            want = y * torch.rsqrt(y.square().mean(-1, keepdim=True) + 1e-6) + n.bias
            assert torch.allclose(n(x), want, atol=1e-5), (kind, zero_centered)


def test_mlp_clips_soft_caps_and_drops_out_where_the_reference_does():
    """``mlp`` / ``gated_mlp``: the up branch clipped to +-limit then soft-capped, the gate capped from
    above only, the offset added after; dropout on the output (``architecture/layers/mlp.py:20-35,88`` there)."""
    import torch
    import torch.nn.functional as F

    from bux_b200.lang import compile
    from bux_b200.models import Model

    torch.manual_seed(0)
    x = torch.randn(2, 3, 16) * 3
    for kind in ("mlp", "gated_mlp"):
        arch = compile(f"d_model=16\nvocab_size=8\nf = {kind}(intermediate_size=32, activation=swish, limit=1.5, up_softcap=1.0"
                       + (", up_offset=1.0" if kind == "gated_mlp" else "") + ")\nmodel = embed [f] head\n", filename="m.bux")
        layer = Model(arch, dtype=torch.float32).graph.items[1].body
        if kind == "gated_mlp":
            h = x @ layer.gate_up.weight.t()
            gate, up = h[..., :32], h[..., 32:]
            up = torch.tanh(up.clamp(-1.5, 1.5) / 1.0) * 1.0
            want = (F.silu(gate.clamp(max=1.5)) * (up + 1.0)) @ layer.down.weight.t()
        else:
            up = torch.tanh((x @ layer.up.weight.t()).clamp(-1.5, 1.5))
            want = F.silu(up) @ layer.down.weight.t()
        assert torch.allclose(layer(x), want, atol=1e-5), kind
