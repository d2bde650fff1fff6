"""The trainer end to end on CPU: the smoke run, resume exactness, remat, schedules, data."""
import json

import numpy as np
import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.train import data, optim
from bux_b200.train.trainer import Trainer, directory, train
from test_lang import SMOKE


def test_smoke_trains_and_writes_the_run_directory(tmp_path):
    run = compile_runs(SMOKE, filename="smoke.bux")[0]
    tr = train(run, out=tmp_path, quiet=True)
    folder = directory(run, tmp_path)
    assert folder.name == "smoke-5a4f0f7d85"
    assert (folder / "run.bux").exists() and (folder / "run.json").exists()
    lines = [json.loads(l) for l in (folder / "metrics.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines] == [10, 20, 30, 40, 50]
    assert 6.0 < lines[-1]["loss"] < 6.5 and lines[-1]["lr"] == 0.0
    assert tr.model.num_params() == 155968


def test_learns_a_repeating_pattern():
    src = SMOKE.replace("steps     = 50", "steps = 60").replace("schedule  = wsd(warmup=10)", "")
    run = compile_runs(src, filename="s.bux")[0]
    tr = Trainer(run, device="cpu")
    ids = np.tile(np.arange(64, dtype=np.int32) % 7, (8, 1))
    batch = data.plain(ids)
    first = tr.train_step(batch)["loss"].item()
    for _ in range(40):
        last = tr.train_step(batch)["loss"].item()
    assert last < first * 0.3


def test_resume_is_exact(tmp_path):
    src = SMOKE.replace("steps     = 50", "steps = 12") + "checkpoint = checkpoint(every=6)\nlog = log(every=1)\n"
    src = src.replace("schedule  = wsd(warmup=10)", "schedule = wsd(warmup=2)")
    run = compile_runs(src, filename="r.bux")[0]
    full = train(run, out=tmp_path / "a", quiet=True)
    # the same run stopped after 6 steps, then resumed
    tr = train(run, out=tmp_path / "b", quiet=True, hooks=[_StopAt(6)])
    assert tr.step == 6
    resumed = train(run, out=tmp_path / "b", quiet=True)
    assert resumed.step == 12
    for (n, p), (_, q) in zip(full.model.named_parameters(), resumed.model.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n  # threaded CPU reductions are not bit-stable
    a = [json.loads(l) for l in (directory(run, tmp_path / "a") / "metrics.jsonl").read_text().splitlines()]
    b = [json.loads(l) for l in (directory(run, tmp_path / "b") / "metrics.jsonl").read_text().splitlines()]
    assert [x["step"] for x in a] == [x["step"] for x in b]
    assert [x["loss"] for x in a] == pytest.approx([x["loss"] for x in b], abs=1e-5)


class _StopAt:
    every = 1

    def __init__(self, step):
        self.at = step

    def start(self, trainer):
        pass

    def due(self, step, trainer, last=False):
        return True

    def __call__(self, step, scalars, trainer, sinks):
        if trainer.step >= self.at:
            trainer.stopping = True

    def stop(self, trainer, sinks):
        pass


def test_microbatches_match_the_whole_batch():
    # a large eps makes the update nearly linear in the gradient, so it can be compared
    opt = "optimizer = adamw(lr=3e-3, eps=1.0)"
    run1 = compile_runs(SMOKE, filename="s.bux", overrides=[opt])[0]
    run4 = compile_runs(SMOKE, filename="s.bux", overrides=[opt, "methods.microbatches = 4"])[0]
    a, b = Trainer(run1, device="cpu"), Trainer(run4, device="cpu")
    batch = next(iter(a.batches()))
    la, lb = a.train_step(batch), b.train_step(batch)
    assert abs(la["loss"].item() - lb["loss"].item()) < 1e-5
    for p, q in zip(a.model.parameters(), b.model.parameters()):
        assert torch.allclose(p, q, atol=1e-6)


def test_fused_optimizer_matches_on_the_first_step():
    run = compile_runs(SMOKE, filename="s.bux", overrides=["clip = none"])[0]
    a, b = Trainer(run, device="cpu"), Trainer(run, device="cpu", fuse_optimizer=True)
    batch = next(iter(a.batches()))
    a.train_step(batch)
    b.train_step(batch)
    for p, q in zip(a.model.parameters(), b.model.parameters()):
        assert torch.allclose(p, q, atol=1e-7)


def test_synthetic_rows_depend_only_on_seed_and_index():
    run = compile_runs(SMOKE, filename="s.bux")[0]
    whole = next(data.batches(run.train, 512, start=3))
    halves = [next(data.batches(run.train, 512, start=3, rank=r, world=2)) for r in range(2)]
    assert np.array_equal(whole.input_ids, np.concatenate([h.input_ids for h in halves]))
    rng = np.random.default_rng((0, 0, 0, 3 * 8))
    assert np.array_equal(whole.input_ids[0], rng.integers(0, 512, 64, np.int32))


def test_schedules():
    run = compile_runs(SMOKE, filename="s.bux")[0]
    m = optim.lr_multiplier(run.train)
    assert m(0) == pytest.approx(0.1) and m(9) == 1.0 and m(39) == 1.0 and m(49) == 0.0
    cos = compile_runs(SMOKE.replace("wsd(warmup=10)", "cosine(warmup=5, final=0.1)"))[0]
    m = optim.lr_multiplier(cos.train)
    assert m(4) == 1.0 and m(49) == pytest.approx(0.1)
    assert all(m(s) >= m(s + 1) for s in range(5, 49))


def test_newton_schulz_orthogonalises():
    g = torch.randn(32, 64)
    o = optim.newton_schulz(g, steps=8, dtype=torch.float32)
    s = torch.linalg.svdvals(o)
    assert s.max() < 1.3 and s.min() > 0.5


def test_muon_steps():
    run = compile_runs(SMOKE, filename="s.bux", overrides=["optimizer = muon(lr=0.02)"])[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    before = [p.clone() for p in tr.model.parameters()]
    tr.train_step(batch)
    assert any(not torch.equal(a, b) for a, b in zip(before, tr.model.parameters()))


def test_ema_ships_a_blend_and_observe_logs_per_layer_stats(tmp_path):
    import json

    from bux_b200.lang import compile_runs
    from bux_b200.train import ema
    from bux_b200.train.trainer import train

    src = SMOKE
    over = ["steps = 12", "schedule = constant", "ema = ema(window=4, blend=0.5)", "observe = observe(every=4, histograms=true)",
            "log = log(every=4)"]
    run = compile_runs(src, filename="smoke.bux", overrides=over)[0]
    assert ema.first(run.train.ema, 12) == 9
    tr = train(run, out=tmp_path, device="cpu", quiet=True)
    st = tr.optimizer.state
    name = next(n for n, _ in tr.model.named_parameters())
    assert "ema" in st[name]
    folder = next(tmp_path.iterdir())
    lines = [json.loads(x) for x in (folder / "metrics.jsonl").read_text().splitlines()]
    keys = set().union(*(set(x) for x in lines))
    assert any(k.startswith("param/") for k in keys) and any(k.startswith("update/") for k in keys)
    assert any(k.startswith("grad/") for k in keys)      # taken between the backward and the update
    assert any(k.startswith("act/graph") for k in keys)
    # the forward of an observed step files the stream and the attention under their branches
    for want in ("act/rms/gqa.00", "act/update_rms/gated_mlp.01", "act/max_abs/gqa.01", "act/kurtosis/gated_mlp.00",
                 "attn/logit_max/gqa.00", "attn/entropy/gqa.01"):
        assert want in keys, want
    observed = [x for x in lines if "act/rms/gqa.00" in x]
    assert [x["step"] for x in observed] == [4, 8, 12] and all(x["act/rms/gqa.00"] > 0 for x in observed)
    hist = [json.loads(x) for x in (folder / "histograms.jsonl").read_text().splitlines()]
    assert hist and hist[0]["step"] == 4 and sum(hist[0]["histograms"][name]) == tr.model.get_parameter(name).numel()
    assert sum(hist[0]["gradients"][name]) == tr.model.get_parameter(name).numel()      # the gradients' too
    assert sum(hist[0]["stream"]["act/hist/gqa.00"]) == 8 * 64 * 64      # batch x seq_len x d_model entries


def test_observe_files_the_routers_statistics():
    src = SMOKE.replace("ffn   = gated_mlp(intermediate_size=4 * d_model, activation=swish)",
                        "ffn   = moe(num_experts=4, top_k=2, load_balancing=aux_free, expert=gated_mlp(intermediate_size=32, activation=swish))")
    run = compile_runs(src, filename="smoke.bux", overrides=["steps = 4", "schedule = constant"])[0]
    tr = Trainer(run, device="cpu")
    tr.observing = {"histograms": False}
    tr.train_step(next(iter(tr.batches())))
    got = tr.observed
    for want in ("router/max_load/moe.00", "router/min_load/moe.01", "router/dead/moe.00", "router/entropy/moe.01",
                 "router/z/moe.00", "router/bias_std/moe.01", "act/rms/moe.00"):
        assert want in got, (want, sorted(got))
    assert 1.0 <= float(got["router/max_load/moe.00"]) <= 4.0 and float(got["router/dead/moe.00"]) == 0.0
    tr.observing = None
    tr.train_step(next(iter(tr.batches())))
    assert tr.observed is got            # an unobserved step files nothing new


def test_remat_auto_takes_the_cheapest_preset_that_fits():
    from bux_b200.train import fitting

    run = compile_runs(SMOKE, filename="smoke.bux")[0]
    tr = Trainer(run, device="cpu")
    peaks = {(False, False, False): 100, (True, True, False): 70, (True, False, False): 50, (True, False, True): 30}

    def probe(trainer, batch):
        rep = next(m for m in trainer.model.modules() if hasattr(m, "keep_attention"))
        p = peaks[(rep.remat, rep.keep_attention, rep.offload)]
        if p == 100:
            raise torch.OutOfMemoryError("no room")
        return p

    got = fitting.fit(tr, None, capacity=60, probe=probe)
    assert got.name == "block" and got.peak_bytes == 50
    assert [n for n, _ in got.tried] == ["none", "block, attention kept", "block"]
    with pytest.raises(MemoryError):
        fitting.fit(tr, None, capacity=10, probe=probe)


def test_profiler_commands():
    from bux_b200.train import profilers

    assert profilers.TOOLS["ncu"][1:3] == ["--clock-control", "none"]
    with pytest.raises(ValueError):
        profilers.command("torch", "out")
    with pytest.raises(ValueError):
        profilers.command("vtune", "out")
    if profilers.available("ncu"):
        cmd = profilers.command("ncu", "runs/x", argv=["-m", "bux_b200", "train", "f.bux"])
        assert cmd[0] == "ncu" and "runs/x/profile" in cmd and cmd[-4:] == ["-m", "bux_b200", "train", "f.bux"]


def test_prefix_token_prediction_weight_schedule_and_loss():
    """``loss(prefix=...)``: the weight holds, falls linearly, ends at zero; the term is the
    first head's cross-entropy of each target's prefix token where it has one."""
    import torch

    from bux_b200.config import training as T
    from bux_b200.data import tokenizer as TK
    from bux_b200.train import objective
    from bux_b200.train.trainer import Trainer

    c = T.PrefixConfig(weight=0.5, hold=0.25, decay=0.5)
    assert [objective.prefix_weight(c, s) for s in (0.0, 0.25, 0.5, 0.75, 0.9)] == [0.5, 0.5, 0.25, 0.0, 0.0]
    # the byte tokenizer's pieces are single bytes: none has a proper prefix
    assert (TK.prefix_tokens(TK.ByteTokenizer()) == -1).all()

    class Pieces:
        vocab_size = 6

        def token_pieces(self):
            return {0: b"a", 1: b"ab", 2: b"abc", 3: b"b", 4: b"bc", 5: b"abc"}

    assert TK.prefix_tokens(Pieces()).tolist() == [-1, 0, 1, -1, 3, 1]

    src = SMOKE.replace("schedule  = wsd(warmup=10)", "schedule  = constant").replace("steps     = 50", "steps     = 8\nloss = loss(prefix=prefix(weight=0.5, hold=0.5, decay=0.25))\n"
                        "tokenizer = tokenizer(name=\"bytes\")")
    run = compile_runs(src, filename="s.bux")[0]
    tr = Trainer(run, device="cpu")
    # every token's prefix is the token before it in the vocabulary (a made-up table)
    vocab = run.arch.vocab_size
    tr._prefixes = torch.arange(-1, vocab - 1)
    feed = iter(tr.batches())
    outs = [tr.train_step(next(feed)) for _ in range(8)]
    assert all("prefix_loss" in o for o in outs)
    first = outs[0]["prefix_loss"].item()
    assert 3.0 < first < 8.0   # near ln(vocab) at the start


def test_evaluation_reports_bits_per_byte_and_position_buckets():
    """`eval(positions=...)`: the loss over the targets of each bucket of positions, and bits
    per byte where a tokenizer says how many bytes a token stands for."""
    import math

    import torch

    from bux_b200.train.trainer import Trainer

    src = SMOKE + 'tokenizer = tokenizer(name="bytes")\neval = eval(data=synthetic, every=10, batches=2, positions=[16, 32])\n'
    run = compile_runs(src, filename="s.bux")[0]
    tr = Trainer(run, device="cpu")
    e = run.train.eval if not isinstance(run.train.eval, (tuple, list)) else run.train.eval[0]
    got = tr.evaluate(e)
    assert set(got) == {"eval_loss", "eval_bpb", "eval_loss_0", "eval_loss_16", "eval_loss_32",
                        "eval_bpb_0", "eval_bpb_16", "eval_bpb_32"}
    # buckets hold 16, 16 and 31 of a row's 63 targets: the loss is their weighted mean
    mean = (16 * got["eval_loss_0"] + 16 * got["eval_loss_16"] + 31 * got["eval_loss_32"]) / 63
    assert mean == pytest.approx(got["eval_loss"], rel=1e-5)
    # ids below 256 stand for one byte each under the byte tokenizer (the few above for none)
    assert got["eval_bpb"] == pytest.approx(got["eval_loss"] / math.log(2), rel=1e-2)


@pytest.mark.parametrize("remat", ["none", "full", "save_attention", "dots_attention", "offload_attention",
                                   "remat(save=[attention], first=1)"])
def test_remat_policies_train_the_same(remat):
    """What a policy keeps changes memory, not numbers: every policy's losses equal `none`'s."""
    def losses(policy):
        run = compile_runs(SMOKE, filename="s.bux", overrides=[f"methods.remat = {policy}", "steps = 20"])[0]
        tr = Trainer(run, device="cpu")
        feed = iter(tr.batches())
        return [tr.train_step(next(feed))["loss"].item() for _ in range(3)], tr

    want, _ = losses("none")
    got, tr = losses(remat)
    assert got == pytest.approx(want, abs=1e-5)
    from bux_b200.models.graph import Repeated

    rep = next(m for m in tr.model.modules() if isinstance(m, Repeated))
    assert rep.remat == (remat != "none")
    assert bool(rep.keep_attention) == (remat not in ("none", "full"))
    assert rep.first == (1 if "first" in remat else None)


PRECISION_SRC = """
d_model=64
vocab_size=64
n = rmsnorm
block = [n gqa(num_heads=2, num_kv_heads=1, rope=rope())] [n gated_mlp(intermediate_size=128, activation=swish)]
model = embed block^3 n head
data = synthetic
optimizer = adamw(lr=1e-3)
seq_len = 32
batch = 2
steps = 10
precision = precision(compute=float32{more})
"""


def _logits(more: str, step: int = 0):
    run = compile_runs(PRECISION_SRC.format(more=more), filename="p.bux")[0]
    tr = Trainer(run, device="cpu")
    tr.step = step
    batch = tr.to_device(next(iter(tr.batches())))
    loss, _ = tr.forward_loss(batch, 1.0 / batch[0].numel(), 1, 1)
    return tr, loss.item()


def test_precision_first_and_last_keep_edge_branches_in_the_compute_dtype():
    from bux_b200.models.graph import count_outer_branches

    tr, plain = _logits("")
    assert count_outer_branches(tr.model.graph) == 6
    _, low = _logits(", matmuls=mxfp8")
    assert low != plain
    _, edges = _logits(", matmuls=mxfp8, first=2, last=4")          # every branch is at an edge
    assert edges == plain
    _, shares = _logits(", matmuls=mxfp8, first=0.5, last=0.5")
    assert shares == plain
    _, some = _logits(", matmuls=mxfp8, first=2")
    assert some != plain and some != low


def test_precision_passes_switch_and_eval():
    _, plain = _logits("")
    _, low = _logits(", matmuls=mxfp8")
    _, none = _logits(", matmuls=mxfp8, passes=[]")
    assert none == plain
    # a switch takes over from a share of the steps on
    _, before = _logits(", matmuls=mxfp8, switch=switch(at=0.5, passes=[])", step=4)
    _, after = _logits(", matmuls=mxfp8, switch=switch(at=0.5, passes=[])", step=5)
    assert before == _logits(", matmuls=mxfp8", step=4)[1] and after == _logits("", step=5)[1]
    # eval=compute evaluates without the low-precision matmuls
    src = PRECISION_SRC.format(more=", matmuls=mxfp8, eval=compute") + "eval = eval(data=synthetic, every=5, batches=2)\n"
    run = compile_runs(src, filename="p.bux")[0]
    tr = Trainer(run, device="cpu")
    e = run.train.eval if not isinstance(run.train.eval, (tuple, list)) else run.train.eval[0]
    in_compute = tr.evaluate(e)
    assert tr.precision.enabled
    tr.train.precision.__dict__["eval"] = "train"
    as_trained = tr.evaluate(e)
    assert in_compute != as_trained


def test_flops_per_token_match_a_count_of_the_products_that_run():
    """The analytic count against torch's FLOP counter over a forward and a backward on CPU
    (which counts every matrix product that actually ran), and its rules for masks."""
    import numpy as np
    from torch.utils.flop_counter import FlopCounterMode

    from bux_b200.train import flops as F

    src = """
d_model=128
vocab_size=256
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, rope=rope())
e = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=64, activation=swish), num_shared_experts=1)
block = [n a] [n gated_mlp(intermediate_size=256, activation=swish)] [n e]
model = embed block^2 n head(tied=false)
data = synthetic
optimizer = adamw(lr=1e-3)
seq_len = 32
batch = 4
steps = 1
precision = precision(compute=float32)
"""
    run = compile_runs(src, filename="f.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    with FlopCounterMode(display=False) as counter:
        tr.train_step(batch)
    measured = counter.get_total_flops() / (4 * 32)
    analytic = F.flops_per_token(run.arch, 32)
    # the eager statement of attention multiplies the whole square (the analytic count stops at
    # the diagonal) and the experts' reference path pads; everything else is the same products
    square = 3 * 2 * 2.0 * 4 * (32 + 32) * (32 - (32 + 1) / 2)
    assert measured == pytest.approx(analytic + square, rel=0.08), (measured, analytic, square)

    assert F.keys_seen(8) == 4.5 and F.keys_seen(8, window=2) == (1 + 2 * 7) / 8
    packed = np.array([[0, 1, 2, 3, 0, 1, 0, 0]])          # documents of 4, 2, 1, 1 tokens
    assert F.keys_seen(8, positions=packed) == (1 + 2 + 3 + 4 + 1 + 2 + 1 + 1) / 8
    assert F.flops_per_token(run.arch, 32, positions=np.zeros((1, 32), int)) < F.flops_per_token(run.arch, 32)
    sparse = compile_runs(src.replace("rope=rope())", "rope=rope(), indexer=indexer(num_heads=2, head_dim=16, top_k=4))"), filename="f.bux")[0]
    long = F.flops_per_token(sparse.arch, 4096) / F.flops_per_token(run.arch, 4096)
    assert long < 1.0           # picks cap the attended keys; the scorer costs less than it saves


def test_trace_reader_splits_communication_from_compute_per_device(tmp_path):
    """A hand-written chrome trace: communication under compute is hidden, beside it exposed;
    one GPU's collective does not hide under another GPU's compute."""
    from bux_b200.train import trace

    def k(name, ts, dur, device):
        return {"ph": "X", "cat": "kernel", "name": name, "ts": ts, "dur": dur, "args": {"device": device}}

    events = [k("gemm_sm100_kernel", 0, 1000, 0), k("ncclDevKernel_AllGather", 500, 1000, 0),   # 500 hidden, 500 exposed
              k("attn_fwd_kernel", 2000, 1000, 0),                                                # 500 idle before it
              k("ep_push_rows_mx", 0, 800, 1), k("gemm_sm100_kernel", 1000, 2000, 1),             # all 800 exposed, 200 idle
              {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5000}]
    path = tmp_path / "profile" / "host0.json"
    path.parent.mkdir()
    path.write_text(json.dumps({"traceEvents": events}))
    got = trace.comm_ms(path, steps=1)
    assert got["comm_ms"] == pytest.approx((1.0 + 0.8) / 2) and got["exposed_comm_ms"] == pytest.approx((0.5 + 0.8) / 2)
    assert got["idle_ms"] == pytest.approx((0.5 + 0.2) / 2)
    assert trace.comm_ms(path, steps=2)["comm_ms"] == pytest.approx(0.45)
    top = trace.kernels(path)
    assert top[0][0] == "gemm_sm100_kernel" and top[0][1] == 2 and top[0][2] == pytest.approx(3.0)
    assert trace.latest(tmp_path) == path and trace.latest(tmp_path, host="host9") is None


INTERLEAVED = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope(), value_residual=learned)
e = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish), aux_loss_coef=0.01)
first = [n a(v=@v)] [n e]
rest = [n a(v=$v)] [n e]
model = embed first @skip rest^3 [$skip! scale] n head
data = synthetic
optimizer = adamw(lr=1e-2, eps=1.0)
seq_len = 16
batch = 8
steps = 4
precision = precision(compute=float32)
methods = methods(microbatches=4{more})
"""


@pytest.mark.parametrize("remat", ["none", "full"])
def test_interleaved_microbatches_give_the_gradients_of_a_plain_accumulation(remat):
    """``methods(interleave=true)``: the forward of each microbatch runs piece by piece beside the
    backward of the one before. A graph with a tap read three pieces later, a port that feeds
    every later attention and auxiliary losses: what crosses pieces crosses them as always."""
    from bux_b200.train import interleave

    plain = compile_runs(INTERLEAVED.format(more=f", remat={remat}"), filename="i.bux")[0]
    mixed = compile_runs(INTERLEAVED.format(more=f", remat={remat}, interleave=true"), filename="i.bux")[0]
    a, b = Trainer(plain, device="cpu"), Trainer(mixed, device="cpu")
    order: list = []
    pieces = interleave.pieces_of(b.model)
    assert len(pieces) == 9     # embed, first, the tap, three passes of rest, the skip's branch, norm, head
    for t, m in enumerate(pieces):
        m.register_forward_hook(lambda mod, args, out, t=t: order.append(("F", t)) if torch.is_grad_enabled() else None)
        m.register_full_backward_hook(lambda mod, gi, go, t=t: order.append(("B", t)))
    feed = iter(a.batches())
    for _ in range(2):
        batch = next(feed)
        la, lb = a.train_step(batch), b.train_step(batch)
        assert la["loss"].item() == pytest.approx(lb["loss"].item(), abs=1e-6)
        assert la["grad_norm"].item() == pytest.approx(lb["grad_norm"].item(), rel=1e-5)
    for (name, p), q in zip(a.model.named_parameters(), b.model.parameters()):
        assert torch.allclose(p, q, atol=1e-6), name
    sched = b._interleave
    assert sched and sched.ticks >= 2 * 3 * len(pieces) - 6      # two steps, three overlapped pairs each
    if remat == "none":
        # inside an overlapped pair the two halves alternate: a forward piece, then a backward piece
        first_b = next(i for i, (kind, _) in enumerate(order) if kind == "B")
        window = order[first_b - 1:first_b + 9]
        assert [k for k, _ in window] == ["F", "B"] * 5, window
        back = [t for k, t in window if k == "B"]
        assert back == list(range(back[0], back[0] - 5, -1)) and back[0] >= 7       # the top pieces first, one a tick


def test_interleave_falls_back_where_it_cannot_run():
    from bux_b200.train import interleave

    run = compile_runs(INTERLEAVED.format(more=", interleave=true"), filename="i.bux")[0]
    tr = Trainer(run, device="cpu", fuse_optimizer=True)
    assert "fused into the backward" in interleave.unsupported(tr)
    with pytest.warns(UserWarning, match="one after another"):
        tr.train_step(next(iter(tr.batches())))
    co = interleave.Coroutine(lambda: (_ for _ in ()).throw(ValueError("inside")), "t")
    with pytest.raises(ValueError, match="inside"):
        co.resume()
    assert not co.resume()


@pytest.mark.parametrize("model", [
    "embed first rest^3 n head",                      # written outside every checkpointed block, read inside three
    "embed first^1 @t rest^2 [$t! scale] n head",     # written inside one checkpointed pass, read inside later ones
    "embed (first @t rest [$t! scale])^2 n head",     # written and read inside one pass
])
def test_checkpointed_blocks_pass_gradients_through_taps_and_ports(model):
    """``remat=full`` reruns a block in the backward. What the block reads from taps other layers
    wrote, and what it writes for later readers, crosses the checkpoint as inputs and outputs of
    the rerun: the gradients are those of a run that keeps everything."""
    src = INTERLEAVED.replace("model = embed first @skip rest^3 [$skip! scale] n head", "model = " + model)
    got = {}
    for remat in ("none", "full"):
        run = compile_runs(src.format(more=f", remat={remat}"), filename="r.bux")[0]
        tr = Trainer(run, device="cpu")
        out = tr.train_step(next(iter(tr.batches())))
        got[remat] = (out["loss"].item(), {n: p.detach().clone() for n, p in tr.model.named_parameters()})
    assert got["none"][0] == pytest.approx(got["full"][0], abs=1e-6)
    for name, p in got["none"][1].items():
        assert torch.allclose(p, got["full"][1][name], atol=1e-6), name


def test_parameters_their_layers_exempt_skip_weight_decay_and_muon():
    """The 2-D parameters that are not matrices of a linear map (RWKV-7's shift mixes and bonus
    keys, Mamba's decay rates, value-embedding and token tables) are marked where the optimizer
    looks: no weight decay for the first three, AdamW instead of Muon for the tables and the head
    (reference: ``recurrent/rwkv7.py:76``, ``recurrent/ssm.py:182,267``, ``layers/embedding.py:60,142,197``)."""
    import torch

    from bux_b200.lang import compile
    from bux_b200.models import Model
    from bux_b200.train import optim

    src = ("d_model=32\nvocab_size=64\nn = rmsnorm\nt = rwkv7(num_heads=2, head_dim=16)\n"
           "s = mamba(state_size=4)\ns2 = mamba2(num_heads=2, head_dim=16, state_size=8)\n"
           "a = gqa(num_heads=2, num_kv_heads=1, rope=rope(), ve=$ve!)\n"
           "f = gated_mlp(intermediate_size=48, activation=swish)\n"
           "model = embed value_embed(features=16, ve=@ve) [n a] [n t] [n s] [n s2] [n f] n head\n")
    arch = compile(src, filename="m.bux")
    model = Model(arch, dtype=torch.float32)
    seen = set()
    for name, p in model.named_parameters():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("shift", "r_k", "A_log"):
            seen.add(leaf)
            assert not optim.weight_decay_mask(name, p), name
        if p.ndim >= 2 and (".embed" in "." + name or "head" in name or "tokens" in name or "table" in name):
            assert not optim.muon_eligible(name, p), name
    assert seen == {"shift", "r_k", "A_log"}
    mats = [n for n, p in model.named_parameters() if optim.muon_eligible(n, p)]
    assert any("gate_up" in n for n in mats) and all(optim.weight_decay_mask(n, dict(model.named_parameters())[n]) for n in mats)
