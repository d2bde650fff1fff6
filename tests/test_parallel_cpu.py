"""Multi-rank logic on CPU: gloo ranks spawned as processes, compared with one rank."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bux_b200.lang import compile_runs

MOE = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=2, num_kv_heads=1, rope=rope())
e = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish))
block = [n a] [n e]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-2, eps=1.0)
seq_len = 16
batch = 8
steps = 4
precision = precision(compute=float32)
"""


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, src, overrides, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.set_num_threads(1)
    run = compile_runs(src, filename="p.bux", overrides=overrides)[0]
    par = Parallel(run.train, torch.device("cpu"))
    tr = Trainer(run, device="cpu", parallel=par)
    feed = iter(tr.batches())
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    if rank == 0:
        torch.save({"losses": losses, "state": state}, out)
    dist.barrier()
    dist.destroy_process_group()


def _single(src, overrides=()):
    from bux_b200.train.trainer import Trainer

    run = compile_runs(src, filename="p.bux", overrides=list(overrides))[0]
    tr = Trainer(run, device="cpu")
    feed = iter(tr.batches())
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    return losses, {n: p.detach().clone() for n, p in tr.model.named_parameters()}


def _spawn(world, src, overrides, tmp_path):
    out = str(tmp_path / "rank0.pt")
    mp.spawn(_worker, args=(world, _free_port(), src, list(overrides), out), nprocs=world, join=True)
    return torch.load(out)


def test_data_parallel_matches_one_rank(tmp_path):
    want_losses, want = _single(MOE)
    got = _spawn(2, MOE, ["mesh = mesh(data=2)"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=1e-5), name


def test_expert_parallel_matches_one_rank(tmp_path):
    want_losses, want = _single(MOE)
    got = _spawn(2, MOE, ["mesh = mesh(expert=2)", "methods.moe = all_to_all", "methods.capacity = 4.0"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    # rank 0 holds the first half of the experts, and the first rows of every other
    # parameter: what is not an expert is sharded over the expert axis like over `fsdp`
    _check_rows(got, want)
    assert any(got["state"][n].shape != p.shape for n, p in want.items() if "experts_" not in n)


def _check_rows(got, want, world=2):
    """Rank 0 holds the first rows of every sharded parameter."""
    for name, p in want.items():
        g = got["state"][name]
        if g.shape != p.shape:
            p = p[: g.shape[0]]
        assert torch.allclose(g, p, atol=1e-5), name


@pytest.mark.parametrize("extra", [
    [],                                   # ZeRO-3: gather per block
    ["methods.remat = full"],             # ... and again in the replay of each block
    ["layout = layout(zero=1)"],          # whole parameters for the step, sharded optimizer state
    ["methods.microbatches = 2"],
    ["methods.microbatches = 2", "methods.accumulate = unreduced"],                          # one reduce-scatter per step
    ["methods.microbatches = 2", "methods.accumulate = unreduced", "methods.remat = full"],
    ["methods.microbatches = 2", "methods.accumulate = unreduced", "methods.gather = step"],
])
def test_fsdp_matches_one_rank(tmp_path, extra):
    base = [e for e in extra if "microbatches" in e]
    want_losses, want = _single(MOE, base)
    got = _spawn(2, MOE, ["mesh = mesh(fsdp=2)", *extra], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    _check_rows(got, want)
    assert any(got["state"][n].shape != p.shape for n, p in want.items())  # something was sharded


def test_hsdp_matches_one_rank(tmp_path):
    want_losses, want = _single(MOE)
    got = _spawn(4, MOE, ["mesh = mesh(data=2, fsdp=2)"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    _check_rows(got, want)


DENSE = MOE.replace("e = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish))",
                    "e = gated_mlp(intermediate_size=48, activation=swish)")


def _tensor_worker(rank, world, port, src, overrides, out):
    """Like `_worker`, but rank 0 saves whole tensors (gathered over the tensor axis)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bux_b200.ckpt.store import state_tree
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.set_num_threads(1)
    run = compile_runs(src, filename="p.bux", overrides=overrides)[0]
    par = Parallel(run.train, torch.device("cpu"))
    tr = Trainer(run, device="cpu", parallel=par)
    feed = iter(tr.batches())
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    tree = par.checkpoint_tree(tr, state_tree)
    if rank == 0:
        torch.save({"losses": losses, "state": tree["0"]}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("src,extra", ids=["dense", "moe", "dense-sp", "moe-sp"], argvalues=[
    (DENSE, []),
    (MOE, []),
    (DENSE, ["layout = layout(stream=tensor)"]),
    (MOE.replace("optimizer = adamw", "loss = loss(); optimizer = adamw"), ["layout = layout(stream=tensor)"]),
])
def test_tensor_parallel_matches_one_rank(tmp_path, src, extra):  # noqa: D103
    src = src.replace("model = embed block^2 n head", "model = embed block^2 n head(tied=false)")
    src = src.replace("num_heads=2, num_kv_heads=1", "num_heads=4, num_kv_heads=2, qk_norm=rmsnorm")
    want_losses, want = _single(src)
    out = str(tmp_path / "rank0.pt")
    mp.spawn(_tensor_worker, args=(2, _free_port(), src, ["mesh = mesh(tensor=2)", *extra], out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=1e-5), name


def test_schedule_tables_are_valid():
    from bux_b200.parallel import schedule as S

    for name, make in S.TABLES.items():
        for stages, micro in [(2, 2), (2, 4), (4, 4), (4, 8), (3, 5)]:
            table = make(stages, micro)
            S.check(table, micro)
            if name in ("1f1b", "zbh1"):  # stage s keeps at most S - s microbatches alive
                assert all(S.alive(ops) <= stages - s for s, ops in enumerate(table))
    assert S.bubble(4, 8) == pytest.approx(3 / 11)
    assert S.bubble(1, 8) == 0.0


def test_pipeline_shares_balance_the_stages():
    from bux_b200.parallel.pipeline import shares

    assert shares([1.0] * 8, 4) == [2, 2, 2, 2]
    assert shares([1.0] * 8, 2, last_extra=2.0) == [5, 3]
    assert sum(shares([1.0, 3.0, 1.0, 1.0, 2.0], 3)) == 5


@pytest.mark.parametrize("method", ["gpipe", "1f1b", "zbh1"])
def test_pipeline_matches_one_rank(tmp_path, method):
    src = DENSE.replace("model = embed block^2 n head", "model = embed block^4 n head(tied=false)")
    over = ["methods.microbatches = 4"]
    want_losses, want = _single(src, over)
    out = str(tmp_path / "rank0.pt")
    mp.spawn(_tensor_worker, args=(2, _free_port(), src, ["mesh = mesh(stage=2)", f"methods.pipeline = \"{method}\"", *over], out),
             nprocs=2, join=True)
    got = torch.load(out)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    assert set(got["state"]) >= set(want)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=1e-5), name


@pytest.mark.parametrize("method,heads", [("ulysses", "num_heads=4, num_kv_heads=2"),
                                          ("gathered", "num_heads=4, num_kv_heads=2"),
                                          ("auto", "num_heads=2, num_kv_heads=1"),
                                          ("ring", "num_heads=4, num_kv_heads=2")])
def test_context_parallel_matches_one_rank(tmp_path, method, heads):
    src = DENSE.replace("num_heads=2, num_kv_heads=1", heads)
    want_losses, want = _single(src)
    got = _spawn(2, src, ["mesh = mesh(context=2)", f"methods.attention = {method}"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=1e-5), name


@pytest.mark.parametrize("how", ["gather", "owner"])
def test_muon_on_fsdp_shards_matches_one_rank(tmp_path, how):
    src = DENSE.replace("optimizer = adamw(lr=1e-2, eps=1.0)", "optimizer = muon(lr=1e-2, ns_dtype=float32)")
    want_losses, want = _single(src)
    got = _spawn(2, src, ["mesh = mesh(fsdp=2)", f"methods.orthogonalize = {how}"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    _check_rows(got, want)


# ------------------------------------------------------------------ resume on a sharded mesh
def _resume_worker(rank, world, port, src, overrides, folder, out):
    """Two steps, a checkpoint, a fresh trainer restored from it, two more steps; and the
    same four steps without the interruption."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bux_b200 import ckpt
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.set_num_threads(1)
    run = compile_runs(src, filename="p.bux", overrides=overrides)[0]

    def fresh():
        par = Parallel(run.train, torch.device("cpu"))
        return Trainer(run, device="cpu", parallel=par)

    whole = fresh()
    feed = iter(whole.batches())
    straight = [whole.train_step(next(feed))["loss"].item() for _ in range(4)]
    first = fresh()
    feed = iter(first.batches())
    resumed = [first.train_step(next(feed))["loss"].item() for _ in range(2)]
    ckpt.save(folder, first.step, first)
    second = fresh()
    ckpt.load(os.path.join(folder, str(first.step)), second)
    assert second.step == 2
    feed = iter(second.batches())
    resumed += [second.train_step(next(feed))["loss"].item() for _ in range(2)]
    if rank == 0:
        torch.save({"straight": straight, "resumed": resumed}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mesh,extra", [
    (2, "mesh(fsdp=2)", []),
    (2, "mesh(expert=2)", ["methods.moe = all_to_all", "methods.capacity = 4.0"]),
    (2, "mesh(tensor=2)", ["a = gqa(num_heads=2, num_kv_heads=2, rope=rope())"]),
    (2, "mesh(stage=2)", ["methods.microbatches = 2", "model = embed block^2 n head(tied=false)"]),
    (4, "mesh(fsdp=2, tensor=2)", ["a = gqa(num_heads=2, num_kv_heads=2, rope=rope())"]),
])
def test_resume_on_a_sharded_mesh_matches_the_uninterrupted_run(tmp_path, world, mesh, extra):
    out = str(tmp_path / "r.pt")
    folder = str(tmp_path / "ckpt")
    os.makedirs(folder)
    mp.spawn(_resume_worker, args=(world, _free_port(), MOE, [f"mesh = {mesh}", *extra], folder, out),
             nprocs=world, join=True)
    got = torch.load(out)
    assert got["resumed"][:2] == pytest.approx(got["straight"][:2], abs=1e-6)
    assert got["resumed"][2:] == pytest.approx(got["straight"][2:], abs=1e-5)


def test_blockwise_context_parallel_over_four_ranks(tmp_path):
    """`ring` with four ranks: every rank works on two half-chunks of the zigzag placement."""
    src = DENSE.replace("num_heads=2, num_kv_heads=1", "num_heads=4, num_kv_heads=2")
    want_losses, want = _single(src)
    got = _spawn(4, src, ["mesh = mesh(context=4)", "methods.attention = ring"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=1e-5)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=1e-5), name


def test_experts_are_built_as_the_ranks_shard():
    """Under `placement.placing` a MoE layer keeps this rank's experts only, with the values a
    whole build draws for them (and every other parameter unchanged)."""
    from bux_b200.lang import compile_runs
    from bux_b200.models import Model, placement

    run = compile_runs(MOE, filename="t.bux")[0]
    whole = Model(run.arch, seed=3)
    with placement.placing(experts=(1, 2)):
        mine = Model(run.arch, seed=3)
    want = dict(whole.named_parameters())
    for name, p in mine.named_parameters():
        if "experts_" in name:
            assert p.shape[0] == 2 and p.placed_rows == slice(2, 4)
            assert torch.equal(p, want[name][2:4])
        else:
            assert torch.equal(p, want[name])


def _packed_cp_worker(rank, world, port, method, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bux_b200.ops import functional as ops
    from bux_b200.parallel import context

    torch.manual_seed(0)
    b, t, h, g, d = 2, 16, 4, 2, 8
    q, k, v = torch.randn(b, t, h, d), torch.randn(b, t, g, d), torch.randn(b, t, g, d)
    go = torch.randn(b, t, h, d)
    segments = torch.tensor([[1] * 5 + [2] * 6 + [3] * 5, [1] * 9 + [2] * 7])   # documents cross the ranks' boundary
    per = t // world
    mine = slice(rank * per, (rank + 1) * per)
    ql, kl, vl = (x[:, mine].clone().requires_grad_() for x in (q, k, v))
    o = context.attend(ops.attention, ql, kl, vl, dist.group.WORLD, method, causal=True, segments=segments[:, mine])
    o.backward(go[:, mine])
    parts = [None] * world
    dist.all_gather_object(parts, (o.detach(), ql.grad, kl.grad, vl.grad))
    if rank == 0:
        torch.save([torch.cat([part[i] for part in parts], dim=1) for i in range(4)], out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("method", ["ulysses", "gathered", "ring"])
def test_context_parallel_of_packed_rows(tmp_path, method):
    """Rows of several documents split by position over two ranks: attention stays inside a
    document on every method (ulysses: whole rows per head; the others: my queries against the
    gathered keys with both sides' document ids)."""
    from bux_b200.ops import reference as ref

    out = str(tmp_path / "o.pt")
    mp.spawn(_packed_cp_worker, args=(2, _free_port(), method, out), nprocs=2, join=True)
    torch.manual_seed(0)
    b, t, h, g, d = 2, 16, 4, 2, 8
    q, k, v = (x.requires_grad_() for x in (torch.randn(b, t, h, d), torch.randn(b, t, g, d), torch.randn(b, t, g, d)))
    go = torch.randn(b, t, h, d)
    segments = torch.tensor([[1] * 5 + [2] * 6 + [3] * 5, [1] * 9 + [2] * 7])
    want, _ = ref.attention(q, k, v, causal=True, segments=segments)
    want.backward(go)
    got = torch.load(out)
    for a, w in zip(got, (want.detach(), q.grad, k.grad, v.grad)):
        assert torch.allclose(a, w, atol=1e-5)


def test_merge_by_lse_equals_attention_over_the_union():
    from bux_b200.ops import reference as ref
    from bux_b200.parallel.context import merge_by_lse

    torch.manual_seed(0)
    q = torch.randn(2, 8, 4, 16)
    k = torch.randn(2, 24, 2, 16)
    v = torch.randn(2, 24, 2, 16)
    want, want_lse = ref.attention(q, k, v, causal=False)
    parts = [ref.attention(q, k[:, s:s + 8], v[:, s:s + 8], causal=False) for s in (0, 8, 16)]
    got, lse = merge_by_lse([p[0] for p in parts], [p[1] for p in parts])
    assert torch.allclose(got, want, atol=1e-5) and torch.allclose(lse, want_lse, atol=1e-5)


RECURRENT = """
d_model=32
vocab_size=64
n = rmsnorm
mixer = {mixer}
m = gated_mlp(intermediate_size=48, activation=swish)
block = [n mixer] [n m]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-2, eps=1.0)
seq_len = 160
batch = 4
steps = 3
precision = precision(compute=float32)
"""


@pytest.mark.parametrize("mixer", [
    "gdn(num_heads=2, head_dim=8, num_v_heads=4, v_head_dim=8)",      # delta rule, a decay per head, short convs
    "kda(num_heads=2, head_dim=8)",                                   # a decay per key channel
    "gla(num_heads=2, head_dim=8)",                                   # no rank-one term
    "rwkv7(num_heads=2, head_dim=8, decay_rank=4, a_rank=4, v_rank=4, gate_rank=4)",   # token shift
    "mamba2(state_size=8, head_dim=8, conv_size=3)",
    "short_conv()",
])
def test_recurrent_mixers_under_context_parallelism(tmp_path, mixer):
    """Positions split over two ranks: the state (and the convolutions' last positions) are
    handed from the first rank to the second; losses and parameters equal one rank's."""
    src = RECURRENT.format(mixer=mixer)
    want_losses, want = _single(src)
    got = _spawn(2, src, ["mesh = mesh(context=2)"], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=2e-5)
    for name, p in want.items():
        assert torch.allclose(got["state"][name], p, atol=2e-5), name


def _node_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      BUX_NODE_NAME=f"node{rank // 2}")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import warnings

    from bux_b200 import runtime
    from bux_b200.parallel.experts import ExpertParallel

    pair = None
    for ranks in ([0, 1], [2, 3]):
        g = dist.new_group(ranks)
        if rank in ranks:
            pair = g
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        across = ExpertParallel(dist.group.WORLD, "fused_ep")
        inside = ExpertParallel(pair, "fused_ep")
    if rank == 0:
        torch.save({"world": runtime.on_one_node(dist.group.WORLD), "pair": runtime.on_one_node(pair),
                    "across": across.method, "inside": inside.method,
                    "warned": [str(w.message) for w in caught]}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_peer_memory_paths_are_for_one_machine(tmp_path):
    """Four ranks that say they run on two machines: the in-kernel expert exchange is kept for a
    group inside one machine and gives way to NCCL's all-to-all for a group across them."""
    out = str(tmp_path / "n.pt")
    mp.spawn(_node_worker, args=(4, _free_port(), out), nprocs=4, join=True)
    got = torch.load(out)
    assert got["pair"] is True and got["world"] is False
    assert got["inside"] == "fused_ep" and got["across"] == "all_to_all"
    assert len(got["warned"]) == 1 and "spans machines" in got["warned"][0]


def _shared_worker(rank, world, port, folder, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from pathlib import Path

    from bux_b200 import runtime

    one = runtime.shared(Path(folder) / "one")                    # the same folder for every rank
    own = runtime.shared(Path(folder) / f"host{rank % 2}")        # two "hosts", each with its own
    refused = False
    try:
        runtime.agree_on_folder(Path(folder) / f"host{rank % 2}")
    except ValueError:
        refused = True
    runtime.build_in_turn()                                       # no rank compiles beside another
    left = sorted(p.name for p in (Path(folder) / "one").iterdir())
    got = [None] * world
    dist.all_gather_object(got, (one, own, refused, left))
    if rank == 0:
        torch.save(got, out)
    dist.barrier()
    dist.destroy_process_group()


def test_ranks_agree_on_whether_a_folder_is_shared(tmp_path):
    """`runtime.shared`: the first rank drops a file, the others must list it; the ranks talk
    through the job's key-value store. A folder only some ranks see is refused for run output."""
    out = str(tmp_path / "r.pt")
    mp.spawn(_shared_worker, args=(3, _free_port(), str(tmp_path), out), nprocs=3, join=True)
    got = torch.load(out)
    assert all(one is True and own is False and refused for one, own, refused, _ in got)
    assert all(left == [] for *_, left in got)                    # the marker is removed again


def _shard_writer(rank, world, port, folder, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import json
    from pathlib import Path

    from bux_b200 import ckpt
    from bux_b200.ckpt import store
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.set_num_threads(1)
    run = compile_runs(MOE, filename="p.bux", overrides=["mesh = mesh(fsdp=2)"])[0]
    tr = Trainer(run, device="cpu", parallel=Parallel(run.train, torch.device("cpu")))
    feed = iter(tr.batches())
    tr.train_step(next(feed))
    mine = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    ckpt.save(folder, tr.step, tr, background=True)
    tr.train_step(next(feed))          # training goes on while the files are written
    ckpt.wait()
    root = Path(folder) / "1" / "default"
    name = next(n for n in tr.parallel.fsdp.sharded)
    leaf = root / "0" / name.replace(".", "/")
    meta = json.loads((leaf / "zarr.json").read_text())
    chunks = sorted(p.relative_to(leaf / "c").as_posix() for p in (leaf / "c").rglob("*") if p.is_file())
    rows = meta["shape"][0] // world
    part = store.read_array(leaf, (rank * rows, (rank + 1) * rows))
    ragged = store.read_array(leaf, (rows - 1, rows + 2))            # rows of two chunks
    whole = store.read_array(leaf)
    got = [None] * world
    dist.all_gather_object(got, {
        "chunk_rows": meta["chunk_grid"]["configuration"]["chunk_shape"][0], "rows": rows, "chunks": chunks,
        "saved_is_the_first_step": bool(torch.equal(part, mine[name].float())),
        "ragged": bool(torch.equal(ragged, whole[rows - 1:rows + 2])),
        "no_tmp": not any(p.name.endswith("tmp") for p in Path(folder).iterdir())})
    if rank == 0:
        torch.save(got, out)
    dist.barrier()
    dist.destroy_process_group()


def test_every_rank_writes_its_own_rows_of_a_checkpoint_in_the_background(tmp_path):
    """A sharded leaf is one array whose chunks are the ranks' rows, each written by the rank
    that holds it while training goes on; a rank reads back only the rows it keeps; what was
    saved is the state of the step it was saved at, not of the steps that ran meanwhile."""
    out = str(tmp_path / "r.pt")
    os.makedirs(tmp_path / "ckpt")
    mp.spawn(_shard_writer, args=(2, _free_port(), str(tmp_path / "ckpt"), out), nprocs=2, join=True)
    for r in torch.load(out):
        assert r["chunk_rows"] == r["rows"] and len(r["chunks"]) == 2 and r["chunks"][0].startswith("0") and r["chunks"][1].startswith("1")
        assert r["saved_is_the_first_step"] and r["ragged"] and r["no_tmp"]


def test_a_failed_background_save_is_raised_by_the_next_wait(tmp_path, monkeypatch):
    from bux_b200 import ckpt
    from bux_b200.ckpt import store
    from bux_b200.train.trainer import Trainer

    run = compile_runs(MOE, filename="p.bux")[0]
    tr = Trainer(run, device="cpu")

    def refuse(*a, **k):
        raise OSError("disk full")

    monkeypatch.setattr(store, "write_tree", refuse)
    ckpt.save(tmp_path, 0, tr, background=True)
    with pytest.raises(OSError, match="disk full"):
        ckpt.wait()
    ckpt.wait()     # raised once
    monkeypatch.undo()
    ckpt.save(tmp_path, 0, tr, background=True)
    ckpt.wait()
    assert (tmp_path / "0" / "default" / "_METADATA.json").exists()


@pytest.mark.parametrize("mesh,extra", [("mesh(data=2)", []),
                                        ("mesh(expert=2)", ["methods.moe = all_to_all", "methods.capacity = 4.0"]),
                                        ("mesh(fsdp=2)", []), ("mesh(fsdp=2)", ["methods.accumulate = unreduced"]),
                                        ("mesh(fsdp=2)", ["layout = layout(zero=1)"])])
def test_interleaved_microbatches_over_ranks_match_one_rank(tmp_path, mesh, extra):
    """``methods(interleave=true)`` over two ranks: every rank issues the two halves of a tick in
    the same order, so the collectives of one microbatch's forward and of the other's backward
    (the expert all-to-alls, the early gradient reductions) meet as they would one after another."""
    n = 4 if "fsdp" in mesh else 2
    over = [f"methods.microbatches = {n}", "methods.interleave = true", "methods.remat = full"]
    want_losses, want = _single(MOE, [f"methods.microbatches = {n}"])
    got = _spawn(2, MOE, [f"mesh = {mesh}", *over, *extra], tmp_path)
    assert got["losses"] == pytest.approx(want_losses, abs=2e-5)
    _check_rows(got, want)


def _placed_worker(rank, world, port, overrides, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      BUX_PLACE_DENSE="always")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bux_b200.models.layers import basic
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.set_num_threads(1)
    # the largest dense parameter this rank ever holds whole: counted where parameters are cut
    largest = [0]
    cut = basic.placement.place_dense

    def counting(p):
        kept = cut(p)
        if kept is p:
            largest[0] = max(largest[0], p.numel())
        return kept

    basic.placement.place_dense = counting
    run = compile_runs(MOE, filename="p.bux", overrides=overrides)[0]
    par = Parallel(run.train, torch.device("cpu"))
    tr = Trainer(run, device="cpu", parallel=par)
    placed = sum(getattr(p, "placed_whole", None) is not None for p in tr.model.parameters())
    feed = iter(tr.batches())
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    if rank == 0:
        torch.save({"losses": losses, "state": state, "placed": placed, "whole_kept": largest[0]}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mesh,extra", [
    (2, "mesh(fsdp=2)", ["methods.microbatches = 2", "methods.remat = full"]),
    (4, "mesh(data=2, fsdp=2)", []),
    (2, "mesh(expert=2)", ["methods.moe = all_to_all", "methods.capacity = 4.0"]),     # experts and dense rows over one axis
    (2, "mesh(fsdp=2)", ["a = gqa(num_heads=2, num_kv_heads=1, rope=rope(), mimetic_vo=0.05)"]),
])
def test_dense_parameters_are_built_as_the_ranks_shard(tmp_path, world, mesh, extra):
    """With dense placement every projection and the token table are cut to the rank's rows as
    they are created (the whole tensor is drawn first, so the values are a one-rank build's): the
    run matches one rank, and no projection is ever kept whole."""
    out = str(tmp_path / "r.pt")
    plain = [e for e in extra if not e.startswith("methods.moe") and not e.startswith("methods.capacity")]
    want_losses, want = _single(MOE, plain)
    mp.spawn(_placed_worker, args=(world, _free_port(), [f"mesh = {mesh}", *extra], out), nprocs=world, join=True)
    got = torch.load(out)
    assert got["placed"] >= 3, got["placed"]
    assert got["losses"] == pytest.approx(want_losses, abs=2e-5)
    _check_rows(got, want)
    if "mimetic" in " ".join(extra):
        assert got["whole_kept"] > 0        # V and O of the mimetic layer were built whole on purpose
    else:
        assert got["whole_kept"] <= 64      # only parameters whose rows do not divide stay whole (none larger than a bias)
