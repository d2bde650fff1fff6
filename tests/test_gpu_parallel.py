"""Multi-GPU paths: NCCL ranks as child processes (needs >= 2 GPUs, else skipped).
NVLS is switched off for these short-lived test ranks."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

MOE = """
d_model=256
vocab_size=512
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, head_dim=64, rope=rope())
e = moe(num_experts=8, top_k=2, expert=gated_mlp(intermediate_size=128, activation=swish))
block = [n a] [n e]
model = embed block^2 n head
data = synthetic
optimizer = adamw(lr=1e-3, eps=1.0)
seq_len = 256
batch = 8
steps = 4
methods = methods(remat=full)
"""


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, overrides, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from bux_b200.lang import compile_runs
    from bux_b200.ops import kernels as K
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    run = compile_runs(MOE, filename="p.bux", overrides=overrides)[0]
    par = Parallel(run.train, dev)
    tr = Trainer(run, device=dev, parallel=par)
    feed = iter(tr.batches())
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    torch.cuda.synchronize()
    K.check_status(dev, "ep test")
    if rank == 0:
        torch.save({"losses": losses,
                    "state": {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fmt,remat,extra", [
    ("compute", "full", []),
    ("mxfp8", "full", ["methods.moe_chunks = 2", "methods.moe_stream = true"]),
    ("mxfp8", "full", ["methods.moe_chunks = 4", "methods.moe_stream = true"]),
    ("mxfp8", "none", ["methods.moe_chunks = 2", "methods.moe_stream = true"]),
])
def test_fused_expert_parallel_matches_one_gpu(cuda, tmp_path, fmt, remat, extra):
    """Every rank count the box offers (2, 4, 8): experts over the ranks with the in-kernel
    exchange, every other parameter sharded over the same ranks, against one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    prec = f"precision = precision(compute=bfloat16, matmuls={fmt})"
    # without checkpointing no replay refills the exchange buffers before a layer's backward
    keep = f"methods.remat = {remat}"
    run = compile_runs(MOE, filename="p.bux", overrides=[prec, keep])[0]
    tr = Trainer(run, device=cuda)
    feed = iter(tr.batches())
    want = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}
    for world in [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]:
        out = str(tmp_path / f"r0_{world}.pt")
        mp.spawn(_worker, args=(world, _free_port(), [prec, keep, f"mesh = mesh(expert={world})",
                                                      "methods.moe = fused_ep", "methods.capacity = 2.0", *extra], out),
                 nprocs=world, join=True)
        got = torch.load(out)
        assert got["losses"] == pytest.approx(want, abs=3e-2), world
        for name, p in state.items():
            g = got["state"][name]
            if g.shape != p.shape:
                p = p[: g.shape[0]]  # rank 0 holds the first experts and the first rows of the rest
            err = ((g - p).norm() / p.norm().clamp_min(1e-9)).item()
            assert err < 2e-2, (world, name, err)


def test_fused_expert_parallel_drops_rows_past_the_capacity(cuda, tmp_path):
    """With a capacity below what the routing needs, the in-kernel exchange and the library
    all-to-all drop the same picks: two ranks of each must agree."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    prec = "precision = precision(compute=bfloat16, matmuls=compute)"
    outs = {}
    for method in ("fused_ep", "all_to_all"):
        out = str(tmp_path / f"{method}.pt")
        mp.spawn(_worker, args=(2, _free_port(), [prec, "mesh = mesh(expert=2)", f"methods.moe = {method}",
                                                  "methods.capacity = 0.6"], out), nprocs=2, join=True)
        outs[method] = torch.load(out)
    assert outs["fused_ep"]["losses"] == pytest.approx(outs["all_to_all"]["losses"], abs=3e-2)
    for name, p in outs["all_to_all"]["state"].items():
        g = outs["fused_ep"]["state"][name]
        err = ((g - p).norm() / p.norm().clamp_min(1e-9)).item()
        assert err < 2e-2, (name, err)


DENSE = MOE.replace("e = moe(num_experts=8, top_k=2, expert=gated_mlp(intermediate_size=128, activation=swish))",
                    "e = gated_mlp(intermediate_size=512, activation=swish)") \
           .replace("model = embed block^2 n head", "model = embed block^2 n head(tied=false)")


def _tensor_worker(rank, world, port, overrides, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from bux_b200.ckpt.store import state_tree
    from bux_b200.lang import compile_runs
    from bux_b200.ops import kernels as K
    from bux_b200.parallel.engine import Parallel
    from bux_b200.train.trainer import Trainer

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    run = compile_runs(DENSE, filename="p.bux", overrides=overrides)[0]
    par = Parallel(run.train, dev)
    tr = Trainer(run, device=dev, parallel=par)
    feed = iter(tr.batches())
    launches = K.launches
    losses = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    torch.cuda.synchronize()
    K.check_status(dev, "tensor parallel test")
    tree = par.checkpoint_tree(tr, state_tree)
    if rank == 0:
        torch.save({"losses": losses, "launches": K.launches - launches,
                    "state": {n: p.detach().float().cpu() for n, p in tree["0"].items()}}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("method", ["gspmd", "fused"])
def test_sequence_parallel_tensor_parallel_matches_one_gpu(cuda, tmp_path, method):
    """`fused`: all-gather→GEMM and GEMM→reduce-scatter inside the kernels over peer memory."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    prec = "precision = precision(compute=bfloat16)"
    run = compile_runs(DENSE, filename="p.bux", overrides=[prec])[0]
    tr = Trainer(run, device=cuda)
    feed = iter(tr.batches())
    want = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}
    out = str(tmp_path / "r0.pt")
    mp.spawn(_tensor_worker, args=(2, _free_port(), [prec, "mesh = mesh(tensor=2)", "layout = layout(stream=tensor)",
                                                     f"methods.tensor = {method}"], out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["losses"] == pytest.approx(want, abs=3e-2)
    for name, p in state.items():
        err = ((got["state"][name] - p).norm() / p.norm().clamp_min(1e-9)).item()
        assert err < 2e-2, (name, err)


@pytest.mark.parametrize("remat,micro", [("full", 1), ("none", 1), ("full", 2)])
def test_fused_fsdp_matches_one_gpu(cuda, tmp_path, remat, micro):
    """Sharded parameters with the all-gather done by peer stores (the consuming GEMM waits for
    its weight's rows in its own producer warp) and the reduce-scatter by peer loads, on every
    rank count the box offers, against one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    prec = "precision = precision(compute=bfloat16, matmuls=compute)"
    base = [prec, f"methods.remat = {remat}", f"methods.microbatches = {micro}"]
    run = compile_runs(DENSE, filename="p.bux", overrides=base)[0]
    tr = Trainer(run, device=cuda)
    feed = iter(tr.batches())
    want = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}
    for world in [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]:
        out = str(tmp_path / f"r0_{world}.pt")
        mp.spawn(_tensor_worker, args=(world, _free_port(), [*base, f"mesh = mesh(fsdp={world})",
                                                            'compiler = compiler(options="--fsdp=fused")'], out),
                 nprocs=world, join=True)
        got = torch.load(out)
        assert got["losses"] == pytest.approx(want, abs=3e-2), world
        # native kernels moved the parameters: pushes, pulls, flags
        assert got["launches"] > 0
        for name, p in state.items():
            err = ((got["state"][name] - p).norm() / p.norm().clamp_min(1e-9)).item()
            assert err < 2e-2, (world, name, err)


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_pipeline_over_two_gpus_matches_one_gpu(cuda, tmp_path, schedule):
    """Two stages over NCCL send / receive (each direction of the pair on its own communicator),
    four microbatches, against one GPU running the same microbatches."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp

    from bux_b200.lang import compile_runs
    from bux_b200.train.trainer import Trainer

    base = ["precision = precision(compute=bfloat16, matmuls=compute)", "methods.microbatches = 4",
            "methods.remat = none"]
    run = compile_runs(DENSE, filename="p.bux", overrides=base)[0]
    tr = Trainer(run, device=cuda)
    feed = iter(tr.batches())
    want = [tr.train_step(next(feed))["loss"].item() for _ in range(2)]
    state = {n: p.detach().float().cpu() for n, p in tr.model.named_parameters()}
    out = str(tmp_path / "r0.pt")
    mp.spawn(_tensor_worker, args=(2, _free_port(), [*base, "mesh = mesh(stage=2)", f"methods.pipeline = \"{schedule}\""], out),
             nprocs=2, join=True)
    got = torch.load(out)
    assert got["losses"] == pytest.approx(want, abs=3e-2)
    for name, p in state.items():
        err = ((got["state"][name] - p).norm() / p.norm().clamp_min(1e-9)).item()
        assert err < 2e-2, (name, err)
