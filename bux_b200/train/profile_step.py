"""Where one training step's GPU time goes: a kernel table from the torch profiler.

    python -m bux_b200.train.profile_step examples/benchmarks/qwen3_30b_a3b_mxfp8.bux \\
        --layers 4 --rows 32 "mesh = mesh(expert=1)" "methods.moe = sorted"

builds the run with its repeat cut to `--layers` blocks (the full model need not fit), trains
two warm-up steps, profiles the third and prints the kernels by total device time. The numbers
explain a step; they are not benchmark values (the profiler is on).

Under ``torchrun`` every rank joins the job and trains its share; rank 0 prints. After the
table come the totals of `trace.classify`: communication time, the part of it no compute
kernel covers, idle time; and the busy time of every stream. ``--trace FILE`` also writes the
chrome trace.
"""

from __future__ import annotations

import argparse
from pathlib import Path

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("file")
    ap.add_argument("overrides", nargs="*")
    ap.add_argument("--layers", type=int, default=4, help="blocks kept of the model's repeat")
    ap.add_argument("--model", default="embed block^{layers} norm head",
                    help="the cut model, in the file's own names ({layers} is filled in)")
    ap.add_argument("--rows", type=int, default=32, help="rows per step")
    ap.add_argument("--top", type=int, default=60, help="table rows")
    ap.add_argument("--offload", action="store_true", help="block inputs in pinned host memory")
    ap.add_argument("--trace", default="", help="write the chrome trace of the profiled step here")
    args = ap.parse_intermixed_args(argv)  # overrides may follow the options

    from .. import runtime
    from ..lang import compile_runs
    from . import trace
    from .trainer import Trainer

    runtime.configure()
    world, rank, local = runtime.world_size(), runtime.rank(), runtime.local_rank()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    path = Path(args.file)
    overrides = [f"batch = {args.rows}", "steps = 100", "log = log(every=1000000)",
                 "model = " + args.model.format(layers=args.layers), *args.overrides]
    run = compile_runs(path.read_text(), filename=str(path), overrides=overrides)[0]
    parallel = None
    if world > 1:
        import torch.distributed as dist

        from ..parallel.engine import Parallel

        dist.init_process_group("nccl", device_id=device)
        parallel = Parallel(run.train, device)
    trainer = Trainer(run, device=device, parallel=parallel, fuse_optimizer=world == 1, moments="fp8", master=False)
    trainer.model.set_remat(True, offload=args.offload)
    feed = iter(trainer.batches())
    for _ in range(2):
        trainer.train_step(next(feed))
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        trainer.train_step(next(feed))
        torch.cuda.synchronize()
    if rank == 0:
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.top, max_name_column_width=70))
        kernels = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        spans = [(e.name, float(e.time_range.start), float(e.time_range.end - e.time_range.start)) for e in kernels]
        print({k: round(v, 2) for k, v in trace.classify(spans).items()})
        streams: dict = {}
        for e in kernels:
            streams.setdefault(e.device_resource_id if hasattr(e, "device_resource_id") else 0, []).append(
                [float(e.time_range.start), float(e.time_range.end)])
        for sid, iv in sorted(streams.items()):
            print(f"stream {sid}: {len(iv)} kernels, busy {trace.length(trace.merge(iv)) / 1000:.2f} ms")
    if args.trace:
        out = Path(args.trace)
        prof.export_chrome_trace(str(out if world == 1 else out.with_name(f"{out.stem}.rank{rank}{out.suffix}")))
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
