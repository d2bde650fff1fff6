"""Where one training step's GPU time goes: a kernel table from the torch profiler.

    python -m bux_b200.train.profile_step examples/benchmarks/qwen3_30b_a3b_mxfp8.bux \\
        --layers 4 --rows 32 "mesh = mesh(expert=1)" "methods.moe = sorted"

builds the run with its repeat cut to `--layers` blocks (the full model need not fit), trains
two warm-up steps, profiles the third and prints the kernels by total device time. The numbers
explain a step; they are not benchmark values (the profiler is on).
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
    args = ap.parse_intermixed_args(argv)  # overrides may follow the options

    from ..lang import compile_runs
    from .trainer import Trainer

    path = Path(args.file)
    overrides = [f"batch = {args.rows}", "steps = 100", "log = log(every=1000000)",
                 "model = " + args.model.format(layers=args.layers), *args.overrides]
    run = compile_runs(path.read_text(), filename=str(path), overrides=overrides)[0]
    trainer = Trainer(run, device="cuda:0", fuse_optimizer=True, moments="fp8", master=False)
    trainer.model.set_remat(True, offload=args.offload)
    feed = iter(trainer.batches())
    for _ in range(2):
        trainer.train_step(next(feed))
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        trainer.train_step(next(feed))
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.top, max_name_column_width=70))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
