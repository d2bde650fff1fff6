"""Fused compute+collective kernels against their library baselines, on the GPUs of one
node: ``python -m torch.distributed.run --nproc-per-node N -m bux_b200.parallel.bench_fused``.

* all-gather → GEMM: `tensor_fused.GatherMatmul` vs NCCL all_gather + cuBLAS matmul;
* GEMM → reduce-scatter: `tensor_fused.MatmulScatter` vs cuBLAS matmul + NCCL reduce_scatter.

Times are CUDA events on each rank's stream after 3 warm-up calls, the maximum over the
ranks of the mean of `iters` calls; a 256 MB buffer is written between calls to flush L2.
The roofline is the slower of FLOPs / measured bf16 peak and NVLink bytes / 770 GB/s.
"""

from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist


def timed(fn, iters: int, flush) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192, help="rows (tokens) per rank")
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--f", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import kernels as K
    from . import tensor_fused as TF

    group = dist.group.WORLD
    peaks = {"bf16_tflops": 1590.0}
    pk = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows, d, f = args.rows, args.d, args.f // world
    x_l = torch.randn(rows, d, device=dev).bfloat16()
    w_col = (torch.randn(f, d, device=dev) * 0.02).bfloat16()       # column-parallel: [f/world, d]
    h = torch.randn(world * rows, f, device=dev).bfloat16()
    w_row = (torch.randn(d, f, device=dev) * 0.02).bfloat16()       # row-parallel: [d, f/world]
    full = torch.empty(world * rows, d, dtype=torch.bfloat16, device=dev)
    part = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)

    def lib_ag():
        dist.all_gather_into_tensor(full, x_l)
        return torch.matmul(full, w_col.t())

    def lib_rs():
        y = torch.matmul(h, w_row.t())
        dist.reduce_scatter_tensor(part, y)
        return part

    with torch.no_grad():
        want_ag, want_rs = lib_ag().float(), lib_rs().float().clone()
        got_ag = TF.GatherMatmul.apply(x_l, w_col, group).float()
        got_rs = TF.MatmulScatter.apply(h, w_row, group, rows).float()
        err_ag = ((got_ag - want_ag).norm() / want_ag.norm()).item()
        err_rs = ((got_rs - want_rs).norm() / want_rs.norm()).item()
        ms = {"ag_gemm fused": timed(lambda: TF.GatherMatmul.apply(x_l, w_col, group), args.iters, flush),
              "ag_gemm library": timed(lib_ag, args.iters, flush),
              "gemm_rs fused": timed(lambda: TF.MatmulScatter.apply(h, w_row, group, rows), args.iters, flush),
              "gemm_rs library": timed(lib_rs, args.iters, flush)}
    K.check_status(dev, "bench_fused")
    if rank == 0:
        flops = 2.0 * world * rows * d * f
        link = (world - 1) * rows * d * 2                      # bytes that must cross NVLink per rank
        floor = max(flops / (peaks["bf16_tflops"] * 1e12), link / 770e9) * 1e3
        out = {"world": world, "rows_per_rank": rows, "d": d, "f_local": f, "relative_error": {"ag_gemm": err_ag, "gemm_rs": err_rs},
               "ms": ms, "roofline_ms": floor,
               "of_roofline": {k: floor / v for k, v in ms.items()}}
        print(json.dumps(out, indent=1))
        if args.json:
            Path(args.json).write_text(json.dumps(out, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
