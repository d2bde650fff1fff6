"""The expert exchange's kernels alone, on the GPUs of one node:
``python -m torch.distributed.run --nproc-per-node N -m bux_b200.parallel.bench_exchange``.

Every rank routes `--tokens` tokens to `--top` of `--experts` experts (uniform picks), then
times, with nothing else on the GPU,

* the push of its rows into the owners' buffers, as bf16 and quantised to MXFP8 on the way;
* the pull of its picks' output rows, summed per token;

for each `--ctas` setting (CTAs per SM the kernels may take). A kernel's bytes are what it
writes (push) or reads (pull); the NVLink share is the part whose owner is another rank.
Times are CUDA events, the maximum over the ranks of the mean of `--iters` calls after three
warm-up calls; the buffers of one call (hundreds of MB) exceed L2.
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def timed(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--top", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", default="0,1,2,4,8")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import kernels as K
    from . import experts as X

    group = dist.group.WORLD
    t, d, k = args.tokens, args.d, args.top
    cap = (t * k * 5 // 4 + 127) // 128 * 128
    ep = X.FusedEP(group, dev, d, cap)
    gen = torch.Generator(device=dev).manual_seed(rank)
    idx = torch.rand(t, args.experts, device=dev, generator=gen).topk(k, dim=1).indices
    r = X.route_chunks(idx, args.experts, group, cap, 1)[0]
    x = torch.randn(t, d, device=dev, generator=gen).bfloat16()
    out = torch.empty(t, d, dtype=torch.bfloat16, device=dev)
    remote = float((r.dst_rank != rank).float().mean().item())
    rows = t * k

    def push():
        K.ep_push_rows(x, r.src_token, r.dst_rank, r.dst_row, ep.tables[("x", 0)])

    def push_mx():
        K.ep_push_rows_mx(x, r.rank_of, r.row_of, ep.tables[("xq", 0)], ep.tables[("xsf", 0)])

    def pull():
        K.ep_pull_combine(ep.tables[("y", 0)], r.rank_of, r.row_of, None, t, d, torch.bfloat16, out=out)

    cases = (("push bf16", push, rows * d * 2), ("push mxfp8", push_mx, rows * d), ("pull-combine", pull, rows * d * 2))
    if rank == 0:
        print(f"{world} GPUs, {t} tokens x top {k} of {args.experts}, d {d}: {remote:.0%} of the rows cross NVLink")
        print(f"{'kernel':14s} {'CTAs/SM':>8s} {'ms':>8s} {'GB/s':>8s} {'NVLink GB/s':>12s}")
    for ctas in [int(c) for c in args.ctas.split(",")]:
        K.set_comm_ctas_per_sm(ctas)
        for name, fn, nbytes in cases:
            ms = timed(fn, args.iters)
            if rank == 0:
                gbs = nbytes / ms / 1e6
                print(f"{name:14s} {ctas or 'default':>8} {ms:8.3f} {gbs:8.0f} {gbs * remote:12.0f}")
    K.set_comm_ctas_per_sm(0)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
