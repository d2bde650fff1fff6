"""Headline benchmark: training throughput of Qwen3-30B-A3B (MXFP8 matmuls, experts
split over the GPUs) in tokens/s over all GPUs of one node, synthetic data, random init.

    python bench.py --gpus 1 --steps 4 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 4 --warmup 3

Prints one JSON line (rank 0). `value` is device-timed (CUDA events around exactly
`steps` steps, max over ranks); `e2e` is the same steps through `Trainer.train_step`
with every step's batch copied from pinned host memory and its loss read back.
`--impl reference` runs the unmodified reference from ``baseline/_ref`` when it can
be imported, else reports why not.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# before torch starts its allocator: segments that grow in place (no fragmentation between the
# step's large transients and the tensors kept across the step)
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

MARGIN_BYTES = 12 << 30  # device memory left free when attention outputs are kept (fragmentation, chunk buffers)
PUBLISHED_TOK_S_PER_GPU = 42391.0  # reference, 8xB300, MXFP8 `sorted` fsdp=8 (docs/performance/benchmarks.md:188)
ROWS_PER_GPU = 32                  # 256 rows of 4096 over 8 GPUs


def reference_arm(args) -> int:
    why = None
    ref = ROOT / "baseline" / "_ref"
    if not ref.exists():
        why = ("baseline/_ref is not installed: the reference's build backend (uv_build) and its JAX stack "
               "(jax, flax, optax, orbax-checkpoint) are neither in the image nor in the offline wheelhouse")
    else:
        sys.path.insert(0, str(ref))
        try:
            import bux  # noqa: F401
        except Exception as err:  # noqa: BLE001
            why = f"the reference does not import here: {type(err).__name__}: {str(err)[:120]}"
    if why is None:
        why = "the reference needs jax/flax/optax (not in this image) to train"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().splitlines() if r.strip()]
        os.unlink(self.file.name)
        clocks = sorted(float(r[1]) for r in rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        reasons = set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            if len(r) >= 9:
                for name, v in zip(names, r[5:9]):
                    if v.strip().lower() == "active":
                        reasons.add(name)
        mx = next((float(r[2]) for r in rows if len(r) >= 9), None)
        med = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(clocks)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bux_b200", choices=["bux_b200", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="debug only: fewer layers (the result is then marked invalid)")
    ap.add_argument("--rows", type=int, default=None, help="rows per GPU per step (default: the benchmark's own)")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--model", default="qwen3_30b_a3b", choices=["qwen3_30b_a3b", "llama3_8b"],
                    help="the flagship (Qwen3-30B-A3B, MXFP8, experts over the GPUs) or the second benchmark "
                         "(Llama-3-8B, bf16, parameters sharded over the GPUs)")
    ap.add_argument("--set", action="append", default=[], metavar="NAME=VALUE",
                    help="one more override of the benchmark's file (an experiment: the JSON line records it)")
    ap.add_argument("--inputs", default="auto", choices=["auto", "host", "device"],
                    help="where the checkpointed block inputs wait for the backward: pinned host memory, the "
                         "device, or (auto) the device when they fit")
    ap.add_argument("--fsdp", default="fused", choices=["fused", "nccl"],
                    help="llama3_8b: all-gather / reduce-scatter by this library's peer-memory kernels or by NCCL")
    args = ap.parse_args()
    llama = args.model == "llama3_8b"
    if args.rows is None:
        args.rows = 8 if llama else ROWS_PER_GPU
    if args.seq_len is None:
        args.seq_len = 8192 if llama else 4096
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from bux_b200 import runtime
    from bux_b200.lang import compile_runs
    from bux_b200.ops import kernels as K
    from bux_b200.train.flops import flops_per_token
    from bux_b200.train.trainer import Trainer

    runtime.configure()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun), found {world}", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    parallel = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        from bux_b200.parallel.engine import Parallel
    n = args.gpus
    total_steps = args.warmup + 2 * args.steps + 2
    overrides = [f"batch = {args.rows * n}", f"steps = {2 * total_steps + 4}",
                 f"seq_len = {args.seq_len}", "log = log(every=1000000)"]
    if llama:
        overrides += [f"mesh = mesh(fsdp={n})", "methods.microbatches = 1"]
        if args.fsdp == "fused" and n > 1:
            overrides.append('compiler = compiler(options="--fsdp=fused")')
        path = ROOT / "examples" / "benchmarks" / "llama3_8b_fsdp8.bux"
    else:
        overrides += [f"mesh = mesh(expert={n})", f"methods.moe = {'fused_ep' if n > 1 else 'sorted'}"]
        path = ROOT / "examples" / "benchmarks" / "qwen3_30b_a3b_mxfp8.bux"
    if args.layers:
        overrides.append(f"model = embed block^{args.layers} norm head")
    overrides += [o.replace("=", " = ", 1) for o in args.set]
    run = compile_runs(path.read_text(), filename=str(path), overrides=overrides)[0]
    if world > 1:
        parallel = Parallel(run.train, device)
    # One state layout and one activation policy at every N, sized by the one-GPU case (the whole
    # 30.5B-parameter model on 180 GB): bf16 weights that the optimizer updates in place, 8-bit
    # block-scaled moments, each block's input kept in pinned host memory, each block rerun in
    # the backward. Dense parameters and their moments are sharded over the ranks like the
    # experts (the mesh's expert axis is also the axis parameters are sharded over).
    # Gradients: with two or more GPUs a rank's gradients (at most 16 GB of bf16) are held to
    # the end of the step and clipped by the step's own norm; the 61 GB of one GPU's gradients
    # do not fit beside its state, so there each gradient is consumed by the optimizer as soon
    # as the backward produces it and the clip factor comes from the previous step's norm.
    # (Llama-3-8B: the recipe of its file as it is: fp32 master weights and moments, sharded.)
    fused_updates = n == 1 and not llama
    offload = not llama
    if llama:
        trainer = Trainer(run, device=device, parallel=parallel)
    else:
        trainer = Trainer(run, device=device, parallel=parallel, fuse_optimizer=fused_updates,
                          moments="fp8", master=False)
    # Attention outputs (and their log-sum-exp) are kept on the device for as many blocks as
    # fit: the backward's rerun of those blocks skips the attention forward. One probe step
    # without them gives the step's peak; what the device has left after a margin is divided
    # by a block's kept bytes. All ranks take the smallest count.
    arch = run.arch
    attn = next(l.config for l in arch.layers() if l.config.type == "gqa")
    blocks = sum(1 for l in arch.layers() if l.config.type == "gqa")
    hd = attn.head_dim or arch.d_model // attn.num_heads
    kept_bytes = args.rows * args.seq_len * attn.num_heads * (hd * 2 + 4)  # o in bf16, lse in fp32
    trainer.model.set_remat(True, offload=offload, keep_attention=False)
    feed = iter(trainer.batches())
    tokens_per_step = args.rows * n * args.seq_len

    def one_step(read_loss: bool):
        batch = next(feed)
        out = trainer.train_step(batch)
        if read_loss:
            return float(out["loss"].item())
        return out

    def note(text: str) -> None:
        if rank == 0:
            print(f"[bench] {text}", file=sys.stderr, flush=True)

    def gib(b) -> str:
        return f"{b / 2 ** 30:.1f} GiB"

    def agreed_min(value: int) -> int:
        if parallel is None:
            return value
        import torch.distributed as dist

        t = torch.tensor([value], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t.item())

    note(f"state built: {gib(torch.cuda.memory_allocated(device))} allocated")
    torch.cuda.reset_peak_memory_stats(device)
    one_step(True)  # the probe step (an extra warm-up step)
    torch.cuda.synchronize()
    free, total_mem = torch.cuda.mem_get_info(device)
    slack = torch.cuda.memory_reserved(device) - torch.cuda.max_memory_allocated(device)
    spare = free + max(0, slack) - MARGIN_BYTES
    # What the device has left goes first to kept attention outputs, then, if every block's
    # fits, to the block inputs (one [rows, seq, d_model] tensor per block, which otherwise wait in
    # pinned host memory). Measured: on one GPU the host copies are hidden (4.72 s a step with 30
    # outputs kept and the inputs on the host, 4.86 s with the inputs on the device and 7 kept);
    # with four ranks on one host they cost 0.3 s a step (5.38 s against 5.09 s). All ranks take
    # the same decision and the smallest count.
    inputs_bytes = blocks * args.rows * args.seq_len * arch.d_model * 2
    if offload and args.inputs == "device":   # asked for: the inputs first, attention outputs with the rest
        offload = False
        spare -= inputs_bytes
    keep_blocks = agreed_min(max(0, min(blocks, int(spare // kept_bytes))))
    if offload and args.inputs == "auto":
        fits = keep_blocks == blocks and spare - blocks * kept_bytes >= inputs_bytes
        if agreed_min(int(fits)):
            offload = False
    note(f"probe step: peak {gib(torch.cuda.max_memory_allocated(device))}, reserved "
         f"{gib(torch.cuda.memory_reserved(device))}, free {gib(free)} of {gib(total_mem)}; "
         f"block inputs ({gib(inputs_bytes)}) wait {'in pinned host memory' if offload else 'on the device'}; "
         f"attention outputs kept for {keep_blocks} of {blocks} blocks ({gib(kept_bytes)} each)")

    def set_keep(count: int) -> None:
        trainer.model.set_remat(True, offload=offload, keep_attention=count if count else False)

    def guarded(loop):
        """Run `loop`; if the device runs out of memory, halve the number of kept blocks
        (all ranks agree on the outcome between loops, never inside a step) and run it again.
        A timed loop that was cut short is timed again from its start."""
        nonlocal keep_blocks, offload
        while True:
            failed = 0
            result = None
            try:
                result = loop()
            except torch.cuda.OutOfMemoryError as err:
                if parallel is not None:
                    raise  # the other ranks are inside a collective: the job ends here
                failed = 1
                note(f"out of memory at step {trainer.step} with {keep_blocks} blocks kept: {str(err)[:300]}")
            if not failed:
                return result
            if not offload and not llama:
                offload = True   # first the block inputs go back to the host
            elif keep_blocks == 0:
                raise RuntimeError("out of device memory with no attention outputs kept")
            else:
                keep_blocks //= 2
            set_keep(keep_blocks)
            import gc

            from bux_b200.models import graph

            graph._OFFLOADED.clear()
            graph._IN_FLIGHT.clear()
            torch.cuda.synchronize()
            gc.collect()
            torch.cuda.empty_cache()
            note(f"after the failure: {gib(torch.cuda.memory_allocated(device))} allocated, "
                 f"{gib(torch.cuda.mem_get_info(device)[0])} free; keeping {keep_blocks} blocks")

    set_keep(keep_blocks)
    guarded(lambda: [one_step(True) for _ in range(args.warmup)])
    note(f"warm-up done: peak {gib(torch.cuda.max_memory_allocated(device))}")
    torch.cuda.synchronize()
    if parallel is not None:
        parallel.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-timed region: exactly `steps` steps
    def timed():
        launches0 = K.launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if parallel is not None:
            parallel.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            one_step(False)
        end.record()
        torch.cuda.synchronize()
        if parallel is not None:
            parallel.barrier()
        return start.elapsed_time(end), K.launches - launches0

    ms, launches = guarded(timed)
    note(f"timed region done: {ms / args.steps:.0f} ms per step, peak {gib(torch.cuda.max_memory_allocated(device))}")
    K.check_status(device, "bench")

    # ---- end-to-end region through the public step API: every step's batch comes from pinned
    # host memory (`Trainer.to_device`) and its loss is read back to the host
    def end_to_end():
        if parallel is not None:
            parallel.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        value = None
        for _ in range(args.steps):
            value = one_step(True)
        torch.cuda.synchronize()
        return time.perf_counter() - t0, value

    e2e_s, loss = guarded(end_to_end)
    K.check_status(device, "bench (end to end)")
    clocks = sampler.stop() if rank == 0 else None
    times = torch.tensor([ms, e2e_s * 1000], device=device, dtype=torch.float64)
    if parallel is not None:
        import torch.distributed as dist

        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    if rank == 0:
        ms_step = ms / args.steps
        value = tokens_per_step / (ms_step / 1000)
        e2e_value = tokens_per_step / (e2e_ms / args.steps / 1000)
        fpt = flops_per_token(run.arch, args.seq_len)
        rows_local = args.rows
        h2d = rows_local * args.seq_len * (4 + 4 + 1)  # ids, positions (int32) and mask per step
        if llama:
            # the second benchmark: its own metric, config and baseline
            result = {
                "metric": "train tokens/sec (Llama-3-8B bf16, parameters sharded over the GPUs)",
                "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": value / n / 32749.0, "dtype": "bf16",
                "data": "synthetic (uniform random tokens), random-init weights",
                "tokens_per_s_per_gpu": value / n, "mfu_bf16_peak": value / n * fpt / 2.25e15,
                "config": {"model": "llama3_8b" + (f" TRUNCATED to {args.layers} layers: INVALID" if args.layers else ""),
                           "global_batch": args.rows * n, "seq_len": args.seq_len,
                           "parallelism": f"fsdp{n}" if n > 1 else "1 gpu",
                           "fsdp_collectives": ("peer-memory kernels (all-gather by peer stores, the consuming GEMM "
                                                "waits per column tile; reduce-scatter by peer loads)")
                           if (args.fsdp == "fused" and n > 1) else "NCCL",
                           "optimizer": "adamw, fp32 master weights and moments, clip by this step's own global norm",
                           "remat": "every block rerun in the backward, attention outputs kept on the device where they fit",
                           "attention_outputs_kept": f"{keep_blocks} of {blocks} blocks",
                           "baseline": "the reference's MXFP8 run on 8 x B300, 32,749 tokens/s/GPU (it publishes no bf16 run)",
                           "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 1e9, 1),
                           "l2": "inputs and weights exceed L2 (126 MB) every step", "loss_last_step": loss},
                "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
                "gpu_launches": launches,
            }
            print(json.dumps(result))
            result = None
        else:
            result = {
            "metric": "train tokens/sec (Qwen3-30B-A3B MXFP8, experts over the GPUs)",
            "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / n / PUBLISHED_TOK_S_PER_GPU, "dtype": "bf16 + mxfp8 matmuls",
            "data": "synthetic (uniform random tokens), random-init weights",
            "tokens_per_s_per_gpu": value / n,
            "mfu_bf16_peak": value / n * fpt / 2.25e15,
            "config": {"model": "qwen3_30b_a3b" + (f" TRUNCATED to {args.layers} layers: INVALID" if args.layers else ""),
                       "global_batch": args.rows * n, "seq_len": args.seq_len,
                       "parallelism": (f"ep{n} + fsdp{n} (experts split over the expert axis, every other parameter "
                                       f"and its moments sharded over the same {n} ranks)") if n > 1
                       else "1 gpu (all experts local)",
                       "optimizer": "adamw, bf16 master weights, 8-bit block-scaled moments",
                       "clip": ("by the previous step's norm, updates fused into the backward (one GPU cannot hold "
                                "61 GB of gradients beside the state)") if fused_updates
                       else "by this step's own global norm",
                       "remat": "every block rerun in the backward, block inputs "
                                + ("in pinned host memory" if offload else "on the device")
                                + ", attention outputs kept on the device where they fit",
                       "attention_outputs_kept": f"{keep_blocks} of {blocks} blocks",
                       "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 1e9, 1), "l2": "inputs and weights exceed L2 (126 MB) every step",
                       "loss_last_step": loss},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
        }
        if result is not None:
            if args.set:
                result["config"]["overrides"] = list(args.set)
            print(json.dumps(result))
    if parallel is not None:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
