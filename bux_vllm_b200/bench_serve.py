"""Serving benchmark of an exported bux model under vLLM with this plugin.

    python -m bux_vllm_b200.bench_serve examples/benchmarks/qwen3_30b_a3b_mxfp8.bux \\
        --requests 256 --prompt 1024 --generate 256 --batch 64 [--layers N] [--tp N]

Builds the model of a ``.bux`` file with random-init weights, exports it in the ``bux``
format (so that vLLM has to go through this plugin; a standard family's own format would be
served by vLLM without it), starts an offline vLLM engine on it and generates
``--generate`` tokens for ``--requests`` uniform-random prompts of ``--prompt`` tokens with
at most ``--batch`` sequences in flight. Prints one JSON line: decode tokens/s over the
whole run and the median time to the first token. The workload is the serving one the
reference's docs describe (``docs/export/vllm.md:741-752`` there measure a different model;
none exists for this one).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time
from pathlib import Path


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("file")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--generate", type=int, default=256)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--layers", type=int, default=None, help="fewer blocks (a smoke run; the result is marked)")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--keep", default=None, help="folder to export into (default: a temporary one)")
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs / compilation in the engine (a quick smoke run)")
    args = ap.parse_args()

    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")   # the plugin is registered in this process
    import torch

    from bux_b200.export import huggingface
    from bux_b200.lang import compile_runs
    from bux_b200.models import Model

    path = Path(args.file)
    overrides = [f"model = embed block^{args.layers} norm head"] if args.layers else []
    run = compile_runs(path.read_text(), filename=str(path), overrides=overrides)[0]
    dtype = getattr(torch, args.dtype)
    t0 = time.perf_counter()
    model = Model(run.arch, dtype=dtype, seed=0, device="cuda" if torch.cuda.is_available() else "cpu")
    folder = Path(args.keep) if args.keep else Path(tempfile.mkdtemp(prefix="bux_serve_"))
    huggingface.save(run, model, folder, dtype=dtype, step=0, family="bux")
    params = sum(p.numel() for p in model.parameters())
    del model
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    export_s = time.perf_counter() - t0

    import bux_vllm_b200

    bux_vllm_b200.register()
    from vllm import LLM, SamplingParams

    t0 = time.perf_counter()
    llm = LLM(model=str(folder), trust_remote_code=True, dtype=args.dtype, tensor_parallel_size=args.tp,
              max_num_seqs=args.batch, max_model_len=args.prompt + args.generate + 8, skip_tokenizer_init=True,
              enforce_eager=args.eager, gpu_memory_utilization=0.9)
    load_s = time.perf_counter() - t0
    g = torch.Generator().manual_seed(0)
    vocab = run.arch.vocab_size
    prompts = [{"prompt_token_ids": torch.randint(0, vocab, (args.prompt,), generator=g).tolist()}
               for _ in range(args.requests)]
    # time to first token: one scheduler batch of prompts, one token each
    first = SamplingParams(max_tokens=1, ignore_eos=True, detokenize=False)
    llm.generate(prompts[:2], first, use_tqdm=False)   # warm-up (graph capture, autotuning)
    ttfts = []
    for start in range(0, min(args.requests, 4 * args.batch), args.batch):
        t0 = time.perf_counter()
        llm.generate(prompts[start:start + args.batch], first, use_tqdm=False)
        ttfts.append(time.perf_counter() - t0)
    full = SamplingParams(max_tokens=args.generate, ignore_eos=True, detokenize=False)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, full, use_tqdm=False)
    total_s = time.perf_counter() - t0
    generated = sum(len(o.outputs[0].token_ids) for o in outs)
    per_request = [m for m in (getattr(o, "metrics", None) for o in outs) if m is not None
                   and getattr(m, "first_token_time", None) and getattr(m, "arrival_time", None)]
    ttft_engine = (statistics.median(m.first_token_time - m.arrival_time for m in per_request)
                   if per_request else None)
    print(json.dumps({
        "metric": "vLLM serving through the bux plugin", "model": run.name,
        "layers": args.layers or "all" + ("" if not args.layers else " (REDUCED: a smoke run)"),
        "parameters": params, "dtype": args.dtype, "tensor_parallel": args.tp,
        "requests": args.requests, "prompt_tokens": args.prompt, "generated_tokens_per_request": args.generate,
        "max_num_seqs": args.batch, "generated_tokens": generated,
        "decode_tokens_per_s": generated / total_s, "total_s": total_s,
        "p50_ttft_s_batch_of_prompts": statistics.median(ttfts),
        "p50_ttft_s_engine": ttft_engine, "export_s": export_s, "engine_start_s": load_s,
        "data": "uniform-random prompts, random-init weights"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
