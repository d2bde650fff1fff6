"""Micro-benchmarks of the native kernels against the library kernels and the measured
peaks: ``python -m bux_b200.ops.bench_kernels [--json out.json]``.

Timing: CUDA events on the launching stream, 3 warm-up launches, then the mean of
`iters` launches with a 256 MB buffer written between launches to flush L2 (126 MB).
Peaks for the fractions come from ``MEASURED_PEAKS.json`` at the repository root when
present (else the documented fallback: 6.65 TB/s, 1.59 PFLOP/s).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import kernels as K


def peaks() -> dict:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush = None


def timed(fn, iters: int = 10) -> float:
    """Mean milliseconds per call, L2 flushed between calls."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def bench_gemm(rows: list, pk: dict) -> None:
    dev = "cuda"
    shapes = [(8192, 8192, 8192), (32768, 5120, 2048), (32768, 2048, 4096), (16384, 14336, 4096)]
    if SMALL:  # a profiler-sized case: the qkv projection of the benchmark model, short K
        shapes = [(32768, 5120, 2048)]
    for m, n, k in shapes:
        a = torch.randn(m, k, device=dev).bfloat16()
        b = torch.randn(n, k, device=dev).bfloat16()
        flops = 2.0 * m * n * k
        ms_lib = timed(lambda: torch.matmul(a, b.t()))
        for bn in (256, 128):
            ms = timed(lambda: K.gemm_bf16(a, b, bn=bn))
            rows.append({"kernel": f"gemm_bf16 bn={bn}", "shape": f"{m}x{n}x{k}", "ms": ms,
                         "tflops": flops / ms / 1e9, "library_tflops": flops / ms_lib / 1e9,
                         "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})
        aq, asf, _, _ = K.quant_mxfp8(a)
        bq, bsf, _, _ = K.quant_mxfp8(b)
        for bn in (128, 256):
            ms = timed(lambda: K.gemm_mxfp8(aq, asf, bq, bsf, m, n, k, bn=bn))
            rows.append({"kernel": f"gemm_mxfp8 bn={bn}", "shape": f"{m}x{n}x{k}", "ms": ms,
                         "tflops": flops / ms / 1e9, "library_tflops": flops / ms_lib / 1e9,
                         "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})
        ms = timed(lambda: K.quant_mxfp8(a, rowwise=True, colwise=True))
        gb = (m * k * 2 + 2 * m * k * 1.03) / 1e9
        rows.append({"kernel": "quant_mxfp8 row+col", "shape": f"{m}x{k}", "ms": ms, "gbs": gb / ms * 1e3,
                     "of_peak": gb / ms * 1e3 / pk["hbm_gbs"]})


def bench_grouped(rows: list, pk: dict) -> None:
    dev = "cuda"
    e, d, f, per = 128, 2048, 768, 8192  # Qwen3-30B-A3B experts, 131k tokens x top-8
    offsets = torch.arange(0, (e + 1) * per, per, dtype=torch.int32, device=dev)
    x = torch.randn(e * per, d, device=dev).bfloat16()
    w = torch.randn(e, 2 * f, d, device=dev).bfloat16() * 0.02
    xq, xsf, _, _ = K.quant_mxfp8(x)
    wq, wsf, _, _ = K.quant_mxfp8_batched(w)
    flops = 2.0 * e * per * d * 2 * f
    for bn in (128, 256):
        ms = timed(lambda: K.grouped_gemm(xq, wq, offsets, 2 * f, d, kind=K.KIND_MXFP8, asf=xsf, bsf=wsf, bn=bn), 5)
        rows.append({"kernel": f"grouped_gemm_mxfp8 up+gate bn={bn}", "shape": f"{e}x{per}x{2 * f}x{d}", "ms": ms,
                     "tflops": flops / ms / 1e9, "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})
    ms = timed(lambda: K.grouped_gemm(x, w.view(-1, d), offsets, 2 * f, d, bn=256), 5)
    rows.append({"kernel": "grouped_gemm_bf16 up+gate bn=256", "shape": f"{e}x{per}x{2 * f}x{d}", "ms": ms,
                 "tflops": flops / ms / 1e9, "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})


SMALL = False
PHASES = False

BWD_PHASES = {13: "loop overhead", 4: "wait S of the step ahead", 5: "P: tmem ld + math, next row statistics",
              8: "wait dQ", 9: "dQ: tmem ld, arrive", 10: "wait dK (P and dS tiles free)",
              11: "stage dQ, fence, issue reduces", 0: "wait dP of the step ahead", 1: "dS: tmem ld + math",
              2: "wait staged dQ read", 3: "store P and dS, fence, arrive",
              16: "mma: wait P and dS", 17: "mma: issue", 18: "mma: wait dQ read", 19: "mma: wait dO",
              21: "mma: wait Q", 22: "mma: wait S read"}


def attention_bwd_phases(q, k, v, o, do, lse) -> None:
    """Cycles per step that softmax warp 0 and the MMA issuer of the first key tile's CTA spend in
    each phase of the backward's schedule."""
    counters = torch.zeros(32, dtype=torch.int32, device=q.device)
    K.attn_bwd(q, k, v, o, do, lse, phase_cycles=counters)
    c = counters.cpu().tolist()
    steps = max(c[23], 1)
    print(f"attention backward phases, CTA of key tile 0: {steps} steps, cycles per step")
    for slot, name in BWD_PHASES.items():
        print(f"  {name:<52} {c[slot] / steps:9.0f}")
    print(f"  {'softmax warp total':<52} {sum(c[:14]) / steps:9.0f}")
    print(f"  {'mma issuer total':<52} {sum(c[16:23]) / steps:9.0f}")


def bench_attention(rows: list, pk: dict) -> None:
    dev = "cuda"
    shapes = [(8, 4096, 32, 4, 128), (8, 4096, 16, 8, 128), (4, 4096, 64, 8, 64)]
    if SMALL:  # a profiler-sized case: same kernel and tile walk, 2 sequences
        shapes = [(2, 4096, 32, 4, 128)]
    for b, t, h, g, d in shapes:
        q = torch.randn(b, t, h, d, device=dev).bfloat16()
        k = torch.randn(b, t, g, d, device=dev).bfloat16()
        v = torch.randn(b, t, g, d, device=dev).bfloat16()
        do = torch.randn_like(q)
        flops_fwd = 4.0 * b * h * t * t * d / 2
        o, lse = K.attn_fwd(q, k, v)
        ms_f = timed(lambda: K.attn_fwd(q, k, v), 5)
        ms_b = timed(lambda: K.attn_bwd(q, k, v, o, do, lse), 5)
        if PHASES:
            attention_bwd_phases(q, k, v, o, do, lse)
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        ms_lib = timed(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True,
                                                                                enable_gqa=True), 5)
        rows.append({"kernel": "attn_fwd", "shape": f"b{b} t{t} h{h}/{g} d{d}", "ms": ms_f,
                     "tflops": flops_fwd / ms_f / 1e9, "library_ms": ms_lib,
                     "of_peak": flops_fwd / ms_f / 1e9 / pk["bf16_tflops"]})
        rows.append({"kernel": "attn_bwd", "shape": f"b{b} t{t} h{h}/{g} d{d}", "ms": ms_b,
                     "tflops": 2.5 * flops_fwd / ms_b / 1e9,
                     "of_peak": 2.5 * flops_fwd / ms_b / 1e9 / pk["bf16_tflops"]})


def bench_memory_bound(rows: list, pk: dict) -> None:
    dev = "cuda"
    n = 1 << 28
    p = torch.randn(n, device=dev).bfloat16()
    g = torch.randn(n, device=dev).bfloat16()
    m = torch.zeros(n, dtype=torch.uint8, device=dev)
    v = torch.zeros(n, dtype=torch.uint8, device=dev)
    sf = torch.ones(n // 32, dtype=torch.uint8, device=dev)
    sf2 = sf.clone()
    ms = timed(lambda: K.adamw(p, g, m, v, lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, step=1, m_sf=sf, v_sf=sf2), 5)
    gb = n * (2 + 2 + 2 + 2 + 2) / 1e9
    rows.append({"kernel": "adamw bf16 master, 8-bit moments", "shape": f"{n}", "ms": ms, "gbs": gb / ms * 1e3,
                 "of_peak": gb / ms * 1e3 / pk["hbm_gbs"]})
    x = torch.randn(131072, 2048, device=dev).bfloat16()
    w = torch.ones(2048, device=dev)
    ms = timed(lambda: K.rmsnorm_fwd(x, w, 1e-6))
    gb = x.numel() * 4 / 1e9
    rows.append({"kernel": "rmsnorm_fwd", "shape": "131072x2048", "ms": ms, "gbs": gb / ms * 1e3,
                 "of_peak": gb / ms * 1e3 / pk["hbm_gbs"]})
    h = torch.randn(262144, 1536, device=dev).bfloat16()
    ms = timed(lambda: K.glu_fwd(h))
    gb = h.numel() * 3 / 1e9
    rows.append({"kernel": "glu_fwd (swiglu)", "shape": "262144x1536", "ms": ms, "gbs": gb / ms * 1e3,
                 "of_peak": gb / ms * 1e3 / pk["hbm_gbs"]})

    def row(name, shape, ms, gb):
        rows.append({"kernel": name, "shape": shape, "ms": ms, "gbs": gb / ms * 1e3,
                     "of_peak": gb / ms * 1e3 / pk["hbm_gbs"]})

    # the quantiser on expert-sized inputs: plain, with a row gather and scale, and computing the
    # gated activation on the way in (bytes: what each variant has to read and write)
    big = 1 << 19 if SMALL else 1 << 20
    xs = torch.randn(big, 2048, device=dev).bfloat16()
    row("quant_mxfp8 row", f"{big}x2048", timed(lambda: K.quant_mxfp8(xs)), xs.numel() * 3.03 / 1e9)
    row("quant_mxfp8 row+col", f"{big}x2048", timed(lambda: K.quant_mxfp8(xs, rowwise=True, colwise=True)),
        xs.numel() * 4.06 / 1e9)
    if not SMALL:
        tok = torch.randn(big // 8, 2048, device=dev).bfloat16()
        index = torch.randint(0, big // 8, (big,), device=dev, dtype=torch.int32)
        scale = torch.rand(big, device=dev)
        row("quant_mxfp8 row+col, gathered and scaled rows", f"{big}x2048 of {big // 8}",
            timed(lambda: K.quant_mxfp8(tok, rowwise=True, colwise=True, row_index=index, rows=big, row_scale=scale)),
            (tok.numel() * 2 + big * 2048 * 2.06) / 1e9)
        hh = torch.randn(big, 1536, device=dev).bfloat16()
        row("quant_mxfp8_glu row (activation never written)", f"{big}x1536", timed(lambda: K.quant_mxfp8_glu(hh)),
            (hh.numel() * 2 + big * 768 * 1.03) / 1e9)
        dyx = torch.randn_like(x)
        _, rstd = K.rmsnorm_fwd(x, w, 1e-6)
        row("rmsnorm_bwd", "131072x2048", timed(lambda: K.rmsnorm_bwd(x, w, dyx, rstd)), x.numel() * 6 / 1e9)
        q = torch.randn(32, 4096, 32, 128, device=dev).bfloat16()
        pos = torch.arange(4096, device=dev).float()
        ang = pos[:, None] / (10000 ** (torch.arange(0, 64, device=dev).float() / 64))[None]
        cos, sin = ang.cos().repeat(32, 1).contiguous(), ang.sin().repeat(32, 1).contiguous()
        wq = torch.ones(128, device=dev)
        _, rq = K.norm_rope_fwd(q, wq, cos, sin, 1e-6)
        row("norm_rope_fwd", "32x4096x32x128", timed(lambda: K.norm_rope_fwd(q, wq, cos, sin, 1e-6)), q.numel() * 4 / 1e9)
        dq = torch.randn_like(q)
        row("norm_rope_bwd", "32x4096x32x128", timed(lambda: K.norm_rope_bwd(q, wq, cos, sin, rq, dq, 1e-6)),
            q.numel() * 6 / 1e9)
        sc = torch.randn(131072, 128, device=dev)
        ms = timed(lambda: K.topk_rows(sc, 8))
        rows.append({"kernel": "topk_rows k=8", "shape": "131072x128", "ms": ms, "gbs": sc.numel() * 4 / 1e9 / ms * 1e3,
                     "of_peak": sc.numel() * 4 / 1e9 / ms * 1e3 / pk["hbm_gbs"], "library_ms": timed(lambda: sc.topk(8, dim=-1))})


def bench_scan(rows: list, pk: dict) -> None:
    """Gated delta rule, 8 rows x 4096 x 16 heads of 128 (the shape the reference quotes for its
    recurrence kernels): the chunk-scan kernel alone, and the whole `scan` forward + backward with
    the serial part on the kernel and as the chunk loop in PyTorch."""
    from ..models.layers import recurrent as R
    from . import functional as F_
    from . import scan as S_

    dev = "cuda"
    b, t, h, d = (2, 4096, 16, 128) if SMALL else (8, 4096, 16, 128)
    n = t // 64
    bf = lambda *shape, scale=1.0: (torch.randn(*shape, device=dev) * scale).bfloat16()
    a1, a4 = bf(b, h, n, 128, 128, scale=0.1), bf(b, h, n, 128, 128, scale=0.1)
    aux1, aux3 = bf(b, h, n, 128, 64, scale=0.1), bf(b, h, n, 64, 64, scale=0.1)
    v = bf(b, h, n, 64, 128)
    lam = torch.rand(b, h, n, 128, device=dev) * 0.5 + 0.5
    ms = timed(lambda: S_._run(a1, aux1, aux3, a4, v, lam, None, want_out=True, reverse=False), 5)
    # four chains of 128-row MMAs per chunk: K = 128, 64, 64, 128 over N = 128
    flops = 2.0 * b * h * n * 128 * 128 * (128 + 64 + 64 + 128)
    rows.append({"kernel": "chunk_scan (serial part, forward walk)", "shape": f"b{b} t{t} h{h} d{d}", "ms": ms,
                 "tflops": flops / ms / 1e9, "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})
    q = torch.nn.functional.normalize(torch.randn(b, t, h, d, device=dev), dim=-1).bfloat16().requires_grad_()
    k = torch.nn.functional.normalize(torch.randn(b, t, h, d, device=dev), dim=-1).bfloat16().requires_grad_()
    vv = torch.randn(b, t, h, d, device=dev).bfloat16().requires_grad_()
    g = (-torch.rand(b, t, h, 1, device=dev) * 0.1).bfloat16()
    beta = torch.rand(b, t, h, device=dev).bfloat16()

    def fwd_bwd():
        o, _ = R.delta_rule(q, k, vv, g, beta)
        o.float().sum().backward()
        q.grad = k.grad = vv.grad = None

    ms_kernel = timed(fwd_bwd, 3)
    F_.set_kernels(False)
    try:
        ms_loop = timed(fwd_bwd, 3)
    finally:
        F_.set_kernels(True)
    rows.append({"kernel": "gated delta rule fwd+bwd (scan on the kernel)", "shape": f"b{b} t{t} h{h} d{d}",
                 "ms": ms_kernel, "tflops": 0.0, "of_peak": 0.0, "library_ms": ms_loop})


def bench_muon(rows: list, pk: dict) -> None:
    """Muon's Newton–Schulz iteration (five quintic steps) on the framework's GEMM beside the
    same iteration on library matmuls."""
    from ..ops import functional as F_
    from ..train import optim

    for m, n in ((2048, 8192), (4096, 4096)):
        g = torch.randn(m, n, device="cuda")
        flops = 5 * (2.0 * m * m * n * 2 + 2.0 * m * m * m)
        ms = timed(lambda: optim.newton_schulz(g, 5))
        F_.set_kernels(False)
        ms_lib = timed(lambda: optim.newton_schulz(g, 5))
        F_.set_kernels(True)
        rows.append({"kernel": "muon newton_schulz x5", "shape": f"{m}x{n}", "ms": ms, "tflops": flops / ms / 1e9,
                     "library_ms": ms_lib, "of_peak": flops / ms / 1e9 / pk["bf16_tflops"]})


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true", help="profiler-sized shapes (gemm, attention)")
    ap.add_argument("--phases", action="store_true", help="attention backward: cycles per phase of its schedule")
    args = ap.parse_args()
    global SMALL, PHASES
    SMALL, PHASES = args.small, args.phases
    pk = peaks()
    rows: list = []
    for name, fn in (("gemm", bench_gemm), ("grouped", bench_grouped), ("attention", bench_attention),
                     ("memory", bench_memory_bound), ("scan", bench_scan), ("muon", bench_muon)):
        if not args.only or args.only in name:
            fn(rows, pk)
    K.check_status(torch.device("cuda"), "bench_kernels")
    print(f"peaks: {pk}")
    for r in rows:
        rate = f"{r['tflops']:.0f} TFLOP/s" if "tflops" in r else f"{r['gbs']:.0f} GB/s"
        lib = ""
        if "library_tflops" in r:
            lib = f"  library {r['library_tflops']:.0f} TFLOP/s"
        if "library_ms" in r:
            lib = f"  library {r['library_ms']:.3f} ms"
        print(f"{r['kernel']:<40} {r['shape']:<28} {r['ms']:8.3f} ms  {rate:>14}  {r['of_peak']:.2f} of {pk['source']} peak{lib}")
    if args.json:
        Path(args.json).write_text(json.dumps({"peaks": pk, "rows": rows}, indent=1))


if __name__ == "__main__":
    main()
