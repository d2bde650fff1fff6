"""Reads a profiler trace and says what a step spent communicating and idle.

Kernels are classed by name into communication (NCCL kernels and this library's own
fused-communication kernels) and compute; intervals are merged per class;
``exposed_comm_ms`` is communication time not covered by compute, ``idle_ms`` the
time neither runs. Reference: ``train/trace.py:38-128`` (there over xplane traces).
"""

from __future__ import annotations

import json
from pathlib import Path

COMM_MARKERS = ("nccl", "bux_comm", "ag_gemm", "gemm_rs", "moe_dispatch", "moe_combine", "all_reduce",
                "allreduce", "reduce_scatter", "all_gather", "ep_push", "ep_pull", "ep_wait", "ep_signal", "tp_push",
                "tp_pull")


def is_comm(name: str) -> bool:
    low = name.lower()
    return any(m in low for m in COMM_MARKERS)


def merge(intervals: list) -> list:
    out: list = []
    for a, b in sorted(intervals):
        if out and a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return out


def length(intervals: list) -> float:
    return sum(b - a for a, b in intervals)


def subtract(a: list, b: list) -> list:
    """Parts of merged intervals `a` not covered by merged intervals `b`."""
    out, j = [], 0
    for s, e in a:
        cur = s
        while j < len(b) and b[j][1] <= cur:
            j += 1
        k = j
        while k < len(b) and b[k][0] < e:
            if b[k][0] > cur:
                out.append([cur, b[k][0]])
            cur = max(cur, b[k][1])
            k += 1
        if cur < e:
            out.append([cur, e])
    return out


def classify(events: list) -> dict:
    """events: (name, start_us, duration_us) of device kernels. Returns totals in ms."""
    comm = merge([[s, s + d] for n, s, d in events if is_comm(n)])
    comp = merge([[s, s + d] for n, s, d in events if not is_comm(n)])
    if not comm and not comp:
        return {"comm_ms": 0.0, "exposed_comm_ms": 0.0, "idle_ms": 0.0}
    lo = min(x[0] for x in comm + comp)
    hi = max(x[1] for x in comm + comp)
    busy = merge(comm + comp)
    return {"comm_ms": length(comm) / 1000, "exposed_comm_ms": length(subtract(comm, comp)) / 1000,
            "idle_ms": ((hi - lo) - length(busy)) / 1000}


def comm_ms(path, steps: int = 1) -> dict:
    """Per-step comm / exposed comm / idle from a chrome trace written by the profiler."""
    data = json.loads(Path(path).read_text())
    events = [(e.get("name", ""), float(e["ts"]), float(e.get("dur", 0.0)))
              for e in data.get("traceEvents", [])
              if e.get("ph") == "X" and e.get("cat", "").lower() in ("kernel", "gpu_memcpy", "gpu_memset")]
    totals = classify(events)
    return {k: v / max(steps, 1) for k, v in totals.items()}
