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


def device_events(path) -> dict:
    """device id → [(name, start_us, duration_us)] of the kernels and copies in a chrome trace
    written by the profiler (one entry when the trace does not say which device ran what)."""
    data = json.loads(Path(path).read_text())
    out: dict = {}
    for e in data.get("traceEvents", []):
        if e.get("ph") != "X" or e.get("cat", "").lower() not in ("kernel", "gpu_memcpy", "gpu_memset"):
            continue
        device = (e.get("args") or {}).get("device", e.get("pid", 0))
        out.setdefault(device, []).append((e.get("name", ""), float(e["ts"]), float(e.get("dur", 0.0))))
    return out


def comm_ms(path, steps: int = 1) -> dict:
    """Per-step comm / exposed comm / idle of a trace: each device's kernels are classed on
    their own timeline (one GPU's collective does not hide under another GPU's compute), and
    the numbers are the mean over the devices."""
    per_device = [classify(events) for events in device_events(path).values()] or [classify([])]
    n = len(per_device) * max(steps, 1)
    return {k: sum(d[k] for d in per_device) / n for k in per_device[0]}


def kernels(path, top: int = 20) -> list:
    """The trace's kernels by total time: (name, launches, total ms, share of the busy time)."""
    totals: dict = {}
    for events in device_events(path).values():
        for name, _, dur in events:
            n, t = totals.get(name, (0, 0.0))
            totals[name] = (n + 1, t + dur)
    whole = sum(t for _, t in totals.values()) or 1.0
    rows = sorted(totals.items(), key=lambda kv: -kv[1][1])[:top]
    return [(name, n, t / 1000, t / whole) for name, (n, t) in rows]


def latest(folder, host: str = None):
    """The newest trace file under a run's ``profile/`` folder (of `host` when given), or None."""
    found = [p for p in Path(folder).rglob("*.json") if host is None or host in p.name]
    return max(found, key=lambda p: p.stat().st_mtime) if found else None
