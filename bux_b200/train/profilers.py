"""``profile(tool=...)``: which profiler a run is traced by, and the capture window.

``torch`` (alias ``jax``, kept so files written for the reference still read) traces in
process with the CUPTI-backed torch profiler. ``nsys`` and ``ncu`` need the run to be
relaunched under the tool: `command` builds that command line (with the clock control
left alone for ncu), and inside the relaunched process `start` / `stop` bracket the
steps with ``cudaProfilerStart/Stop`` so the tool captures only them. ``BUX_PROFILER``
names the tool a process already runs under. Reference: ``train/profilers.py:38-143``.
"""

from __future__ import annotations

import os
import shutil
import sys

BUX_PROFILER = "BUX_PROFILER"

TOOLS = {
    "torch": None,
    "jax": None,
    "nsys": ["nsys", "profile", "--capture-range=cudaProfilerApi", "--capture-range-end=stop", "--trace=cuda,nvtx",
             "--force-overwrite=true", "-o", "{out}/profile"],
    "ncu": ["ncu", "--clock-control", "none", "--profile-from-start", "off", "--set", "full", "-f", "-o", "{out}/profile"],
}
ONE_GPU = {"ncu"}  # replays kernels: never around a multi-rank job


def available(tool: str) -> bool:
    return TOOLS.get(tool) is None or shutil.which(TOOLS[tool][0]) is not None


def under() -> str:
    """The external tool this process runs under, "" for none."""
    return os.environ.get(BUX_PROFILER, "")


def command(tool: str, out, argv=None, options: str = "") -> list:
    """The command line that reruns this program under `tool`."""
    if tool not in TOOLS:
        raise ValueError(f"profile(tool={tool!r}): one of {', '.join(TOOLS)}")
    if TOOLS[tool] is None:
        raise ValueError(f"profile(tool={tool!r}) traces in process: nothing to relaunch")
    if not available(tool):
        raise FileNotFoundError(f"profile(tool={tool!r}): `{TOOLS[tool][0]}` is not on PATH")
    if tool in ONE_GPU and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise ValueError(f"profile(tool={tool!r}) replays kernels: run it on one GPU")
    head = [a.format(out=out) for a in TOOLS[tool]] + (options.split() if options else [])
    return head + [sys.executable, *(argv if argv is not None else sys.argv)]


def start() -> None:
    import torch

    if torch.cuda.is_available():
        torch.cuda.profiler.start()   # cudaProfilerStart


def stop() -> None:
    import torch

    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()    # cudaProfilerStop
