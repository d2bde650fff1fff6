"""Where a run's metrics go: the console, ``metrics.jsonl``, trackers.

The console line and the JSONL record follow the reference's formats
(``train/sinks.py:81-276``, sample in ``docs/training/running.md:14-18``) so that run
directories are interchangeable: ``<name> step 10/50  loss 6.2429  lr 3.00e-03 ...``.
Only the main process writes. A resumed run's JSONL drops the lines past its step.
"""

from __future__ import annotations

import json
import math
import time
from pathlib import Path
from typing import Callable, Mapping, Optional

from .. import runtime


def is_main_process() -> bool:
    return runtime.rank() == 0


def echo(line: str) -> None:
    print(line, flush=True)


def hms(seconds: float) -> str:
    if not math.isfinite(seconds):
        return "?"
    m, s = divmod(round(seconds), 60)
    return f"{m // 60}:{m % 60:02d}:{s:02d}"


class Sink:
    def write(self, step: int, scalars: Mapping) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def histograms(self, step: int, data: Mapping) -> None:
        pass

    def close(self) -> None:
        pass


class Console(Sink):
    FORMATS = {
        "loss": "loss {:.4f}",
        "mtp": "mtp {:.4f}",
        "lr": "lr {:.2e}",
        "grad_norm": "grad {:.3f}",
        "tokens_per_s": "{:,.0f} tok/s",
        "mfu": "mfu {:.1%}",
        "eval_loss": "eval loss {:.4f}",
        "eval_bpb": "eval bpb {:.4f}",
        "time/step_ms": "{:.0f} ms/step",
        "time/data_ms": "data {:.1f} ms",
        "mem/peak_gib": "mem {:.1f} GiB",
        "time/compile_s": "compiled in {:.1f}s",
    }
    FINITE = ("loss", "grad_norm", "eval_loss")

    def __init__(self, name: str, steps: int, out: Callable = echo, formats: Optional[Mapping] = None):
        self.name, self.steps, self.out = name, steps, out
        self.formats = dict(formats or self.FORMATS)
        self.started = time.perf_counter()

    def write(self, step: int, scalars: Mapping) -> None:
        if not is_main_process():
            return
        shown = [f.format(scalars[k]) for k, f in self.formats.items() if k in scalars]
        for k in scalars:  # named evals: web_loss, web_bpb
            if k not in self.formats and (k.endswith("_loss") or k.endswith("_bpb")) and "/" not in k \
                    and k.split("_")[0] not in ("balance", "indexer", "z", "mtp1", "mtp2", "mtp3"):
                shown.append(f"{k.replace('_', ' ')} {scalars[k]:.4f}")
        if not shown:
            return
        width = len(str(self.steps))
        tail = []
        if "time/step_ms" in scalars:
            spent = time.perf_counter() - self.started
            left = scalars["time/step_ms"] / 1000 * (self.steps - step)
            tail.append(f"{hms(spent)} < {hms(left)}")
        bad = [k for k in self.FINITE if k in scalars and not math.isfinite(scalars[k])]
        if bad:
            tail.append(f"!! not finite: {', '.join(bad)}")
        self.out(f"{self.name} step {step:>{width}}/{self.steps}  " + "  ".join([*shown, *tail]))


class JSONL(Sink):
    """``metrics.jsonl`` (+ ``histograms.jsonl``), one record per logged step."""

    def __init__(self, folder, resume_step: Optional[int] = None):
        self.folder = Path(folder)
        self.path = self.folder / "metrics.jsonl"
        self.hist_path = self.folder / "histograms.jsonl"
        if is_main_process():
            self.folder.mkdir(parents=True, exist_ok=True)
            if resume_step is not None:
                for p in (self.path, self.hist_path):
                    self._drop_after(p, resume_step)
            elif self.path.exists():
                self.path.unlink()

    @staticmethod
    def _drop_after(path: Path, step: int) -> None:
        if not path.exists():
            return
        kept = []
        for line in path.read_text().splitlines():
            try:
                if json.loads(line).get("step", 0) <= step:
                    kept.append(line)
            except json.JSONDecodeError:
                continue  # a half-written last line of a killed run
        path.write_text("".join(k + "\n" for k in kept))

    def write(self, step: int, scalars: Mapping) -> None:
        if not is_main_process():
            return
        with self.path.open("a") as f:
            f.write(json.dumps({"step": step, **{k: float(v) for k, v in scalars.items()}}) + "\n")

    def histograms(self, step: int, data: Mapping) -> None:
        if not is_main_process() or not data:
            return
        with self.hist_path.open("a") as f:
            f.write(json.dumps({"step": step, **data}) + "\n")


class LatestMetrics(Sink):
    """Keeps the last value of every metric (what a search's objective reads)."""

    def __init__(self):
        self.latest: dict = {}
        self.history: list = []

    def write(self, step: int, scalars: Mapping) -> None:
        self.latest.update(scalars)
        self.history.append((step, dict(scalars)))


def read_metrics(folder) -> list:
    path = Path(folder) / "metrics.jsonl"
    if not path.exists():
        return []
    out = []
    for line in path.read_text().splitlines():
        try:
            out.append(json.loads(line))
        except json.JSONDecodeError:
            pass
    return out
