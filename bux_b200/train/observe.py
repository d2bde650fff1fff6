"""``observe(every=N, histograms=...)``: per-layer statistics every N steps.

For every parameter: RMS of the weight, of its gradient (where one is still held) and of
the last update, as ``param/<path>``, ``grad/<path>``, ``update/<path>``; for every module
that is a block of a repeat: RMS of its output activations (``act/<path>``) from a
forward hook that is armed only on observed steps. With `histograms`, log2-magnitude
histograms of weights go to ``histograms.jsonl``. Reference: ``train/observe.py``,
``architecture/observe.py``.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .hooks import Hook


def rms(t: torch.Tensor) -> float:
    return float(t.detach().float().square().mean().sqrt())


def log2_histogram(t: torch.Tensor, lo: int = -24, hi: int = 8) -> list:
    mag = t.detach().float().abs().flatten()
    e = torch.floor(torch.log2(mag.clamp_min(2.0 ** lo))).clamp(lo, hi).long() - lo
    return torch.bincount(e, minlength=hi - lo + 1).tolist()


class Observe(Hook):
    def __init__(self, config, folder=None):
        self.c, self.every = config, config.every
        self.folder = None if folder is None else Path(folder)
        self.acts: dict = {}
        self.handles: list = []
        self.before: dict = {}

    def start(self, trainer) -> None:
        from ..models.graph import Repeated

        for path, m in trainer.model.named_modules():
            if isinstance(m, Repeated):
                for i, block in enumerate(m.items):
                    name = f"{path}.items.{i}"

                    def hook(mod, args, out, name=name):
                        if self.armed and isinstance(out, torch.Tensor):
                            self.acts[name] = rms(out)

                    self.handles.append(block.register_forward_hook(hook))
        self.armed = False
        self.trainer = trainer
        self._arm_for(trainer.step + 1)

    def _arm_for(self, step: int) -> None:
        self.armed = step % self.every == 0
        if self.armed:
            self.before = {n: p.detach().float().clone() for n, p in self.trainer.model.named_parameters()}

    def due(self, step: int, trainer, last: bool = False) -> bool:
        return True

    def __call__(self, step: int, scalars: dict, trainer, sinks) -> None:
        if step % self.every == 0:
            stats = {f"act/{k}": v for k, v in self.acts.items()}
            for n, p in trainer.model.named_parameters():
                stats[f"param/{n}"] = rms(p)
                g = trainer.optimizer.grad_of(p)
                if g is not None:
                    stats[f"grad/{n}"] = rms(g)
                if n in self.before:
                    stats[f"update/{n}"] = rms(p.detach().float() - self.before[n])
            for s in sinks or ():
                s.write(step, stats)
            if self.c.histograms and self.folder is not None:
                with open(self.folder / "histograms.jsonl", "a") as f:
                    f.write(json.dumps({"step": step, "histograms": {
                        n: log2_histogram(p) for n, p in trainer.model.named_parameters()}}) + "\n")
            self.acts, self.before = {}, {}
        self._arm_for(step + 1)

    def stop(self, trainer, sinks) -> None:
        for h in self.handles:
            h.remove()
