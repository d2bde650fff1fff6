"""``observe(every=N, histograms=...)``: per-layer statistics every N steps.

For every parameter: RMS of the weight, of its gradient (where one is still held) and of
the last update, as ``param/<path>``, ``grad/<path>``, ``update/<path>``. From the model's
forward of an observed step (`bux_b200.models.observe`): the residual stream after every
outer branch (``act/rms/gqa.03``, ``act/update_rms/...``, ``act/max_abs/...``,
``act/kurtosis/...``), every MoE's routing (``router/max_load/moe.01``, ``router/dead/...``,
``router/entropy/...``, ``router/z/...``) and a sample of every attention's logits
(``attn/logit_max/...``, ``attn/entropy/...``). With `histograms`, log2-magnitude histograms of
the weights, of the gradients still held and of the stream after each branch go to
``histograms.jsonl``.
Reference: ``train/observe.py``, ``architecture/observe.py``.
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


def gradient_stats(trainer, histograms: bool) -> dict:
    """name -> (RMS, log2-magnitude histogram or None) of every gradient the step still holds
    (this rank's part of it, under sharding). The trainer calls it on an observed step between
    the backward and the update."""
    out = {}
    for n, p in trainer.model.named_parameters():
        g = trainer.optimizer.grad_of(p)
        if g is not None:
            out[n] = (rms(g), log2_histogram(g) if histograms else None)
    return out


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
        self.reports: dict = {}     # step -> what its forward and its update showed
        trainer.pre_step.append(self._arm_for)   # before the step is launched, not a step later

    def _arm_for(self, step: int) -> None:
        self._collect()   # the step before may have been an observed one
        self.armed = step % self.every == 0
        self.armed_step = step
        self.trainer.observing = {"histograms": bool(self.c.histograms)} if self.armed else None
        if self.armed:
            self.before = {n: p.detach().float().clone() for n, p in self.trainer.model.named_parameters()}

    def _collect(self) -> None:
        """After an observed step has been launched: what it showed, kept until its hook call
        (the trainer launches the next step before it calls the hooks of this one)."""
        if not self.armed:
            return
        tr = self.trainer
        stats = {f"act/{k}": v for k, v in self.acts.items()}
        stats.update({k: float(v) for k, v in tr.observed.items()})
        streams = {k: v.tolist() for k, v in tr.observed_histograms.items()}
        tr.observed, tr.observed_histograms = {}, {}
        weights, grads = {}, {}
        seen, tr.observed_gradients = tr.observed_gradients, {}
        for n, p in tr.model.named_parameters():
            stats[f"param/{n}"] = rms(p)
            if n in seen:
                stats[f"grad/{n}"] = seen[n][0]
                if seen[n][1] is not None:
                    grads[n] = seen[n][1]
            if n in self.before:
                stats[f"update/{n}"] = rms(p.detach().float() - self.before[n])
            if self.c.histograms:
                weights[n] = log2_histogram(p)
        self.reports[self.armed_step] = (stats, weights, streams, grads)
        self.acts, self.before, self.armed = {}, {}, False

    def due(self, step: int, trainer, last: bool = False) -> bool:
        return True

    def __call__(self, step: int, scalars: dict, trainer, sinks) -> None:
        if step == getattr(self, "armed_step", None):
            self._collect()   # the run's last step: nothing was launched after it
        if step in self.reports:
            stats, weights, streams, grads = self.reports.pop(step)
            for s in sinks or ():
                s.write(step, stats)
            if self.c.histograms and self.folder is not None:
                with open(self.folder / "histograms.jsonl", "a") as f:
                    f.write(json.dumps({"step": step, "histograms": weights, "stream": streams, "gradients": grads}) + "\n")

    def stop(self, trainer, sinks) -> None:
        for h in self.handles:
            h.remove()
        if self._arm_for in trainer.pre_step:
            trainer.pre_step.remove(self._arm_for)
        trainer.observing = None
