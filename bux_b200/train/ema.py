"""A tail EMA of the weights, which a run ends on (``ema(window=..., blend=...)``).

The average (fp32, one tensor per parameter, sharded as the parameter is) is seeded with
the weights after the first step of the window and moves toward every later step's by
``2 / (window + 1)``; it lives in the optimizer's state (``ema/<name>``), so checkpoints
keep it and a run resumes inside its window. `Ship` ends the run on
``last + blend·(average − last)`` before the last step's eval and checkpoint read the
weights. Reference: ``train/ema.py``.
"""

from __future__ import annotations

import torch

from .hooks import Hook


def first(config, steps: int) -> int:
    """The step whose weights seed the average, of a run of `steps`."""
    return max(steps - config.steps(steps) + 1, 1)


class Ship(Hook):
    every = 1

    def __init__(self, config, steps: int):
        self.c, self.steps = config, steps
        self.first_step = first(config, steps)
        self.rate = 2.0 / (config.steps(steps) + 1)
        self.shipped = False

    def due(self, step: int, trainer, last: bool = False) -> bool:
        return step >= self.first_step

    @torch.no_grad()
    def __call__(self, step: int, scalars: dict, trainer, sinks) -> None:
        opt = trainer.optimizer
        for name, p in trainer.model.named_parameters():
            if not p.requires_grad:
                continue
            st = opt.state.setdefault(name, {})
            w = st.get("master", p.data).float()
            if "ema" not in st or step == self.first_step:
                st["ema"] = w.clone()
            else:
                st["ema"].lerp_(w, self.rate)
        if step >= self.steps and not self.shipped:
            self.ship(trainer)

    @torch.no_grad()
    def ship(self, trainer) -> None:
        """weights ← last + blend·(average − last)"""
        opt = trainer.optimizer
        for name, p in trainer.model.named_parameters():
            st = opt.state.get(name, {})
            if "ema" not in st:
                continue
            target = st.get("master", p.data)
            target.copy_(torch.lerp(target.float(), st["ema"], self.c.blend).to(target.dtype))
            if "master" in st:
                p.data.copy_(target.to(p.dtype))
        self.shipped = True
