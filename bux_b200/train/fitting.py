"""``remat=auto``: the cheapest activation-checkpointing preset that fits the device.

The reference compiles the candidates side by side and reads their memory from the
compiler (``train/fitting.py`` there: `MARGIN`, `Fitting`). Here a candidate is tried by
running one real step under the CUDA allocator's peak counter: presets are ordered by
recomputation cost, and the first whose peak stays within `MARGIN` of the device's
memory is kept (an out-of-memory error just moves on to the next preset; the trial
steps' effect on weights and optimizer state is undone from a snapshot).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

MARGIN = 0.97

#: (name, remat, keep_attention, offload): cheapest recomputation first
CANDIDATES = (
    ("none", False, False, False),
    ("block, attention kept", True, True, False),
    ("block", True, False, False),
    ("block, inputs on the host", True, False, True),
)


@dataclass
class Fitting:
    name: str
    peak_bytes: Optional[int]
    tried: list


def _default_probe(trainer, batch) -> int:
    dev = trainer.device
    torch.cuda.reset_peak_memory_stats(dev)
    trainer.train_step(batch)
    torch.cuda.synchronize(dev)
    return torch.cuda.max_memory_allocated(dev)


def fit(trainer, batch, capacity: Optional[int] = None, probe: Optional[Callable] = None) -> Fitting:
    """Sets the model's checkpointing to the first candidate that fits and returns it."""
    if capacity is None:
        capacity = torch.cuda.get_device_properties(trainer.device).total_memory
    probe = probe or _default_probe
    snapshot = trainer.state() if probe is _default_probe else None
    tried = []
    chosen = None
    for name, remat, keep, offload in CANDIDATES:
        trainer.model.set_remat(remat, offload=offload, keep_attention=keep)
        try:
            peak = probe(trainer, batch)
        except torch.OutOfMemoryError:
            peak = None
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        tried.append((name, peak))
        if snapshot is not None:
            trainer.load(snapshot)
        if peak is not None and peak <= MARGIN * capacity:
            chosen = Fitting(name, peak, tried)
            break
    if chosen is None:
        raise MemoryError("no checkpointing preset fits this device: " +
                          ", ".join(f"{n}: {'out of memory' if p is None else f'{p / 2**30:.1f} GiB'}" for n, p in tried))
    return chosen
