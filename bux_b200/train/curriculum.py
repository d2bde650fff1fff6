"""Curricula: settings that change at a step (seq_len / batch / data / RoPE) and
batch ramps, cut into *stretches* of constant shape.

Behaviour follows the reference (``src/bux/train/curriculum.py:28-228``): a phase
starts at a step or a share of the steps, phases go in order, a ramp grows the
batch linearly in multiples, and token accounting sums batch x seq_len per stretch.
"""

from __future__ import annotations

import itertools
from typing import NamedTuple, Sequence

CHANGES = ("seq_len", "batch", "data")
ROPE = {"rope_scaling": "scaling", "rope_base": "base"}


class Stretch(NamedTuple):
    start: int
    stop: int
    config: object  # TrainConfig with that stretch's seq_len, batch and data


def phases(t) -> list:
    """(first step, settings then) for the start of the run and of every phase."""
    out = [(0, t)]
    for ph in t.curriculum:
        changed = {k: getattr(ph, k) for k in CHANGES if getattr(ph, k) is not None}
        out.append((ph.start(t.steps), out[-1][1].model_copy(update=changed)))
    return out


def ropes(t) -> list:
    out = [(0, {})]
    for ph in t.curriculum:
        changed = {f: getattr(ph, k) for k, f in ROPE.items() if getattr(ph, k) is not None}
        out.append((ph.start(t.steps), {**out[-1][1], **changed}))
    return out


def rope_at(t, step: int) -> dict:
    return next(r for start, r in reversed(ropes(t)) if start <= step)


def ramped(ramp, batch: int, step: int) -> int:
    """Rows per step at `step` of a linear ramp, rounded down to the multiple."""
    if step >= ramp.steps:
        return batch
    grown = ramp.start + (batch - ramp.start) * step // ramp.steps
    mult = ramp.multiple or ramp.start
    return max(ramp.start, grown // mult * mult)


def _ramp_cuts(ramp, batch: int) -> list:
    mult, rise = ramp.multiple or ramp.start, batch - ramp.start
    sizes = range((ramp.start // mult + 1) * mult, batch, mult)
    return [-(-(v - ramp.start) * ramp.steps // rise) for v in sizes]


def check_phases(t) -> None:
    starts = [s for s, _ in phases(t)]
    for n, (before, start) in enumerate(itertools.pairwise(starts), 1):
        if start >= t.steps:
            raise ValueError(f"phase {n} starts at step {start}, and the run has {t.steps}")
        if start <= before:
            raise ValueError(
                f"phase {n} starts at step {start}, not after the phase before it "
                f"(step {before}): phases go in the order they start")
    ramp = t.batch_ramp
    for n, ph in enumerate(t.curriculum, 1):
        if ramp is not None and ph.batch is not None and starts[n] < ramp.steps:
            raise ValueError(
                f"phase {n} sets the batch at step {starts[n]}, before the batch ramp is "
                f"over at step {ramp.steps}")


def check_ramp(t) -> None:
    ramp = t.batch_ramp
    if ramp is None:
        return
    if ramp.start >= t.batch:
        raise ValueError(f"the batch ramp starts at {ramp.start} rows, not below the run's "
                         f"batch of {t.batch}, which it grows to")
    if ramp.steps > t.steps:
        raise ValueError(f"the batch ramp takes {ramp.steps} steps, and the run has {t.steps}")


def check(t) -> None:
    check_ramp(t)
    check_phases(t)


def stretches(t) -> tuple:
    check(t)
    starts = phases(t)
    cuts = {s for s, _ in starts}
    ramp = t.batch_ramp
    if ramp is not None:
        cuts.update(_ramp_cuts(ramp, t.batch), [ramp.steps])
    bounds = [*sorted(c for c in cuts if c < t.steps), t.steps]
    out: list = []
    for start, stop in itertools.pairwise(bounds):
        config = next(c for s, c in reversed(starts) if s <= start)
        if ramp is not None and start < ramp.steps:
            config = config.model_copy(update={"batch": ramped(ramp, t.batch, start)})
        if out and out[-1].config == config:
            out[-1] = out[-1]._replace(stop=stop)
        else:
            out.append(Stretch(start, stop, config))
    return tuple(out)


def varies(t) -> bool:
    return bool(t.curriculum) or t.batch_ramp is not None


def tokens(parts: Sequence, steps: int) -> int:
    total = 0
    for k, s in enumerate(parts):
        stop = steps if k == len(parts) - 1 else min(s.stop, steps)
        total += max(0, stop - s.start) * s.config.batch * s.config.seq_len
    return total


def si(n: float) -> str:
    for suffix, scale in (("", 1), ("k", 1e3), ("M", 1e6), ("B", 1e9)):
        shown = f"{n / scale:.3g}"
        if "e" not in shown:
            return shown + suffix
    return f"{n / 1e12:.3g}T"


def summary(t) -> str:
    shape = "" if varies(t) else f" × {t.batch} × {t.seq_len} tokens"
    return f"{t.steps:,} steps{shape} = {si(tokens(stretches(t), t.steps))} tokens"
