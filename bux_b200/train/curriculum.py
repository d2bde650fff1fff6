"""Curricula: a run whose shape changes over its steps.

Two things change a run's shape: *phases* (``curriculum = phase(at=..., seq_len=...,
batch=..., data=..., rope_scaling=..., rope_base=...)``), which switch settings at a step
or at a share of the steps, and the *batch ramp*, which grows the batch from a small start
to the run's batch over its first steps. `Timeline` lays both on one axis of steps;
`stretches` cuts that axis where anything changes, so that the trainer, the data feed and
the schedules can each walk ranges of steps over which batch, sequence length and data are
constant.

What it computes matches the reference (``train/curriculum.py:28-228`` there): phase
starts round a share of the steps to a step, a ramp's batch is linear in the step and
rounded down to its multiple, tokens are summed stretch by stretch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import NamedTuple, Sequence


class Stretch(NamedTuple):
    start: int
    stop: int
    config: object  # the TrainConfig with that range's seq_len, batch and data


@dataclass
class _Switch:
    """One phase on the timeline: its first step, the run's settings from then on and the
    RoPE settings in force from then on."""

    step: int
    config: object
    rope: dict


class Timeline:
    """A run's phases and ramp on the axis of steps."""

    SHAPE_FIELDS = ("seq_len", "batch", "data")
    ROPE_FIELDS = (("rope_scaling", "scaling"), ("rope_base", "base"))

    def __init__(self, t):
        self.t = t
        self.ramp = t.batch_ramp
        self.switches = [_Switch(0, t, {})]
        for phase in t.curriculum:
            last = self.switches[-1]
            shape = {}
            for field in self.SHAPE_FIELDS:
                value = getattr(phase, field)
                if value is not None:
                    shape[field] = value
            rope = dict(last.rope)
            for field, name in self.ROPE_FIELDS:
                value = getattr(phase, field)
                if value is not None:
                    rope[name] = value
            self.switches.append(_Switch(phase.start(t.steps), last.config.model_copy(update=shape), rope))

    # ---- lookups
    def switch_at(self, step: int) -> _Switch:
        current = self.switches[0]
        for sw in self.switches[1:]:
            if sw.step <= step:
                current = sw
        return current

    def ramp_rows(self, step: int) -> int:
        """Rows per step at `step` while the ramp runs, rounded down to its multiple."""
        ramp, full = self.ramp, self.t.batch
        if step >= ramp.steps:
            return full
        unit = ramp.multiple or ramp.start
        linear = ramp.start + (full - ramp.start) * step // ramp.steps
        return max(ramp.start, linear - linear % unit)

    def ramp_steps(self) -> list:
        """The steps at which the ramp's batch reaches each further multiple."""
        ramp, full = self.ramp, self.t.batch
        unit = ramp.multiple or ramp.start
        out = []
        size = (ramp.start // unit + 1) * unit
        while size < full:
            # the first step whose linear value is at least `size`
            out.append(-((ramp.start - size) * ramp.steps // (full - ramp.start)))
            size += unit
        return out

    def config_at(self, step: int):
        config = self.switch_at(step).config
        if self.ramp is not None and step < self.ramp.steps:
            config = config.model_copy(update={"batch": self.ramp_rows(step)})
        return config

    def boundaries(self) -> list:
        marks = {sw.step for sw in self.switches}
        if self.ramp is not None:
            marks.update(self.ramp_steps())
            marks.add(self.ramp.steps)
        return sorted(m for m in marks if m < self.t.steps) + [self.t.steps]

    # ---- validity
    def check_ramp(self) -> None:
        ramp, t = self.ramp, self.t
        if ramp is None:
            return
        if ramp.start >= t.batch:
            raise ValueError(f"the batch ramp starts at {ramp.start} rows, not below the run's "
                             f"batch of {t.batch}, which it grows to")
        if ramp.steps > t.steps:
            raise ValueError(f"the batch ramp takes {ramp.steps} steps, and the run has {t.steps}")

    def check_phases(self) -> None:
        t = self.t
        for n in range(1, len(self.switches)):
            start, before = self.switches[n].step, self.switches[n - 1].step
            if start >= t.steps:
                raise ValueError(f"phase {n} starts at step {start}, and the run has {t.steps}")
            if start <= before:
                raise ValueError(
                    f"phase {n} starts at step {start}, not after the phase before it "
                    f"(step {before}): phases go in the order they start")
        if self.ramp is None:
            return
        for n, phase in enumerate(t.curriculum, 1):
            start = self.switches[n].step
            if phase.batch is not None and start < self.ramp.steps:
                raise ValueError(
                    f"phase {n} sets the batch at step {start}, before the batch ramp is "
                    f"over at step {self.ramp.steps}")


# ---- the module's functions (what the compiler, the trainer and the CLI call)
def phases(t) -> list:
    """(first step, settings then) for the start of the run and of every phase."""
    return [(sw.step, sw.config) for sw in Timeline(t).switches]


def rope_at(t, step: int) -> dict:
    """The RoPE settings (``scaling``, ``base``) the phases have set by `step`."""
    return Timeline(t).switch_at(step).rope


def ramped(ramp, batch: int, step: int) -> int:
    line = Timeline.__new__(Timeline)
    line.ramp, line.t = ramp, _Rows(batch)
    return line.ramp_rows(step)


class _Rows:
    def __init__(self, batch: int):
        self.batch = batch


def check_ramp(t) -> None:
    Timeline(t).check_ramp()


def check_phases(t) -> None:
    Timeline(t).check_phases()


def check(t) -> None:
    line = Timeline(t)
    line.check_ramp()
    line.check_phases()


def stretches(t) -> tuple:
    """Ranges of steps with constant batch, sequence length and data, in order."""
    line = Timeline(t)
    line.check_ramp()
    line.check_phases()
    marks = line.boundaries()
    out: list = []
    for start, stop in zip(marks, marks[1:]):
        config = line.config_at(start)
        if out and out[-1].config == config:
            out[-1] = Stretch(out[-1].start, stop, config)
        else:
            out.append(Stretch(start, stop, config))
    return tuple(out)


def varies(t) -> bool:
    return bool(t.curriculum) or t.batch_ramp is not None


def tokens(parts: Sequence, steps: int) -> int:
    """Tokens the first `steps` steps read (the last range is open-ended)."""
    total, last = 0, len(parts) - 1
    for k, part in enumerate(parts):
        end = steps if k == last else min(part.stop, steps)
        if end > part.start:
            total += (end - part.start) * part.config.batch * part.config.seq_len
    return total


def si(n: float) -> str:
    """Three significant digits with an SI suffix (1.31B, 819k)."""
    for suffix, scale in (("", 1), ("k", 1e3), ("M", 1e6), ("B", 1e9)):
        shown = f"{n / scale:.3g}"
        if "e" not in shown:
            return shown + suffix
    return f"{n / 1e12:.3g}T"


def summary(t) -> str:
    shape = "" if varies(t) else f" × {t.batch} × {t.seq_len} tokens"
    return f"{t.steps:,} steps{shape} = {si(tokens(stretches(t), t.steps))} tokens"
