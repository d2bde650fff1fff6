"""Pipeline schedules as tables: for each stage, the ordered list of what it runs.

An entry is ``(op, microbatch)`` with op "F" (forward), "B" (backward; with a split
backward only the input gradient) or "W" (the weight gradient of a split backward).
Reference: ``parallel/schedule.py:60-280`` (`Table`, `lockstep`, `one_f_one_b`,
`zero_bubble_h1`, `TABLES`), ``parallel/pipeline.py:70`` (`bubble`).
"""

from __future__ import annotations


def bubble(stages: int, microbatches: int, rounds: int = 1) -> float:
    """Share of a step a stage idles: (S-1) / (M·rounds + S-1)."""
    if stages <= 1:
        return 0.0
    return (stages - 1) / (microbatches * rounds + stages - 1)


def gpipe(stages: int, microbatches: int) -> list:
    """Every forward, then every backward (most recent activations freed last)."""
    return [[("F", m) for m in range(microbatches)] + [("B", m) for m in range(microbatches)]
            for _ in range(stages)]


def one_f_one_b(stages: int, microbatches: int) -> list:
    """Stage s warms up with S-1-s forwards, then alternates one forward and one
    backward, then drains: at most S-s microbatches are alive on stage s."""
    table = []
    for s in range(stages):
        warm = min(stages - 1 - s, microbatches)
        ops = [("F", m) for m in range(warm)]
        f, b = warm, 0
        while f < microbatches:
            ops.append(("F", f))
            f += 1
            ops.append(("B", b))
            b += 1
        while b < microbatches:
            ops.append(("B", b))
            b += 1
        table.append(ops)
    return table


def zero_bubble_h1(stages: int, microbatches: int) -> list:
    """1F1B with the backward split: the weight gradient W of a microbatch is delayed to
    fill the drain's idle slots (ZB-H1: same activation memory as 1F1B)."""
    table = []
    for s in range(stages):
        warm = min(stages - 1 - s, microbatches)
        ops = [("F", m) for m in range(warm)]
        f, b, w = warm, 0, 0
        while f < microbatches:
            ops.append(("F", f))
            f += 1
            ops.append(("B", b))
            b += 1
            if b - w > s:  # keep at most s weight gradients pending: they fill the drain
                ops.append(("W", w))
                w += 1
        while b < microbatches:
            ops.append(("B", b))
            b += 1
            if w < b - 0 and b - w > max(0, s - (microbatches - b)):
                ops.append(("W", w))
                w += 1
        while w < microbatches:
            ops.append(("W", w))
            w += 1
        table.append(ops)
    return table


TABLES = {"gpipe": gpipe, "circular": gpipe, "1f1b": one_f_one_b, "zbh1": zero_bubble_h1}


def check(table: list, microbatches: int) -> None:
    """Every stage runs each microbatch's F before its B before its W, exactly once."""
    for s, ops in enumerate(table):
        seen = {"F": set(), "B": set(), "W": set()}
        for op, m in ops:
            if op == "B" and m not in seen["F"]:
                raise AssertionError(f"stage {s}: B{m} before F{m}")
            if op == "W" and m not in seen["B"]:
                raise AssertionError(f"stage {s}: W{m} before B{m}")
            if m in seen[op]:
                raise AssertionError(f"stage {s}: {op}{m} twice")
            seen[op].add(m)
        if seen["F"] != set(range(microbatches)) or seen["B"] != set(range(microbatches)):
            raise AssertionError(f"stage {s}: not every microbatch runs")


def alive(ops: list) -> int:
    """Most microbatches a stage holds activations of at once."""
    cur = peak = 0
    for op, _ in ops:
        if op == "F":
            cur += 1
            peak = max(peak, cur)
        elif op == "B":
            cur -= 1
    return peak
