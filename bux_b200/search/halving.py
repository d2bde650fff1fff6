"""Asynchronous successive halving (ASHA) and Hyperband brackets.

A trial runs rung 0's steps; it is promoted to the next rung (eta times the steps) when
it is in the best 1/eta of the results its rung has seen. `next_job` promotes before it
starts new trials, so workers never wait for a rung to fill."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class Bracket:
    eta: int
    rungs: int
    first: int = 0                       # the rung new trials of this bracket start at
    results: dict = field(default_factory=dict)    # rung → {trial: objective}
    promoted: dict = field(default_factory=dict)   # rung → set of trials sent up

    def report(self, trial: int, rung: int, value: float) -> None:
        self.results.setdefault(rung, {})[trial] = value

    def promotable(self) -> Optional[tuple]:
        """(trial, next rung) of the best not yet promoted result that has earned it,
        highest rung first."""
        for rung in range(self.rungs - 2, self.first - 1, -1):
            seen = self.results.get(rung, {})
            done = self.promoted.setdefault(rung, set())
            keep = len(seen) // self.eta
            ranked = sorted(seen, key=lambda t: seen[t])[:keep]
            for t in ranked:
                if t not in done:
                    done.add(t)
                    return t, rung + 1
        return None


class Halving:
    def __init__(self, config, steps: int):
        self.c, self.steps = config, steps
        self.brackets = [Bracket(config.eta, config.rungs, first=b) for b in range(config.brackets)]
        self.where: dict = {}  # trial → bracket index

    def rung_steps(self, rung: int) -> int:
        return self.c.steps(self.steps, rung)

    def next_job(self, new_trial: Optional[int]) -> Optional[tuple]:
        """(trial, rung, steps): a promotion if any bracket has one, else `new_trial` at its
        bracket's first rung (brackets take new trials round-robin)."""
        for b in self.brackets:
            p = b.promotable()
            if p is not None:
                return p[0], p[1], self.rung_steps(p[1])
        if new_trial is None:
            return None
        i = new_trial % len(self.brackets)
        self.where[new_trial] = i
        first = self.brackets[i].first
        return new_trial, first, self.rung_steps(first)

    def report(self, trial: int, rung: int, value: float) -> None:
        self.brackets[self.where.get(trial, 0)].report(trial, rung, value)
