"""The search driver: proposes trials, records them in ``<out>/<name>-search-<key>/
trials.jsonl``, resumes from that file, and writes ``best.bux`` (the best trial's run as
source). Trials are trained by a `train` callable (the launcher's queue in ``bux
launch``, or in-process), and the objective is read from the run's latest metrics."""

from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path
from typing import Callable, Optional

import numpy as np

from ..config import training as T
from ..lang.printer import run_to_source
from . import gp, tpe
from .halving import Halving
from .methods import POINTS
from .space import Cube


def objective_of(config, metrics: dict) -> Optional[float]:
    """The weighted sum of the objective's terms (lower is better); None if a metric is
    missing or not a number."""
    if config is None:
        v = metrics.get("eval/loss", metrics.get("loss"))
        return None if v is None or not math.isfinite(v) else float(v)
    total = config.constant
    for term in config.terms:
        v = metrics.get(term.metric)
        if v is None or not math.isfinite(v):
            return None
        total += term.weight * float(v)
    return total


class Search:
    def __init__(self, space, out="runs"):
        self.space = space
        run = space.run
        self.config: T.SearchConfig = run.train.search or T.SearchConfig()
        self.cube = Cube(space.dimensions)
        key = hashlib.sha256(json.dumps({"run": run.id, "dims": self.cube.names,
                                         "search": self.config.model_dump(mode="json")},
                                        sort_keys=True).encode()).hexdigest()[:10]
        self.folder = Path(out) / f"{run.name}-search-{key}"
        self.folder.mkdir(parents=True, exist_ok=True)
        self.path = self.folder / "trials.jsonl"
        self.trials: list = []
        if self.path.exists():
            for line in self.path.read_text().splitlines():
                if line.strip():
                    self.trials.append(json.loads(line))
        self.halving = Halving(self.config.halving, run.train.steps) if self.config.halving else None
        if self.halving:
            for t in self.trials:
                self.halving.where.setdefault(t["trial"], t["trial"] % len(self.halving.brackets))
                if t.get("objective") is not None:
                    self.halving.report(t["trial"], t.get("rung", 0), t["objective"])
        self.pending: dict = {}

    # ------------------------------------------------------------------ proposing
    def _finished(self):
        last: dict = {}
        for t in self.trials:  # a trial's highest rung speaks for it
            if t.get("objective") is not None:
                last[t["trial"]] = t
        xs = [self.cube.unit(t["values"]) for t in last.values()]
        ys = [t["objective"] for t in last.values()]
        return (np.array(xs), np.array(ys)) if xs else (np.empty((0, len(self.cube))), np.empty(0))

    def point(self, index: int) -> np.ndarray:
        m = self.config.method
        dims, seed = len(self.cube), self.config.seed
        rng = np.random.default_rng((seed, index, 7))
        x, y = self._finished()
        if m.type in POINTS:
            return POINTS[m.type](index, dims, seed)
        if len(y) < m.startup:
            return POINTS["halton" if dims <= 20 else "random"](index, dims, seed)
        if m.type == "tpe":
            cats = self.cube.categorical()
            opts = [len(s.options) if c else 0 for s, c in zip(self.cube.spaces, cats)]
            return tpe.suggest(x, y, dims, rng, m.gamma, m.candidates, m.multivariate, cats, opts)
        pending = np.array([self.cube.unit(v) for v in self.pending.values()]) if self.pending else None
        return gp.suggest(x, y, dims, rng, m.acquisition, m.beta, pending)

    def started(self) -> int:
        return len({t["trial"] for t in self.trials} | set(self.pending))

    def next_job(self) -> Optional[dict]:
        """{"trial", "rung", "steps", "values", "run"} or None when the budget is spent."""
        new = self.started() if self.started() < self.config.trials else None
        if self.halving is not None:
            job = self.halving.next_job(new)
            if job is None:
                return None
            trial, rung, steps = job
        else:
            if new is None:
                return None
            trial, rung, steps = new, 0, None
        known = next((t["values"] for t in self.trials if t["trial"] == trial), None) or self.pending.get(trial)
        values = known or self.cube.values(self.point(trial))
        self.pending[trial] = values
        run = self.space.trial(values, steps)
        return {"trial": trial, "rung": rung, "steps": steps, "values": values, "run": run}

    def report(self, job: dict, metrics: dict) -> Optional[float]:
        value = objective_of(self.space.run.train.objective, metrics)
        rec = {"trial": job["trial"], "rung": job["rung"], "steps": job["steps"], "values": job["values"],
               "run": job["run"].id, "objective": value}
        self.trials.append(rec)
        with open(self.path, "a") as f:
            f.write(json.dumps(rec, default=float) + "\n")
        self.pending.pop(job["trial"], None)
        if self.halving is not None and value is not None:
            self.halving.report(job["trial"], job["rung"], value)
        self._write_best()
        return value

    # ------------------------------------------------------------------ results
    def best(self) -> Optional[dict]:
        done = [t for t in self.trials if t.get("objective") is not None]
        if not done:
            return None
        top_rung = max(t.get("rung", 0) for t in done)
        return min((t for t in done if t.get("rung", 0) == top_rung), key=lambda t: t["objective"])

    def _write_best(self) -> None:
        b = self.best()
        if b is not None:
            run = self.space.trial(b["values"])
            (self.folder / "best.bux").write_text(
                f"# objective {b['objective']:.6g} (trial {b['trial']})\n" + run_to_source(run))

    def run(self, train: Callable, echo=print) -> Optional[dict]:
        """Sequential driver: `train(run) -> metrics dict`."""
        while True:
            job = self.next_job()
            if job is None:
                break
            value = self.report(job, train(job["run"]))
            echo(f"trial {job['trial']} rung {job['rung']}: "
                 f"{'no objective' if value is None else f'{value:.5g}'}  {job['values']}")
        return self.best()
