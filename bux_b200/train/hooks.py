"""Hooks the training loop calls after steps: logging, evals, checkpoints, profiling.

A hook says when it is `due`; the loop calls it with the metrics of the step *before*
the one it just launched, so reading them never stalls the device pipeline.

Reference: ``train/hooks.py:61-549`` (`Hook`, `Log`, `Eval`, `Checkpoint`, `Profile`).
"""

from __future__ import annotations

import json
import os
import shutil
import time
from pathlib import Path
from typing import Optional

import torch

from .. import runtime
from ..config import training as T
from . import flops as F


class Hook:
    every: int = 1

    def start(self, trainer) -> None:
        pass

    def due(self, step: int, trainer, last: bool = False) -> bool:
        return step % self.every == 0 or last

    def __call__(self, step: int, scalars: dict, trainer, sinks) -> None:
        raise NotImplementedError

    def stop(self, trainer, sinks) -> None:
        pass


def _host(scalars: dict) -> dict:
    out = {}
    for k, v in scalars.items():
        out[k] = float(v.item()) if isinstance(v, torch.Tensor) else float(v)
    return out


class Log(Hook):
    """tokens/s, MFU, host timers, peak memory, every ``log.every`` steps and at the end."""

    def __init__(self, c: T.LogConfig, run, trainer):
        self.every = c.every
        self.run = run
        self.last_time: Optional[float] = None
        self.last_tokens = 0
        self.last_step = 0
        self.flops_per_token = None
        try:
            self.flops_per_token = F.flops_per_token(run.arch, run.train.seq_len)
        except Exception:  # noqa: BLE001  (an exotic layer the counter does not know)
            self.flops_per_token = None
        self.peak = F.device_peak(trainer.device)

    def start(self, trainer) -> None:
        self.last_time = time.perf_counter()
        self.last_tokens = trainer.tokens
        self.last_step = trainer.step

    def __call__(self, step, scalars, trainer, sinks) -> None:
        host = _host(scalars)  # waits for that step only; the next one is already launched
        trainer.check_kernels(f"step {step}")
        now = time.perf_counter()
        tokens = int(host.get("tokens", trainer.tokens))
        dt = max(now - (self.last_time or now), 1e-9)
        steps = max(step - self.last_step, 1)
        rate, step_ms = (tokens - self.last_tokens) / dt, dt / steps * 1000
        previous = getattr(self, "previous", None)
        if previous is not None and step_ms < 0.05 * previous[1]:
            # the last step's scalars are read right after the step before it was logged (the
            # log runs one step behind): no time has passed, so the earlier rate stands
            rate, step_ms = previous
        self.previous = (rate, step_ms)
        host["tokens_per_s"] = rate
        host["time/step_ms"] = step_ms
        host.update(trainer.timers.flush())
        world = trainer.parallel.world if trainer.parallel is not None else 1
        if self.flops_per_token and self.peak:
            host["mfu"] = host["tokens_per_s"] * self.flops_per_token / (self.peak * world)
        if trainer.device.type == "cuda":
            host["mem/peak_gib"] = torch.cuda.max_memory_allocated(trainer.device) / 2 ** 30
        self.last_time, self.last_tokens, self.last_step = now, tokens, step
        for s in sinks:
            s.write(step, host)


class Eval(Hook):
    def __init__(self, c: T.EvalConfig):
        self.c = c
        self.every = c.every

    def __call__(self, step, scalars, trainer, sinks) -> None:
        metrics = trainer.evaluate(self.c)
        for s in sinks:
            s.write(step, metrics)


class Checkpoint(Hook):
    """Saves ``<run>/checkpoints/<step>/default/`` every N steps and at the end (the files are
    written in the background while training goes on, see `bux_b200.ckpt.store.save`), keeps
    the most recent `keep`, drops half-written ones on restore. The directory layout and
    state-tree paths are the reference's; array payloads are written by `bux_b200.ckpt`."""

    def __init__(self, folder, c: T.CheckpointConfig):
        self.folder = Path(folder) / "checkpoints"
        self.c = c
        self.every = c.every
        self.saved_at = -1

    def steps(self) -> list:
        if not self.folder.exists():
            return []
        return sorted(int(p.name) for p in self.folder.iterdir() if p.name.isdigit())

    def drop_unfinished(self) -> None:
        if not self.folder.exists():
            return
        for p in self.folder.iterdir():
            if p.name.endswith(".orbax-checkpoint-tmp") or p.name.endswith(".tmp"):
                shutil.rmtree(p, ignore_errors=True)

    def restore(self, trainer) -> Optional[int]:
        from .. import ckpt

        ckpt.wait()   # a save of this process that still writes in the background
        if runtime.rank() == 0:
            self.drop_unfinished()
        if trainer.parallel is not None:
            trainer.parallel.barrier()
        steps = self.steps()
        if not steps:
            return None
        step = steps[-1]
        ckpt.load(self.folder / str(step), trainer)
        self.saved_at = step
        return step

    def save(self, trainer) -> None:
        from .. import ckpt

        step = trainer.step
        if step == self.saved_at:
            return
        if trainer.device.type == "cuda":
            torch.cuda.synchronize(trainer.device)  # the state read below is the finished step's
        trainer.check_kernels(f"checkpoint at step {step}")
        ckpt.save(self.folder, step, trainer)
        self.saved_at = step
        if runtime.rank() == 0:
            for old in self.steps()[:-self.c.keep]:
                shutil.rmtree(self.folder / str(old), ignore_errors=True)

    def due(self, step, trainer, last=False) -> bool:
        return step % self.every == 0 or last or trainer.stopping

    def __call__(self, step, scalars, trainer, sinks) -> None:
        # the loop is one step ahead: save the state it has now, under its own step
        self.save(trainer)

    def stop(self, trainer, sinks) -> None:
        from .. import ckpt

        self.save(trainer)
        ckpt.wait()   # the run ends with its last checkpoint readable
        if runtime.rank() == 0:
            for old in self.steps()[:-self.c.keep]:
                shutil.rmtree(self.folder / str(old), ignore_errors=True)


class Profile(Hook):
    """Traces steps [start, start + steps) with the torch (CUPTI) profiler, or brackets
    them with cudaProfilerStart/Stop when the process runs under nsys / ncu."""

    def __init__(self, c: T.ProfileConfig, folder):
        self.c = c
        self.folder = Path(folder) / "profile"
        self.prof = None
        self.every = 1
        self.external = os.environ.get("BUX_PROFILER") in ("nsys", "ncu")

    def due(self, step, trainer, last=False) -> bool:
        return step in (self.c.start, self.c.start + self.c.steps) or (last and self.prof is not None)

    def __call__(self, step, scalars, trainer, sinks) -> None:
        cuda = trainer.device.type == "cuda"
        if step == self.c.start and self.prof is None:
            if cuda:
                torch.cuda.synchronize(trainer.device)
            if self.external and cuda:
                torch.cuda.cudart().cudaProfilerStart()
                self.prof = "external"
                return
            acts = [torch.profiler.ProfilerActivity.CPU]
            if cuda:
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(activities=acts)
            self.prof.__enter__()
        elif self.prof is not None:
            if cuda:
                torch.cuda.synchronize(trainer.device)
            if self.prof == "external":
                torch.cuda.cudart().cudaProfilerStop()
                self.prof = None
                return
            self.prof.__exit__(None, None, None)
            self.folder.mkdir(parents=True, exist_ok=True)
            rank = runtime.rank()
            path = self.folder / f"trace_rank{rank}.json"
            self.prof.export_chrome_trace(str(path))
            from . import trace

            try:
                metrics = trace.comm_ms(path, steps=self.c.steps)
                for s in sinks:
                    s.write(step, metrics)
            except Exception:  # noqa: BLE001
                pass
            self.prof = None


class Stop(Hook):
    """Cooperative stop: a signal sets a flag; every step all ranks take the max of
    their flags so that all stop after the same step and the checkpoint hook saves it.
    (reference: ``launch.py:172-260``)."""

    def __init__(self):
        self.signal = 0
        self.every = 1

    def request(self, signum: int) -> None:
        self.signal = signum

    def due(self, step, trainer, last=False) -> bool:
        return True

    def __call__(self, step, scalars, trainer, sinks) -> None:
        flag = self.signal
        if trainer.parallel is not None and trainer.parallel.world > 1:
            flag = trainer.parallel.max_int(flag)
        if flag:
            self.signal = flag
            trainer.stopping = True
