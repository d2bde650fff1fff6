"""`bux launch`: train every run of a file; sweeps go over the machine's GPUs.

What it keeps from the reference's launcher (``launch.py:100-843`` there):

* ``status.json`` per run directory (`running` / `done` / `failed` / `stopped`, host,
  pid, GPUs, times, step, latest metrics); a run that is `done` is not trained again,
  any other resumes from its latest checkpoint;
* one run trains in this process; a sweep starts one worker process per run
  (``python -m bux_b200.launch FOLDER CACHE``) with its own ``CUDA_VISIBLE_DEVICES``,
  first-fit over the free GPUs, each worker's output in ``train.log``;
* signals: the first SIGTERM / SIGINT stops after the current step (and checkpoints if
  the run has a checkpoint setting); a second one at least a second later stops at
  once; an earlier duplicate is ignored; exit codes 0 / 1 / 128+signal;
* a multi-process job (torchrun, SLURM or Open MPI variables) joins before training and
  agrees on stopping through a max-reduction each step;
* the summary table, and `results` to print it again without training.
"""

from __future__ import annotations

import datetime as _dt
import json
import os
import signal
import socket
import subprocess
import sys
import time
from pathlib import Path
from typing import Optional

from . import runtime
from .lang import compile_runs, ir


# ------------------------------------------------------------------ status.json
def _now() -> str:
    return _dt.datetime.now(_dt.timezone.utc).replace(microsecond=0).isoformat()


def status(folder) -> dict:
    path = Path(folder) / "status.json"
    try:
        return json.loads(path.read_text())
    except (OSError, ValueError):
        return {}


def record(folder, **fields) -> dict:
    """Merge `fields` into the directory's status.json (written whole, then renamed)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cur = status(folder)
    cur.update(fields)
    tmp = folder / "status.json.tmp"
    tmp.write_text(json.dumps(cur, indent=1, default=float))
    os.replace(tmp, folder / "status.json")
    return cur


def _scalar_metrics(metrics: dict) -> dict:
    out = {}
    for k, v in metrics.items():
        if "/" in k and not k.startswith(("time/", "mem/", "eval/")):
            continue  # per-layer statistics stay in metrics.jsonl
        try:
            out[k] = float(v)
        except (TypeError, ValueError):
            pass
    return out


# ------------------------------------------------------------------ processes of one job
def processes() -> int:
    env = os.environ
    return int(env.get("WORLD_SIZE") or env.get("SLURM_STEP_NUM_TASKS") or env.get("OMPI_COMM_WORLD_SIZE") or 1)


def visible_gpus() -> list:
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env is not None:
        return [g for g in env.split(",") if g.strip() != ""]
    try:
        import torch

        return [str(i) for i in range(torch.cuda.device_count())]
    except Exception:  # noqa: BLE001
        return []


def need(run: ir.Run) -> int:
    """GPUs one run takes: the size of its mesh (the free axis counts as one)."""
    from .parallel import mesh as M

    sizes = M.sizes(run.train.mesh, None)
    n = 1
    for v in sizes.values():
        n *= max(1, v)
    return n


# ------------------------------------------------------------------ signals
class Stop:
    """First signal: finish the step, checkpoint, leave. A second one a second or more
    later: leave now. One that comes sooner is the first delivered twice."""

    def __init__(self, children=None):
        self.signal: Optional[int] = None
        self.at = 0.0
        self.children = children if children is not None else []
        self.trainer = None
        self._old = {}

    def __enter__(self):
        for s in (signal.SIGTERM, signal.SIGINT):
            try:
                self._old[s] = signal.signal(s, self._on)
            except ValueError:  # not the main thread
                pass
        return self

    def __exit__(self, *exc):
        for s, h in self._old.items():
            signal.signal(s, h)

    def _on(self, signum, frame):
        now = time.monotonic()
        if self.signal is not None:
            if now - self.at < 1.0:
                return
            for c in self.children:
                c.kill()
            os._exit(128 + signum)
        self.signal, self.at = signum, now
        for c in self.children:
            try:
                c.send_signal(signum)
            except OSError:
                pass
        if self.trainer is not None:
            self.trainer.stopping = True
        elif not self.children:
            raise SystemExit(128 + signum)  # before training starts: stop at once


class _Report:
    """A hook: keeps status.json current and spreads a stop over the job's processes."""

    def __init__(self, folder, stop: Stop, every: int, parallel=None):
        self.folder, self.stopper, self.every, self.parallel = folder, stop, max(1, every), parallel
        self.last: dict = {}

    def start(self, trainer) -> None:
        self.stopper.trainer = trainer
        if self.stopper.signal is not None:
            trainer.stopping = True

    def due(self, step: int, trainer, last: bool = False) -> bool:
        return self.parallel is not None or step % self.every == 0 or last or trainer.stopping

    def __call__(self, step: int, scalars: dict, trainer, sinks) -> None:
        if self.parallel is not None:
            # every process leaves after the same step: a max over the job
            trainer.stopping = bool(self.parallel.max_int(1 if trainer.stopping else 0))
        if step % self.every == 0 or trainer.stopping or step >= trainer.train.steps:
            from .train.sinks import LatestMetrics

            for s in sinks or ():
                if isinstance(s, LatestMetrics):
                    self.last.update(_scalar_metrics(s.latest))
            if not self.last:
                self.last.update(_scalar_metrics({k: (v.item() if hasattr(v, "item") else v)
                                                  for k, v in scalars.items()}))
            self._write(trainer)

    def _write(self, trainer) -> None:
        if runtime.rank() == 0:
            record(self.folder, step=trainer.step, metrics=self.last)

    def stop(self, trainer, sinks) -> None:
        self._write(trainer)


# ------------------------------------------------------------------ one run, here
def train_here(run: ir.Run, out="runs", cache=".", device=None, quiet: bool = False,
               stop: Optional[Stop] = None) -> str:
    """Train one run in this process; returns its final state."""
    from .runtime import configure
    from .train import trainer as TR

    configure()
    folder = TR.directory(run, out)
    main = runtime.rank() == 0
    parallel = None
    if processes() > 1 or need(run) > 1:
        import torch

        from .parallel.engine import Parallel, init_distributed

        dev = torch.device(device) if device else None
        if dev is None and torch.cuda.is_available():
            dev = torch.device("cuda", runtime.local_rank())
        if init_distributed(dev):
            # before anything is written or compiled: the run's folder must be one for all
            # ranks, and the native library is built by one rank per copy of the package
            runtime.agree_on_folder(out)
            if dev is not None and dev.type == "cuda":
                runtime.build_in_turn()
            parallel = Parallel(run.train, dev)
            device = dev
    if main:
        record(folder, state="running", host=socket.gethostname(), pid=os.getpid(),
               gpus=os.environ.get("CUDA_VISIBLE_DEVICES"), started=_now(), ended=None, error=None)
    own = stop is None
    stop = stop or Stop()
    state = "failed"
    try:
        if own:
            stop.__enter__()
        hook = _Report(folder, stop, run.train.log.every, parallel)
        trainer = TR.train(run, out=out, cache=cache, device=device, parallel=parallel, quiet=quiet,
                           hooks=[hook])
        state = "done" if trainer.step >= run.train.steps else "stopped"
        if main:
            record(folder, state=state, ended=_now(), step=trainer.step)
    except BaseException as e:  # noqa: BLE001
        if main:
            record(folder, state="stopped" if isinstance(e, (KeyboardInterrupt, SystemExit)) else "failed",
                   ended=_now(), error=f"{type(e).__name__}: {e}")
        raise
    finally:
        if own:
            stop.__exit__(None, None, None)
    return state


# ------------------------------------------------------------------ sweeps: a queue over the GPUs
class Queue:
    """First fit: the next waiting run that fits the free GPUs starts."""

    def __init__(self, gpus: list):
        self.free = list(gpus)
        self.cpu_slot = not gpus

    def take(self, n: int) -> Optional[list]:
        if not self.free and self.cpu_slot:
            return []
        if n > len(self.free):
            return None
        got, self.free = self.free[:n], self.free[n:]
        return got

    def give(self, gpus: list) -> None:
        self.free.extend(gpus)


def _spawn(run: ir.Run, folder: Path, cache: str, gpus: list):
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "run.json").write_text(run.model_dump_json(indent=1))
    env = dict(os.environ)
    if gpus:
        env["CUDA_VISIBLE_DEVICES"] = ",".join(gpus)
    log = open(folder / "train.log", "ab")
    n = len(gpus)
    if n > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               "-m", "bux_b200.launch", str(folder), str(cache)]
    else:
        cmd = [sys.executable, "-m", "bux_b200.launch", str(folder), str(cache)]
    proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT)
    proc._bux_log = log
    return proc


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def supervise(runs: list, out, cache, echo=print) -> dict:
    """Train `runs` as worker processes; returns {run name: state}."""
    from .train import trainer as TR

    gpus = visible_gpus()
    queue = Queue(gpus)
    waiting = list(runs)
    running: dict = {}
    states: dict = {}
    with Stop(children=[]) as stop:
        while waiting or running:
            if stop.signal is None:
                for run in list(waiting):
                    if not gpus and running:
                        break  # on CPU: one at a time
                    got = queue.take(need(run))
                    if got is None:
                        continue
                    waiting.remove(run)
                    folder = TR.directory(run, out)
                    proc = _spawn(run, folder, cache, got)
                    stop.children.append(proc)
                    running[proc] = (run, got, folder)
                    echo(f"{run.name}: started on {'GPUs ' + ','.join(got) if got else 'cpu'}, output in {folder / 'train.log'}")
            else:
                for run in waiting:
                    states[run.name] = status(TR.directory(run, out)).get("state", "stopped")
                waiting = []
            for proc in list(running):
                code = proc.poll()
                if code is None:
                    continue
                run, got, folder = running.pop(proc)
                stop.children.remove(proc)
                proc._bux_log.close()
                queue.give(got)
                st = status(folder).get("state")
                if code != 0 and st not in ("stopped", "done"):
                    st = "failed"
                    record(folder, state="failed", ended=_now(), error=f"exit {code}")
                    echo(f"{run.name}: failed (exit {code}); its output is in {folder / 'train.log'}")
                else:
                    echo(f"{run.name}: {st}")
                states[run.name] = st
            time.sleep(0.2)
        states["__signal__"] = stop.signal
    return states


# ------------------------------------------------------------------ the table
def _fmt(v, digits=4) -> str:
    return "-" if v is None else f"{v:.{digits}f}"


def summary(runs: list, out) -> str:
    from .train import trainer as TR

    rows = []
    counts: dict = {}
    objective = any(r.train.objective is not None for r in runs)
    for r in runs:
        st = status(TR.directory(r, out))
        state = st.get("state", "waiting")
        counts[state] = counts.get(state, 0) + 1
        m = st.get("metrics", {})
        ev = next((m[k] for k in sorted(m) if k.startswith("eval/") and k.endswith("loss")), None)
        row = [state, f"{st.get('step', 0)}/{r.train.steps}", _fmt(m.get("loss")), _fmt(ev)]
        if objective:
            key = r.train.objective.metric if r.train.objective is not None else None
            row.append(_fmt(m.get(key)) if key else "-")
        row.append(r.name)
        rows.append(row)
    head = ["state", "step", "loss", "eval loss"] + (["objective"] if objective else []) + ["run"]
    widths = [max(len(str(x[i])) for x in [head, *rows]) for i in range(len(head))]
    order = ["done", "stopped", "failed", "running", "waiting"]
    tally = ", ".join(f"{counts[s]} {s}" for s in order if s in counts)
    lines = [f"{len(runs)} run{'s' if len(runs) != 1 else ''}: {tally}"]
    for row in [head, *rows]:
        lines.append("  ".join(str(c).ljust(w) for c, w in zip(row, widths)).rstrip())
    return "\n".join(lines)


def results(runs: list, out) -> str:
    return summary(runs, out)


# ------------------------------------------------------------------ entry points
def launch(file, overrides=(), out="runs", cache=".", only=None, index=None, entry=None,
           device=None, echo=print) -> int:
    from .train import trainer as TR

    src = Path(file).read_text()
    runs = compile_runs(src, filename=str(file), overrides=list(overrides or ()), entry=entry) \
        if entry else compile_runs(src, filename=str(file), overrides=list(overrides or ()))
    if only:
        runs = [r for r in runs if only in r.name]
    if index is not None:
        runs = [runs[index]]
    todo = [r for r in runs if status(TR.directory(r, out)).get("state") != "done"]
    if not todo:
        echo(f"{len(runs)} of {len(runs)} runs done already")
        return 0
    have = len(visible_gpus())
    for r in todo:
        if have and need(r) > have:
            echo(f"{r.name}: its mesh needs {need(r)} GPUs and this machine shows {have}")
            return 1
    for r in todo:
        st = status(TR.directory(r, out))
        if st.get("state") in ("stopped", "failed", "running") and r.train.checkpoint is None and st.get("step"):
            echo(f"{r.name}: has no checkpoint setting, so it starts over")
    if len(todo) == 1 and (processes() > 1 or need(todo[0]) <= 1):
        with Stop() as stop:
            try:
                state = train_here(todo[0], out, cache, device=device, stop=stop)
            except SystemExit as e:
                return int(e.code or 0)
            except Exception as e:  # noqa: BLE001
                echo(f"{todo[0].name}: failed ({type(e).__name__}: {e})")
                return 1
        if len(runs) > 1:
            echo(summary(runs, out))
        if stop.signal is not None and state != "done":
            return 128 + stop.signal
        return 0 if state == "done" else 1
    if processes() > 1:
        echo("a sweep takes one launcher process: it starts a worker per run itself")
        return 1
    echo(f"training {len(todo)} runs" + (", one at a time" if not visible_gpus() else ""))
    states = supervise(todo, out, cache, echo)
    sig = states.pop("__signal__", None)
    echo(summary(runs, out))
    if sig is not None:
        return 128 + sig
    return 0 if all(s == "done" for s in states.values()) else 1


def main(argv=None) -> int:
    """Worker of a sweep: ``python -m bux_b200.launch FOLDER CACHE`` trains the run that
    the launcher wrote to FOLDER/run.json."""
    argv = list(sys.argv[1:] if argv is None else argv)
    folder, cache = Path(argv[0]), (argv[1] if len(argv) > 1 else ".")
    run = ir.Run.model_validate_json((folder / "run.json").read_text())
    with Stop() as stop:
        try:
            state = train_here(run, out=folder.parent, cache=cache, stop=stop)
        except SystemExit as e:
            return int(e.code or 0)
    if stop.signal is not None and state != "done":
        return 128 + stop.signal
    return 0 if state == "done" else 1


if __name__ == "__main__":
    sys.exit(main())
