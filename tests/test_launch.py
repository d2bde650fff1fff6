"""The launcher: status.json, done runs are skipped, sweeps as worker processes, signals."""
import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

from bux_b200 import launch as L

ROOT = Path(__file__).resolve().parent.parent
SMOKE = ROOT / "examples" / "experiments" / "smoke.bux"


def _say(lines):
    return lambda *a: lines.append(" ".join(str(x) for x in a))


def test_single_run_writes_status_and_is_not_trained_twice(tmp_path):
    said = []
    code = L.launch(SMOKE, overrides=["steps = 6", "log = log(every=2)", "schedule = constant"], out=tmp_path, device="cpu", echo=_say(said))
    assert code == 0
    (folder,) = [p for p in tmp_path.iterdir() if p.is_dir()]
    st = json.loads((folder / "status.json").read_text())
    assert st["state"] == "done" and st["step"] == 6 and st["error"] is None
    assert st["host"] and st["pid"] == os.getpid() and st["started"] <= st["ended"]
    assert "loss" in st["metrics"] and "tokens_per_s" in st["metrics"]
    said.clear()
    assert L.launch(SMOKE, overrides=["steps = 6", "log = log(every=2)", "schedule = constant"], out=tmp_path, device="cpu", echo=_say(said)) == 0
    assert said == ["1 of 1 runs done already"]


def test_sweep_runs_as_workers_and_prints_the_table(tmp_path):
    said = []
    env_before = os.environ.get("CUDA_VISIBLE_DEVICES")
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        code = L.launch(SMOKE, overrides=["steps = 4", "schedule = constant", "optimizer.lr = 1e-3 | 3e-3"], out=tmp_path, echo=_say(said))
    finally:
        if env_before is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES")
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env_before
    assert code == 0, said
    assert said[0] == "training 2 runs, one at a time"
    table = said[-1].splitlines()
    assert table[0] == "2 runs: 2 done"
    assert table[1].split() == ["state", "step", "loss", "eval", "loss", "run"]
    assert table[2].startswith("done   4/4") and table[2].endswith("smoke[optimizer.lr=1e-3]")
    logs = list(tmp_path.glob("*/train.log"))
    assert len(logs) == 2 and all(p.stat().st_size > 0 for p in logs)
    runs = L.compile_runs(SMOKE.read_text(), filename=str(SMOKE), overrides=["steps = 4", "schedule = constant", "optimizer.lr = 1e-3 | 3e-3"])
    assert L.results(runs, tmp_path) == said[-1]


def test_sigterm_stops_after_the_step_with_a_checkpoint(tmp_path):
    cmd = [sys.executable, "-m", "bux_b200", "launch", str(SMOKE), "steps = 100000", "log = log(every=5)",
           "checkpoint = checkpoint(every=100000)", "--out", str(tmp_path), "--device", "cpu"]
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=tmp_path)
    try:
        deadline = time.time() + 120
        step = 0
        while time.time() < deadline and step == 0:
            for p in tmp_path.glob("*/status.json"):
                step = json.loads(p.read_text()).get("step", 0)
            time.sleep(0.2)
        assert step > 0, "the run never reported a step"
        proc.send_signal(signal.SIGTERM)
        code = proc.wait(timeout=120)
    finally:
        if proc.poll() is None:
            proc.kill()
    assert code == 128 + signal.SIGTERM
    (status,) = list(tmp_path.glob("*/status.json"))
    st = json.loads(status.read_text())
    assert st["state"] == "stopped" and 0 < st["step"] < 100000
    saved = [p.name for p in (status.parent / "checkpoints").iterdir()]
    assert str(st["step"]) in saved


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_train_joins_the_job_torchrun_describes(tmp_path):
    """`bux train` under torchrun is one sharded job, not a copy of the run per rank: two
    gloo ranks report a world of two and each holds half the parameters."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           "-m", "bux_b200", "train", str(SMOKE), "steps = 3", "schedule = constant", "mesh = mesh(fsdp=2)",
           "--device", "cpu", "--out", str(tmp_path)]
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    done = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=tmp_path,
                          timeout=240, text=True)
    assert done.returncode == 0, done.stdout[-2000:]
    assert "on 2 × cpu" in done.stdout
    assert "78k parameters" in done.stdout       # the 156k-parameter model, sharded over two ranks
    (status,) = list(tmp_path.glob("*/status.json"))
    assert json.loads(status.read_text())["state"] == "done"
