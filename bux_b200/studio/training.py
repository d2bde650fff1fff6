"""Training from the studio's page: the file's runs launched in a background process
(``bux launch``), their states and the tail of their metrics. Reference: ``studio/training.py``."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path
from typing import Optional


class Trainings:
    def __init__(self, file: Path, out: Path):
        self.file, self.out = Path(file), Path(out)
        self.job: Optional[subprocess.Popen] = None
        self.log = self.out / "studio-launch.log"

    def state(self) -> str:
        if self.job is None:
            return "idle"
        code = self.job.poll()
        return "training" if code is None else ("done" if code == 0 else f"failed (exit {code})")

    def start(self, only: Optional[str] = None) -> dict:
        """Launch the file's runs (those whose name contains `only`); a launch already going is left alone."""
        if self.state() == "training":
            return {"state": "training"}
        self.out.mkdir(parents=True, exist_ok=True)
        cmd = [sys.executable, "-m", "bux_b200", "launch", str(self.file), "--out", str(self.out)]
        if only:
            cmd += ["--only", only]
        self.job = subprocess.Popen(cmd, stdout=open(self.log, "w"), stderr=subprocess.STDOUT, start_new_session=True)
        return {"state": "training", "pid": self.job.pid}

    def stop(self) -> dict:
        """Ask the launch to stop after the step it is in (it checkpoints first), as a first Ctrl-C does."""
        import signal

        if self.job is not None and self.job.poll() is None:
            self.job.send_signal(signal.SIGINT)
        return {"state": self.state()}

    def runs(self, compiled: list, last: int = 200) -> list:
        """State and the latest metrics of every compiled run that has a folder under `out`."""
        from ..train.trainer import directory

        out = []
        for r in compiled:
            folder = directory(r, self.out)
            status, points = {}, []
            if (folder / "status.json").exists():
                try:
                    status = json.loads((folder / "status.json").read_text())
                except ValueError:
                    pass
            metrics = folder / "metrics.jsonl"
            if metrics.exists():
                for line in metrics.read_text().splitlines()[-last:]:
                    try:
                        row = json.loads(line)
                    except ValueError:
                        continue
                    if "loss" in row:
                        points.append([row.get("step"), row["loss"]])
            out.append({"name": r.name, "id": r.id, "state": status.get("state"), "step": status.get("step"),
                        "loss": points[-1][1] if points else None, "curve": points})
        return out

    def tail(self, lines: int = 30) -> str:
        return "\n".join(self.log.read_text(errors="replace").splitlines()[-lines:]) if self.log.exists() else ""
