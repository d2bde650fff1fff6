"""Experiment trackers behind ``log(trackers=[wandb(...), tensorboard()])``: sinks that
forward every logged step. Both are optional imports: a missing package is an error at
start, naming the package. W&B resumes a run from ``<run>/wandb_id``; TensorBoard writes
under ``<run>/tensorboard``. Reference: ``train/trackers.py:52-237``."""

from __future__ import annotations

from pathlib import Path
from typing import Mapping

from .sinks import Sink


class TensorBoard(Sink):
    def __init__(self, folder, config=None):
        try:
            from torch.utils.tensorboard import SummaryWriter
        except ImportError as err:
            raise ImportError("log(trackers=[tensorboard()]) needs the `tensorboard` package") from err
        self.writer = SummaryWriter(str(Path(folder) / "tensorboard"))

    def write(self, step: int, scalars: Mapping) -> None:
        for k, v in scalars.items():
            try:
                self.writer.add_scalar(k, float(v), step)
            except (TypeError, ValueError):
                pass

    def close(self) -> None:
        self.writer.close()


class Wandb(Sink):
    def __init__(self, folder, config, run):
        try:
            import wandb
        except ImportError as err:
            raise ImportError("log(trackers=[wandb()]) needs the `wandb` package") from err
        folder = Path(folder)
        id_file = folder / "wandb_id"
        run_id = id_file.read_text().strip() if id_file.exists() else wandb.util.generate_id()
        id_file.write_text(run_id)
        self.run = wandb.init(project=config.project, entity=config.entity, group=config.group,
                              tags=list(config.tags), mode=config.mode, id=run_id, resume="allow",
                              name=run.name, dir=str(folder), config=run.model_dump(mode="json"))

    def write(self, step: int, scalars: Mapping) -> None:
        self.run.log({k: v for k, v in scalars.items()}, step=step)

    def close(self) -> None:
        self.run.finish()


def build(trackers, folder, run) -> list:
    out = []
    for t in trackers or ():
        out.append(TensorBoard(folder, t) if t.type == "tensorboard" else Wandb(folder, t, run))
    return out
