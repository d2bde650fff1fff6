"""Reading a trained run: ``run.json`` → the run, its checkpoint → the model's weights.
Reference: ``export/runs.py:92-269`` (`read_run`, `restore`, `as_trained`)."""

from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

from ..lang import ir


def read_run(run_dir) -> ir.Run:
    path = Path(run_dir) / "run.json"
    if not path.exists():
        raise FileNotFoundError(f"{run_dir} is no run directory: it has no run.json")
    return ir.Run.model_validate_json(path.read_text())


def steps(run_dir) -> list:
    folder = Path(run_dir) / "checkpoints"
    if not folder.is_dir():
        return []
    return sorted(int(p.name) for p in folder.iterdir() if p.name.isdigit() and (p / "default").is_dir())


def restore(run_dir, step: Optional[int] = None) -> tuple:
    """(step, model tree "0": parameter path → tensor) of the run's checkpoint."""
    from ..ckpt import store

    have = steps(run_dir)
    if not have:
        raise FileNotFoundError(f"{run_dir} has no finished checkpoint")
    step = have[-1] if step is None else step
    if step not in have:
        raise FileNotFoundError(f"{run_dir} has no checkpoint of step {step}; it has {have}")
    tree, _ = store.read_tree(Path(run_dir) / "checkpoints" / str(step) / "default")
    return step, {k: torch.as_tensor(v) for k, v in tree["0"].items()}


def as_trained(run_dir, step: Optional[int] = None, dtype=torch.float32):
    """(run, step, model with the checkpoint's weights)."""
    from ..models import Model

    run = read_run(run_dir)
    step, tree = restore(run_dir, step)
    model = Model(run.arch, dtype=dtype, seed=run.train.seed)
    own = model.state_dict()
    missing = [k for k in own if k not in tree and not k.endswith("inv_freq")]
    if missing:
        raise KeyError(f"the checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
    model.load_state_dict({k: tree[k].to(own[k].dtype).reshape(own[k].shape) for k in own if k in tree}, strict=False)
    return run, step, model
