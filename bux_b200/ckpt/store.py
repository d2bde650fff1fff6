"""Reading and writing checkpoint trees."""

from __future__ import annotations

import json
import os
import shutil
from pathlib import Path

import numpy as np
import torch

from .. import runtime

_ZARR_DTYPES = {"float32": "float32", "float64": "float64", "int32": "int32", "int64": "int64",
                "uint8": "uint8", "bfloat16": "bfloat16", "bool": "bool", "float16": "float16"}


def _to_numpy(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy(), "bfloat16"
    return t.numpy(), str(t.dtype).replace("torch.", "")


def write_array(folder: Path, t: torch.Tensor) -> dict:
    arr, dtype = _to_numpy(t)
    folder.mkdir(parents=True, exist_ok=True)
    shape = list(t.shape)
    meta = {"zarr_format": 3, "node_type": "array", "shape": shape, "data_type": _ZARR_DTYPES[dtype],
            "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": shape or [1]}},
            "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
            "fill_value": 0, "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}]}
    (folder / "zarr.json").write_text(json.dumps(meta))
    chunk = folder / "c" / "/".join("0" for _ in shape) if shape else folder / "c"
    chunk.parent.mkdir(parents=True, exist_ok=True)
    chunk.write_bytes(arr.tobytes())
    return {"dtype": dtype, "shape": shape}


def read_array(folder: Path) -> torch.Tensor:
    meta = json.loads((folder / "zarr.json").read_text())
    shape, dtype = meta["shape"], meta["data_type"]
    chunk = folder / "c" / "/".join("0" for _ in shape) if shape else folder / "c"
    raw = chunk.read_bytes()
    if dtype == "bfloat16":
        return torch.from_numpy(np.frombuffer(raw, dtype=np.uint16).copy()).view(torch.bfloat16).reshape(shape)
    return torch.from_numpy(np.frombuffer(raw, dtype=np.dtype(dtype)).copy()).reshape(shape)


def flatten(tree, prefix: str = "") -> dict:
    out: dict = {}
    if isinstance(tree, dict):
        for k, v in tree.items():
            out.update(flatten(v, f"{prefix}/{k}" if prefix else str(k)))
    elif isinstance(tree, torch.Tensor):
        out[prefix] = tree
    else:
        out[prefix] = torch.tensor(tree)
    return out


def unflatten(flat: dict) -> dict:
    tree: dict = {}
    for path, v in flat.items():
        node = tree
        parts = path.split("/")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = v
    return tree


def write_tree(folder, tree: dict, metadata: dict | None = None) -> None:
    folder = Path(folder)
    index = {}
    for path, t in flatten(tree).items():
        index[path] = write_array(folder / path.replace(".", "/"), t)
    (folder / "_METADATA.json").write_text(json.dumps({"tree": index, "custom_metadata": metadata or {}}))


def read_tree(folder) -> tuple:
    folder = Path(folder)
    meta = json.loads((folder / "_METADATA.json").read_text())
    flat = {path: read_array(folder / path.replace(".", "/")) for path in meta["tree"]}
    return unflatten(flat), meta.get("custom_metadata", {})


def state_tree(trainer) -> dict:
    """The checkpoint's tree: "0" the model (fp32, from the master copy where there is
    one), "1" the optimizer (step, moments by parameter path)."""
    opt = trainer.optimizer
    model = {}
    for name, p in trainer.model.named_parameters():
        st = opt.state.get(name, {})
        model[name] = st.get("master", p.detach()).float()
    for name, b in trainer.model.named_buffers():
        if name.split(".")[-1] in ("inv_freq",):
            continue
        model[name] = b.detach()
    optim_tree: dict = {"count": torch.tensor(opt.step_count), "tokens": torch.tensor(trainer.tokens)}
    shapes = {name: tuple(p.shape) for name, p in trainer.model.named_parameters()}
    for name in opt.state:
        for k, v in opt.moments_for_checkpoint(name, shapes[name]).items():
            optim_tree[f"{k}/{name}"] = v
    return {"0": model, "1": optim_tree}


def save(folder, step: int, trainer) -> None:
    folder = Path(folder)
    rank = runtime.rank()
    final = folder / str(step)
    tmp = folder / f"{step}.orbax-checkpoint-tmp"
    tree = state_tree(trainer) if trainer.parallel is None else trainer.parallel.checkpoint_tree(trainer, state_tree)
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        (tmp / "default").mkdir(parents=True, exist_ok=True)
    if trainer.parallel is not None:
        trainer.parallel.barrier()
    if tree is not None:
        meta = {"step": step, "methods.stages": trainer.train.methods.stages,
                "repeat": trainer.train.methods.repeat, "rounds": trainer.train.methods.rounds}
        write_tree(tmp / "default", tree, meta)
    if trainer.parallel is not None:
        trainer.parallel.barrier()
    if rank == 0:
        shutil.rmtree(final, ignore_errors=True)
        os.replace(tmp, final)
    if trainer.parallel is not None:
        trainer.parallel.barrier()


def load(folder, trainer) -> None:
    """Restore `trainer` from a checkpoint of whole leaves: every rank reads the tree and
    keeps its own part of each leaf (`Parallel.restore_tree` inverts what
    `Parallel.checkpoint_tree` gathered), so a run resumes on the mesh it was saved on
    or on another one."""
    tree, meta = read_tree(Path(folder) / "default")
    if trainer.parallel is not None:
        tree = trainer.parallel.restore_tree(trainer, tree)
    opt = trainer.optimizer
    model_state = tree["0"]
    flat_model = flatten(model_state)
    with torch.no_grad():
        params = dict(trainer.model.named_parameters())
        buffers = dict(trainer.model.named_buffers())
        for path, value in flat_model.items():
            name = path.replace("/", ".")
            if name in params:
                p = params[name]
                st = opt.state.get(name, {})
                if "master" in st:
                    st["master"].copy_(value.to(st["master"].device))
                p.data.copy_(value.to(p.device).to(p.dtype))
            elif name in buffers:
                buffers[name].copy_(value.to(buffers[name].device))
            else:
                raise KeyError(f"the checkpoint holds '{name}', which this model has not: the "
                               "architecture or a method that changes the state's layout differs")
        flat_opt = flatten(tree["1"])
        for path, value in flat_opt.items():
            if path == "count":
                opt.step_count = int(value)
            elif path == "tokens":
                trainer.tokens = int(value)
            else:
                kind, name = path.split("/", 1)
                name = name.replace("/", ".")
                if name not in opt.state:
                    raise KeyError(f"the checkpoint holds optimizer state of '{name}', which this model has not")
                opt.load_moment(name, kind, value)
    trainer.step = int(meta.get("step", opt.step_count))
