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


def state_leaves(trainer):
    """(part, key, tensor) of every leaf of the checkpoint's tree, one at a time: "0" the model
    (fp32, from the master copy where there is one), "1" the optimizer (step, moments by
    parameter path, in the parameter's shape). Each tensor is formed when it is asked for, so
    a writer that lets go of one before it takes the next holds one leaf's copy at a time."""
    opt = trainer.optimizer
    for name, p in trainer.model.named_parameters():
        st = opt.state.get(name, {})
        yield "0", name, st.get("master", p.detach()).float()
    for name, b in trainer.model.named_buffers():
        if name.split(".")[-1] in ("inv_freq",):
            continue
        yield "0", name, b.detach()
    yield "1", "count", torch.tensor(opt.step_count)
    yield "1", "tokens", torch.tensor(trainer.tokens)
    shapes = {name: tuple(p.shape) for name, p in trainer.model.named_parameters()}
    for name in opt.state:
        for k, v in opt.moments_for_checkpoint(name, shapes[name]).items():
            yield "1", f"{k}/{name}", v


def state_tree(trainer) -> dict:
    """The whole tree at once (small models, tests): ``{"0": model, "1": optimizer}``."""
    tree: dict = {"0": {}, "1": {}}
    for part, key, value in state_leaves(trainer):
        tree[part][key] = value
    return tree


def save(folder, step: int, trainer) -> None:
    folder = Path(folder)
    rank = runtime.rank()
    final = folder / str(step)
    tmp = folder / f"{step}.orbax-checkpoint-tmp"
    par = trainer.parallel
    meta = {"step": step, "methods.stages": trainer.train.methods.stages,
            "repeat": trainer.train.methods.repeat, "rounds": trainer.train.methods.rounds}
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        (tmp / "default").mkdir(parents=True, exist_ok=True)
    if par is not None:
        par.barrier()
    if par is not None and getattr(par, "pipeline", None) is None:
        # leaf by leaf: every rank takes part in putting a leaf together, the first rank
        # writes it and lets go of it before the next one (a 30B model with its moments never
        # sits whole on one device)
        index = {}
        for part, key, value in state_leaves(trainer):
            whole = par.whole_leaf(key, value)
            if rank == 0:
                path = f"{part}/{key}"
                index[path] = write_array(tmp / "default" / path.replace(".", "/"), whole)
            del whole, value
        if rank == 0:
            (tmp / "default" / "_METADATA.json").write_text(json.dumps({"tree": index, "custom_metadata": meta}))
        tree = None
    else:
        tree = state_tree(trainer) if par is None else par.checkpoint_tree(trainer, state_tree)
    if tree is not None:
        write_tree(tmp / "default", tree, meta)
    if trainer.parallel is not None:
        trainer.parallel.barrier()
    if rank == 0:
        shutil.rmtree(final, ignore_errors=True)
        os.replace(tmp, final)
    if trainer.parallel is not None:
        trainer.parallel.barrier()


def load(folder, trainer) -> None:
    """Restore `trainer` from a checkpoint of whole leaves, leaf by leaf: every rank reads a
    leaf, keeps its own part of it (`Parallel.restore_leaf` inverts what the save gathered)
    and lets go of the rest before it reads the next, so a run resumes on the mesh it was
    saved on or on another one without any rank ever holding the whole state."""
    folder = Path(folder) / "default"
    meta = json.loads((folder / "_METADATA.json").read_text())
    custom = meta.get("custom_metadata", {})
    mine = trainer.parallel.restore_leaf(trainer) if trainer.parallel is not None else (lambda name, t: t)
    opt = trainer.optimizer
    params = dict(trainer.model.named_parameters())
    buffers = dict(trainer.model.named_buffers())
    with torch.no_grad():
        for path in meta["tree"]:
            part, key = path.split("/", 1)
            value = read_array(folder / path.replace(".", "/"))
            if part == "0":
                name = key.replace("/", ".")
                value = mine(name, value)
                if value is None:
                    continue
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
            elif key == "count":
                opt.step_count = int(value)
            elif key == "tokens":
                trainer.tokens = int(value)
            else:
                kind, name = key.split("/", 1)
                name = name.replace("/", ".")
                value = mine(name, value)
                if value is None:
                    continue
                if name not in opt.state:
                    raise KeyError(f"the checkpoint holds optimizer state of '{name}', which this model has not")
                opt.load_moment(name, kind, value)
    trainer.step = int(custom.get("step", opt.step_count))
