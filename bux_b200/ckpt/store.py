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


def _to_numpy(t: torch.Tensor, copy: bool = False):
    """`t` on the host as (numpy array, dtype name); with `copy` never the live tensor's own
    memory (a background writer reads it while training updates the tensor)."""
    host = t.detach().cpu().contiguous()
    if copy and host.data_ptr() == t.data_ptr():
        host = host.clone()
    t = host
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy(), "bfloat16"
    return t.numpy(), str(t.dtype).replace("torch.", "")


def _chunk_path(folder: Path, index: int, dims: int) -> Path:
    return folder / "c" / "/".join([str(index), *("0" for _ in range(dims - 1))]) if dims else folder / "c"


def array_meta(shape: list, dtype: str, parts: int = 1) -> dict:
    """zarr v3 metadata of an array cut into `parts` equal chunks along its first axis."""
    chunk = ([shape[0] // parts, *shape[1:]] if shape else [1])
    return {"zarr_format": 3, "node_type": "array", "shape": shape, "data_type": _ZARR_DTYPES[dtype],
            "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": chunk}},
            "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
            "fill_value": 0, "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}]}


def write_chunk(folder: Path, payload: bytes, index: int, dims: int) -> None:
    chunk = _chunk_path(folder, index, dims)
    chunk.parent.mkdir(parents=True, exist_ok=True)
    chunk.write_bytes(payload)


def write_array(folder: Path, t: torch.Tensor) -> dict:
    """A whole array as one chunk."""
    arr, dtype = _to_numpy(t)
    folder.mkdir(parents=True, exist_ok=True)
    shape = list(t.shape)
    (folder / "zarr.json").write_text(json.dumps(array_meta(shape, dtype)))
    write_chunk(folder, arr.tobytes(), 0, len(shape))
    return {"dtype": dtype, "shape": shape}


def read_array(folder: Path, rows: tuple | None = None) -> torch.Tensor:
    """The array, put together from its chunks; with `rows` = (lo, hi) only those rows of it,
    reading only the chunks that hold them."""
    meta = json.loads((folder / "zarr.json").read_text())
    shape, dtype = meta["shape"], meta["data_type"]
    np_dtype = np.uint16 if dtype == "bfloat16" else np.dtype(dtype)

    def typed(a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(a)
        return t.view(torch.bfloat16) if dtype == "bfloat16" else t

    if not shape:
        return typed(np.frombuffer((folder / "c").read_bytes(), dtype=np_dtype).copy()).reshape(())
    per = meta["chunk_grid"]["configuration"]["chunk_shape"][0] or 1
    lo, hi = rows if rows is not None else (0, shape[0])
    out = np.empty([hi - lo, *shape[1:]], dtype=np_dtype)
    for c in range(lo // per, (max(hi, lo + 1) - 1) // per + 1 if hi > lo else 0):
        held = np.frombuffer(_chunk_path(folder, c, len(shape)).read_bytes(), dtype=np_dtype)
        held = held.reshape([-1, *shape[1:]])
        a, b = max(lo, c * per), min(hi, c * per + held.shape[0])
        out[a - lo:b - lo] = held[a - c * per:b - c * per]
    return typed(out)


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


class _Writer:
    """Writes a checkpoint's files: at once, or (``background``) on a thread while training
    goes on. The arrays it is given are host copies already, so the device state may change."""

    def __init__(self, background: bool):
        self.background = background
        self.jobs: list = []

    def put(self, fn, *args) -> None:
        if self.background:
            self.jobs.append((fn, args))
        else:
            fn(*args)


_pending: list = []     # the thread of a save that is still writing, and what it raised


def wait() -> None:
    """Block until a save that writes in the background has finished (and raise what it raised)."""
    while _pending:
        thread, failed = _pending.pop()
        thread.join()
        if failed:
            raise failed[0]


def _room_for(nbytes: int) -> bool:
    try:
        import psutil

        return nbytes * 2 < psutil.virtual_memory().available
    except Exception:  # noqa: BLE001
        return False


def state_bytes(trainer) -> int:
    """Bytes of this rank's part of a checkpoint (fp32 weights and moments of what it holds)."""
    n = sum(p.numel() for p in trainer.model.parameters())
    return n * 4 * (1 + len(getattr(trainer.optimizer, "MOMENTS", ("m", "v"))))


def save(folder, step: int, trainer, background: bool | None = None) -> None:
    """Write ``<folder>/<step>/default``. Every rank writes the rows it holds of the leaves
    that are sharded by rows (FSDP shards, an expert-parallel rank's experts) as chunks of one
    array; leaves split another way are put together leaf by leaf and written by the first
    rank. With `background` (the default when the host has room for a copy of this rank's
    state; ``BUX_CHECKPOINT_SYNC=1`` turns it off) the files are written by a thread while
    training goes on, and the folder gets its final name when every rank has finished."""
    wait()
    folder = Path(folder)
    rank, world = runtime.rank(), runtime.world_size()
    final = folder / str(step)
    tmp = folder / f"{step}.orbax-checkpoint-tmp"
    par = trainer.parallel
    meta = {"step": step, "methods.stages": trainer.train.methods.stages,
            "repeat": trainer.train.methods.repeat, "rounds": trainer.train.methods.rounds}
    if background is None:
        background = os.environ.get("BUX_CHECKPOINT_SYNC", "") in ("", "0") and _room_for(state_bytes(trainer))
    if par is not None and world > 1 and runtime.store() is None:
        background = False
    if rank == 0:
        shutil.rmtree(tmp, ignore_errors=True)
        (tmp / "default").mkdir(parents=True, exist_ok=True)
    if par is not None:
        par.barrier()
    out = _Writer(background)
    root = tmp / "default"
    if par is not None and getattr(par, "pipeline", None) is None:
        index = {}
        for part, key, value in state_leaves(trainer):
            path = f"{part}/{key}"
            where = root / path.replace(".", "/")
            place = par.leaf_placement(key, value)
            if place is None:
                # split some other way: every rank takes part in putting the leaf together, the
                # first rank writes it and lets go of it before the next one
                whole = par.whole_leaf(key, value)
                if rank == 0:
                    arr, dtype = _to_numpy(whole, copy=background)
                    shape = list(whole.shape)
                    index[path] = {"dtype": dtype, "shape": shape}
                    out.put(_write_whole, where, arr, shape, dtype)
                del whole
            else:
                parts, mine, writer = place
                shape = [value.shape[0] * parts, *value.shape[1:]] if value.dim() else []
                dtype = "bfloat16" if value.dtype == torch.bfloat16 else str(value.dtype).replace("torch.", "")
                if rank == 0:
                    index[path] = {"dtype": dtype, "shape": shape}
                    out.put(_write_meta, where, shape, dtype, parts)
                if writer:
                    arr, _ = _to_numpy(value, copy=background)
                    out.put(_write_rows, where, arr, mine, len(shape))
            del value
        if rank == 0:
            out.put(_write_text, root / "_METADATA.json", json.dumps({"tree": index, "custom_metadata": meta}))
    else:
        tree = state_tree(trainer) if par is None else par.checkpoint_tree(trainer, state_tree)
        if tree is not None:
            if background:   # host copies now: the thread must not read tensors that training updates
                tree = {k: {n: (v.detach().cpu().clone() if isinstance(v, torch.Tensor) else v) for n, v in part.items()}
                        for k, part in tree.items()}
            out.put(write_tree, root, tree, meta)

    def finish() -> None:
        for fn, args in out.jobs:
            fn(*args)
        _arrived(step, rank, world, par, background)
        if rank == 0:
            shutil.rmtree(final, ignore_errors=True)
            os.replace(tmp, final)
        _named(step, rank, world, par, background)

    if not background:
        finish()
        if par is not None:
            par.barrier()
        return
    import threading

    failed: list = []

    def run() -> None:
        try:
            finish()
        except BaseException as err:  # noqa: BLE001 - handed to the thread that waits
            failed.append(err)

    thread = threading.Thread(target=run, name=f"bux-checkpoint-{step}", daemon=False)
    _pending.append((thread, failed))
    thread.start()


def _arrived(step: int, rank: int, world: int, par, background: bool) -> None:
    """Every rank has written its files: a barrier on the calling thread, or (from a writer
    thread, which must not run collectives) a count in the job's key-value store."""
    if par is None or world == 1:
        return
    if not background:
        par.barrier()
        return
    kv = runtime.store()
    kv.set(f"bux/ckpt/{step}/{rank}", "1")
    if rank == 0:
        _poll(kv, [f"bux/ckpt/{step}/{r}" for r in range(world)])


def _named(step: int, rank: int, world: int, par, background: bool) -> None:
    """The first rank has given the folder its final name: a writer thread of another rank
    ends only then, so that `wait` means the same on every rank (the checkpoint can be read)."""
    if par is None or world == 1 or not background:
        return
    kv = runtime.store()
    if rank == 0:
        kv.set(f"bux/ckpt/{step}/named", "1")
    else:
        _poll(kv, [f"bux/ckpt/{step}/named"])


def _poll(kv, keys: list, limit_s: float = 7200.0) -> None:
    """Wait for `keys` without a blocking call: the store's client serves one request at a
    time, and the training thread uses the same client (a new process group waits in it), so
    a writer thread that blocked there could hold up the very ranks it waits for."""
    import time

    deadline = time.monotonic() + limit_s
    while not kv.check(keys):
        if time.monotonic() > deadline:
            raise TimeoutError(f"a checkpoint's writers did not all finish within {limit_s:.0f} s: {keys}")
        time.sleep(0.02)


def _write_whole(where: Path, arr, shape: list, dtype: str) -> None:
    where.mkdir(parents=True, exist_ok=True)
    (where / "zarr.json").write_text(json.dumps(array_meta(shape, dtype)))
    write_chunk(where, arr.tobytes(), 0, len(shape))


def _write_meta(where: Path, shape: list, dtype: str, parts: int) -> None:
    where.mkdir(parents=True, exist_ok=True)
    (where / "zarr.json").write_text(json.dumps(array_meta(shape, dtype, parts)))


def _write_rows(where: Path, arr, index: int, dims: int) -> None:
    write_chunk(where, arr.tobytes(), index, dims)


def _write_text(path: Path, text: str) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(text)


def load(folder, trainer) -> None:
    """Restore `trainer` from a checkpoint of whole leaves, leaf by leaf: every rank reads a
    leaf, keeps its own part of it (`Parallel.restore_leaf` inverts what the save gathered)
    and lets go of the rest before it reads the next, so a run resumes on the mesh it was
    saved on or on another one without any rank ever holding the whole state."""
    wait()
    folder = Path(folder) / "default"
    meta = json.loads((folder / "_METADATA.json").read_text())
    custom = meta.get("custom_metadata", {})
    par = trainer.parallel
    whole = par.restore_leaf(trainer) if par is not None else (lambda name, t: t)
    rows_of = par.restore_rows(trainer) if par is not None else (lambda name, shape: None)

    def read(path: str, name: str):
        """This rank's part of the leaf: only its rows are read where rows are all it is cut by."""
        shape = meta["tree"][path].get("shape") if isinstance(meta["tree"][path], dict) else None
        rows = rows_of(name, shape) if shape else None
        if rows is not None:
            return read_array(folder / path.replace(".", "/"), rows).contiguous()
        return whole(name, read_array(folder / path.replace(".", "/")))

    opt = trainer.optimizer
    params = dict(trainer.model.named_parameters())
    buffers = dict(trainer.model.named_buffers())
    with torch.no_grad():
        for path in meta["tree"]:
            part, key = path.split("/", 1)
            if part == "0":
                name = key.replace("/", ".")
                value = read(path, name)
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
                opt.step_count = int(read_array(folder / path.replace(".", "/")))
            elif key == "tokens":
                trainer.tokens = int(read_array(folder / path.replace(".", "/")))
            else:
                kind, name = key.split("/", 1)
                name = name.replace("/", ".")
                value = read(path, name)
                if value is None:
                    continue
                if name not in opt.state:
                    raise KeyError(f"the checkpoint holds optimizer state of '{name}', which this model has not")
                opt.load_moment(name, kind, value)
    trainer.step = int(custom.get("step", opt.step_count))
