"""Process-wide defaults set before CUDA / NCCL start; a user's own values win.

Reference: ``runtime.py:48-161`` (XLA / NCCL defaults, memory pool fraction, compile
cache agreement). Here: NCCL knobs for NVLink-5 / NVSwitch, the caching allocator's
expandable segments (fewer fragmentation stalls at 180 GB), TF32 off for fp32 islands.
"""

from __future__ import annotations

import os

NCCL_DEFAULTS = {
    "NCCL_NVLS_ENABLE": "1",          # in-switch reductions where the fabric offers them
    "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1",
    "TORCH_NCCL_AVOID_RECORD_STREAMS": "1",
}
ALLOC_DEFAULT = "expandable_segments:True"


def configure() -> None:
    for k, v in NCCL_DEFAULTS.items():
        os.environ.setdefault(k, v)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", ALLOC_DEFAULT)
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")


def _first_int(names, default: int) -> int:
    for name in names:
        v = os.environ.get(name)
        if v not in (None, ""):
            return int(v)
    return default


def rank() -> int:
    """This process's rank in the job: from torch.distributed once the job is joined, else
    from the launcher's environment (torchrun, SLURM's srun, Open MPI's mpirun)."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:  # noqa: BLE001
        pass
    return _first_int(("RANK", "SLURM_PROCID", "OMPI_COMM_WORLD_RANK"), 0)


def local_rank() -> int:
    """This process's index among the processes of its node (the GPU it takes)."""
    return _first_int(("LOCAL_RANK", "SLURM_LOCALID", "OMPI_COMM_WORLD_LOCAL_RANK"), 0)


def world_size() -> int:
    return _first_int(("WORLD_SIZE", "SLURM_STEP_NUM_TASKS", "SLURM_NTASKS", "OMPI_COMM_WORLD_SIZE"), 1)


def store():
    """The job's key-value store (what the processes joined through), or None before they
    joined: small strings between ranks without a collective and without a device."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return None
    return dist.distributed_c10d._get_default_store()


_asked = 0


def shared(folder, timeout_s: float = 60.0) -> bool:
    """Whether `folder` is one directory for every process of the job: the first process
    makes a file there and the others must see it. Every process calls it (the same number of
    times); they talk through `store`, so no rank needs a GPU or a collective for it.
    A job of one process shares every folder with itself. Reference: ``runtime.py:139``."""
    import secrets
    from datetime import timedelta
    from pathlib import Path

    global _asked
    kv = store()
    me, n = rank(), world_size()
    if kv is None or n == 1:
        return True
    _asked += 1
    key = f"bux/shared/{_asked}"
    folder = Path(folder)
    if me == 0:
        marker = f".bux-{secrets.token_hex(8)}"
        folder.mkdir(parents=True, exist_ok=True)
        (folder / marker).touch()
        kv.set(f"{key}/marker", marker)
    kv.wait([f"{key}/marker"], timedelta(seconds=timeout_s))
    marker = kv.get(f"{key}/marker").decode()
    # a listing, not a lookup: a network file system may cache that a name was missing
    seen = folder.is_dir() and marker in os.listdir(folder)
    kv.set(f"{key}/seen/{me}", "1" if seen else "0")
    names = [f"{key}/seen/{i}" for i in range(n)]
    kv.wait(names, timedelta(seconds=timeout_s))
    every = [kv.get(k) == b"1" for k in names]
    kv.add(f"{key}/read", 1)
    if me == 0:
        while kv.add(f"{key}/read", 0) < n:   # the others have read the answers
            import time

            time.sleep(0.01)
        (folder / marker).unlink(missing_ok=True)
    return all(every)


def agree_on_folder(folder) -> None:
    """Fail early unless every process sees `folder`: checkpoints, logs and the run's status
    are written by the first process and read by all (reference: ``train/hooks.py:508``)."""
    if not shared(folder):
        raise ValueError(f"{folder} is not one directory for every process of the job: checkpoints and "
                         "logs need a folder every host mounts")


def build_in_turn() -> None:
    """Build (or find) the native library without every rank compiling it at once. Where the
    package's folder is one for the whole job, the first process builds and the others wait;
    where each host has its own copy, the first process of each host does. (The build itself
    also takes a file lock, which covers processes of one host that never joined a job.)
    The counterpart of the reference's agreement on one compile cache, ``runtime.py:116``."""
    from .ops import _build

    kv = store()
    if kv is None or world_size() == 1:
        _build.load()
        return
    import torch.distributed as dist

    one_copy = shared(_build.EXT_DIR.parent)
    builder = rank() == 0 if one_copy else local_rank() == 0
    if builder:
        _build.load()
    dist.barrier()
    if not builder:
        _build.load()


def node_name() -> str:
    """The machine this process runs on (``BUX_NODE_NAME`` overrides the host name: for tests,
    and for containers that share a host name across nodes)."""
    import socket

    return os.environ.get("BUX_NODE_NAME") or socket.gethostname()


_one_node: dict = {}


def on_one_node(group) -> bool:
    """Whether every rank of `group` runs on the same machine: the kernels that load and store
    over peer memory (NVLink) need that; across machines the NCCL paths take over."""
    import torch.distributed as dist

    key = id(group)
    if key not in _one_node:
        local = _first_int(("LOCAL_WORLD_SIZE", "SLURM_NTASKS_PER_NODE", "OMPI_COMM_WORLD_LOCAL_SIZE"), 0)
        if "BUX_NODE_NAME" not in os.environ and local and local >= dist.get_world_size():
            _one_node[key] = True    # the launcher says the whole job is on this machine: nothing to ask
            return True
        names = [None] * dist.get_world_size(group)
        dist.all_gather_object(names, node_name(), group=group)
        _one_node[key] = len(set(names)) == 1
    return _one_node[key]
