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


def agree_on_folder(folder, rank: int, world: int, barrier) -> None:
    """Fail early unless every rank sees the same (shared) folder: rank 0 drops a file,
    the others must see it (reference: ``runtime.py:116``, ``train/hooks.py:508``)."""
    from pathlib import Path

    marker = Path(folder) / ".bux_shared_check"
    if rank == 0:
        Path(folder).mkdir(parents=True, exist_ok=True)
        marker.write_text(str(world))
    barrier()
    seen = marker.exists()
    barrier()
    if rank == 0:
        marker.unlink(missing_ok=True)
    if not seen:
        raise ValueError(f"rank {rank} does not see {folder}: checkpoints and logs need a folder "
                         "every process shares")


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
