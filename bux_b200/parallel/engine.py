"""`Parallel`: what one rank knows about the mesh, and the explicit collectives of a step.

One process per GPU (``torch.distributed``, NCCL on GPUs, gloo on CPU). The mesh's six
axes become process groups; the trainer asks this object for its batch rows, hands it
the model to shard (`prepare_model`), and calls it around the backward
(`grad_sync`, `finish_grads`) and for scalars (`sum_scalar`, `max_int`).

What is explicit here was implicit in the reference (GSPMD inserted it from sharding
annotations, ``parallel/layout.py:95-220``, ``parallel/place.py:70-137``):
data-parallel gradient all-reduce, ZeRO-1 / FSDP sharding of parameters and optimizer
state (`fsdp.py`), tensor parallelism (`tensor.py`), expert parallelism
(`experts.py`), pipeline stages (`pipeline.py`).
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist

from . import mesh as M


class Parallel:
    def __init__(self, train, device=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.train = train
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.device = device if device is not None else torch.device("cpu")
        self.shape = M.sizes(train.mesh, self.world)
        if M.size(train.mesh, self.world) != self.world:
            raise ValueError(f"the mesh {self.shape} needs {M.size(train.mesh, self.world)} devices, "
                             f"and {self.world} joined")
        self.coords = M.coordinates(self.rank, self.shape)
        self._groups: dict = {}
        layout = train.layout
        batch_axes = tuple(a for a in M._axes_of(layout.batch) if self.shape[a] > 1)
        self.batch_axes = batch_axes
        # every rank creates every group, in the same order
        for axes in self._all_axis_sets():
            self._make_groups(axes)
        self.data_group = self.group(batch_axes) if batch_axes else None
        self.data_world = 1
        for a in batch_axes:
            self.data_world *= self.shape[a]
        self.data_rank = self._index_in(batch_axes)
        self.expert_group = self.group(("expert",)) if self.shape["expert"] > 1 else None
        self.tensor_group = self.group(("tensor",)) if self.shape["tensor"] > 1 else None
        self.stage_group = self.group(("stage",)) if self.shape["stage"] > 1 else None
        self.context_group = self.group(("context",)) if self.shape["context"] > 1 else None
        self.replicated: list = []   # (param, group) whose gradients are summed over group
        self._norm_w: dict = {}
        self.fsdp = None
        self.tensor_sharded: set = set()
        self.tensor_layout: dict = {}

    # ------------------------------------------------------------------ groups
    def _all_axis_sets(self) -> list:
        sets = [tuple(a for a in M._axes_of(self.train.layout.batch) if self.shape[a] > 1)]
        sets += [(a,) for a in M.AXES if self.shape[a] > 1]
        sets.append(self.shard_axes())
        sets.append(tuple(a for a in M.AXES if self.shape[a] > 1 and a not in ("expert",)))
        out = []
        for s in sets:
            if s and s not in out:
                out.append(s)
        return out

    def shard_axes(self) -> tuple:
        """The mesh axes whole parameters are sharded over: the layout's ``fsdp`` axes that
        are larger than one (``fsdp`` and ``expert`` by default, as the reference maps the
        sharded dimension over (fsdp, context, expert), ``train/config.py:959`` there).
        ``context`` is left out: its ranks hold different positions of the same rows and sum
        every gradient over the axis afterwards."""
        return tuple(a for a in M.AXES if a in M._axes_of(self.train.layout.fsdp)
                     and a in ("fsdp", "expert") and self.shape[a] > 1)

    def _make_groups(self, axes: tuple) -> None:
        seen = set()
        for r in range(self.world):
            ranks = tuple(M.group_ranks(r, self.shape, axes))
            if ranks in seen:
                continue
            seen.add(ranks)
            g = dist.new_group(list(ranks))
            if self.rank in ranks:
                self._groups[axes] = g

    def group(self, axes: tuple):
        axes = tuple(a for a in axes if self.shape[a] > 1)
        if not axes:
            return None
        if axes not in self._groups:
            raise KeyError(f"no process group over {axes}")
        return self._groups[axes]

    def _index_in(self, axes: tuple) -> int:
        idx = 0
        for a in M.AXES:
            if a in axes:
                idx = idx * self.shape[a] + self.coords[a]
        return idx

    # ------------------------------------------------------------------ the model
    def placement(self, arch=None, dtype=torch.bfloat16):
        """The context a model is built under, so that sharded stacks of experts are created
        as this rank's shard (`bux_b200.models.placement`). Pipeline stages still build the
        whole model first: a stage's share of the blocks is decided on the built graph."""
        from ..models import placement

        experts = rows = None
        if self.expert_group is not None and self.stage_group is None:
            experts = (dist.get_rank(self.expert_group), self.shape["expert"])
        if self.places_dense(arch, dtype):
            group = self.group(self.shard_axes())
            rows = (dist.get_rank(group), dist.get_world_size(group))
        return placement.placing(experts=experts, rows=rows)

    DENSE_PLACEMENT_BYTES = 16 << 30

    def places_dense(self, arch=None, dtype=torch.bfloat16) -> bool:
        """Whether dense parameters are cut to this rank's rows as they are created. Only where
        rows are all that cuts them (no tensor parallelism, no pipeline, NCCL gathers) and, by
        default, where a whole copy would be large (``BUX_PLACE_DENSE=always | never`` overrides)."""
        how = os.environ.get("BUX_PLACE_DENSE", "auto")
        options = getattr(getattr(self.train, "compiler", None), "options", "") or ""
        if (how == "never" or not self.shard_axes() or self.tensor_group is not None or self.stage_group is not None
                or "--fsdp=fused" in options.split()):
            return False
        if how == "always":
            return True
        if arch is None:
            return False
        from ..models import Model

        try:
            with torch.device("meta"):     # shapes only: what a whole copy of the dense parameters would take
                shapes = Model(arch, dtype=dtype)
        except Exception:  # noqa: BLE001 - a layer that cannot be built without memory: keep the old path
            return False
        dense = sum(p.numel() for n, p in shapes.named_parameters() if "experts_gate_up" not in n and "experts_down" not in n)
        return dense * torch.empty((), dtype=dtype).element_size() >= self.DENSE_PLACEMENT_BYTES

    def prepare_model(self, model) -> None:
        """Shard what the mesh shards: experts over ``expert``, then (tensor / fsdp) the
        rest; what stays whole is marked for gradient all-reduce over the batch axes."""
        from ..models import placement
        from ..models.layers.moe import MoE
        from .experts import ExpertParallel

        t = self.train
        expert_params = set()
        self.pipeline = None
        if self.stage_group is not None:
            from .pipeline import Pipeline

            self.pipeline = Pipeline(model, self)  # first: the rest shards what this stage keeps
        if self.expert_group is not None:
            me, n = dist.get_rank(self.expert_group), self.shape["expert"]
            ep = ExpertParallel(self.expert_group, t.methods.moe, t.methods.capacity)
            for m in model.modules():
                if isinstance(m, MoE):
                    el = m.c.num_experts // n
                    for name in ("experts_gate_up", "experts_down"):
                        p = getattr(m, name)
                        if getattr(p, "placed_rows", None) is None:   # built whole: keep this rank's experts
                            p = placement.keep_rows(p, slice(me * el, (me + 1) * el))
                            setattr(m, name, p)
                        elif p.placed_rows != slice(me * el, (me + 1) * el):
                            raise ValueError(f"{name} was built for experts {p.placed_rows}, this rank owns "
                                             f"{me * el}:{(me + 1) * el}")
                        expert_params.add(p)
                    m.ep = ep
            self.ep = ep
        if self.tensor_group is not None:
            from . import tensor

            tensor.shard_model(model, self)
        fs_axes = self.shard_axes()
        if fs_axes:
            from .fsdp import FSDP

            self.fsdp = FSDP(model, self, skip=expert_params, axes=fs_axes)
        # gradients of whole (replicated) parameters are summed over the batch axes;
        # expert shards are replicated only over the batch axes that are not `expert`
        for name, p in model.named_parameters():
            if getattr(p, "_bux_sharded", False):
                # the reduce-scatter summed over the sharding axes; other replicas (HSDP) all-reduce
                axes = tuple(a for a in self.batch_axes if a not in fs_axes)
            elif p in expert_params:
                axes = tuple(a for a in self.batch_axes if a != "expert")
            else:
                axes = self.batch_axes
            g = self.group(axes) if axes else None
            copies = 1
            if g is not None:
                self.replicated.append((p, g))
                copies = dist.get_world_size(g)
            if self.tensor_group is not None and id(p) not in self.tensor_sharded:
                copies *= self.shape["tensor"]
            if copies > 1:
                self._norm_w[name] = 1.0 / copies
        with torch.no_grad():
            for p, g in self.replicated:
                dist.broadcast(p.data, src=dist.get_global_rank(g, 0), group=g)
        # whole parameters with a partial gradient under tensor parallelism: summed there too
        for p in getattr(self, "tensor_partial", ()):
            self.replicated.append((p, self.tensor_group))
        # context parallelism: every rank sees its positions only, so every gradient is partial
        if self.context_group is not None and "context" not in self.batch_axes:
            n = self.shape["context"]
            for name, p in model.named_parameters():
                self.replicated.append((p, self.context_group))
                self._norm_w[name] = self._norm_w.get(name, 1.0) / n
        self._install_early_reduction()

    # ------------------------------------------------------------------ early gradient reduction
    EARLY_BUCKET_BYTES = 64 << 20

    def _install_early_reduction(self) -> None:
        """Replicated parameters' gradients are all-reduced while the backward still runs: as
        each gradient of the step's last microbatch is accumulated it joins a bucket, and a
        full bucket is summed asynchronously (NCCL's stream beside the backward's kernels);
        `finish_grads` waits for the buckets and sums what never passed a hook. Parameters that
        are summed over two groups (context parallelism beside data parallelism) keep the
        late path. Reference: the overlap pass of ``train/reorder.py:46`` there."""
        self._early_on = False
        self._early_open: dict = {}     # group -> (grads, bytes) of the bucket being filled
        self._early_flying: list = []   # (work, flat, grads)
        self._early_done: set = set()
        counts: dict = {}
        for p, _ in self.replicated:
            counts[id(p)] = counts.get(id(p), 0) + 1
        for p, g in self.replicated:
            if counts[id(p)] != 1 or not p.requires_grad:
                continue

            def hook(param, group=g):
                if not self._early_on or param.grad is None:
                    return
                grads, size = self._early_open.get(group, ([], 0))
                grads.append(param.grad)
                size += param.grad.numel() * param.grad.element_size()
                self._early_done.add(id(param))
                if size >= self.EARLY_BUCKET_BYTES:
                    self._launch_bucket(grads, group)
                    grads, size = [], 0
                self._early_open[group] = (grads, size)

            p.register_post_accumulate_grad_hook(hook)

    def _launch_bucket(self, grads: list, group) -> None:
        by_dtype: dict = {}
        for gr in grads:
            by_dtype.setdefault(gr.dtype, []).append(gr)
        for same in by_dtype.values():
            flat = torch.cat([gr.reshape(-1) for gr in same])
            work = dist.all_reduce(flat, group=group, async_op=True)
            self._early_flying.append((work, flat, same))

    def _finish_early(self) -> None:
        for group, (grads, _) in self._early_open.items():
            if grads:
                self._launch_bucket(grads, group)
        self._early_open = {}
        for work, flat, grads in self._early_flying:
            work.wait()
            off = 0
            for gr in grads:
                n = gr.numel()
                gr.copy_(flat[off:off + n].view_as(gr))
                off += n
        self._early_flying = []

    def norm_weight(self, name: str) -> float:
        """Share of a parameter's squared gradient this rank contributes to the global
        norm: 1 for shards, 1/replicas for replicated parameters (summed over all ranks)."""
        return self._norm_w.get(name, 1.0)

    # ------------------------------------------------------------------ gradients
    @contextmanager
    def grad_sync(self, model, last: bool):
        self._early_on = last   # gradients are complete after the last microbatch's backward
        try:
            if self.fsdp is not None:
                with self.fsdp.microbatch(last):
                    yield
            else:
                yield
        finally:
            self._early_on = False

    def finish_grads(self, model) -> None:
        """Sum the gradients of replicated parameters over their replicas (bucketed)."""
        if self.fsdp is not None:
            self.fsdp.finish()
        self._finish_early()
        early, self._early_done = self._early_done, set()
        by_group: dict = {}
        for p, g in self.replicated:
            if id(p) in early:
                continue   # summed while the backward ran
            grad = getattr(p, "main_grad", None)
            grad = grad if grad is not None else p.grad
            if grad is not None:
                by_group.setdefault(g, []).append(grad)
        for g, grads in by_group.items():
            bucket: list = []
            size = 0
            for grad in grads:
                bucket.append(grad)
                size += grad.numel() * grad.element_size()
                if size >= 256 << 20:
                    self._all_reduce_bucket(bucket, g)
                    bucket, size = [], 0
            if bucket:
                self._all_reduce_bucket(bucket, g)

    @staticmethod
    def _all_reduce_bucket(grads: list, group) -> None:
        by_dtype: dict = {}
        for gr in grads:
            by_dtype.setdefault(gr.dtype, []).append(gr)
        for same in by_dtype.values():
            flat = torch.cat([gr.reshape(-1) for gr in same])
            dist.all_reduce(flat, group=group)
            off = 0
            for gr in same:
                n = gr.numel()
                gr.copy_(flat[off:off + n].view_as(gr))
                off += n

    # ------------------------------------------------------------------ scalars
    def sum_scalar(self, t: torch.Tensor, data_only: bool = False) -> torch.Tensor:
        g = self.data_group if data_only else None
        if data_only and g is None:
            return t
        dist.all_reduce(t, group=g)
        return t

    def sum_positions(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks that hold different positions of the same rows."""
        if self.context_group is not None:
            dist.all_reduce(t, group=self.context_group)
        return t

    def positions_span(self, length: int) -> tuple:
        """(start, stop) of this rank's positions of a row of `length`."""
        if self.context_group is None:
            return 0, length
        n, r = self.shape["context"], self.coords["context"]
        if length % n:
            raise ValueError(f"seq_len {length} does not divide over context={n}")
        per = length // n
        return r * per, (r + 1) * per

    def max_int(self, value: int) -> int:
        t = torch.tensor([value], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item())

    def barrier(self) -> None:
        dist.barrier()

    # ------------------------------------------------------------------ checkpoints
    def checkpoint_tree(self, trainer, state_tree):
        """The tree this rank writes: rank 0 writes whole leaves; shards are gathered to
        it first (parameters here are small next to a node's host memory)."""
        tree = state_tree(trainer)
        if self.fsdp is not None:
            tree = self.fsdp.gather_tree(tree)
        if self.tensor_group is not None:
            from . import tensor

            tree = tensor.gather_tree(tree, self)
        if self.expert_group is not None:
            tree = _gather_experts(tree, self.expert_group)
        if getattr(self, "pipeline", None) is not None:
            tree = self.pipeline.gather_tree(tree)
        return tree if self.rank == 0 else None

    def whole_leaf(self, key: str, t):
        """One leaf of the checkpoint's tree put together from every rank's part (all ranks
        call it, in the same order): `checkpoint_tree` for a single leaf, so that a writer can
        go leaf by leaf. `key` is the leaf's key in its part (``name`` or ``kind/name``)."""
        if not isinstance(t, torch.Tensor) or t.dim() == 0:
            return t
        name = key.split("/", 1)[1] if "/" in key else key
        if self.fsdp is not None:
            rows = self.fsdp.sharded.get(name)
            if rows is not None and t.shape[0] * self.fsdp.world == rows:
                t = t.contiguous()
                whole = torch.empty(self.fsdp.world * t.numel(), dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(whole, t.reshape(-1), group=self.fsdp.group)
                t = whole.view(rows, *t.shape[1:])
        lay = self.tensor_layout.get(name)
        if self.tensor_group is not None and lay is not None and t.dim() > lay[0]:
            from . import tensor

            t = tensor.whole(t, lay[0], lay[1], self.tensor_group)
        if self.expert_group is not None and ("experts_gate_up" in name or "experts_down" in name):
            world = dist.get_world_size(self.expert_group)
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous(), group=self.expert_group)
            t = torch.cat(parts, dim=0)
        return t

    def _row_split(self, name: str, rows: int):
        """(parts, index, axes) when the leaf called `name` is cut over the ranks by rows only
        (the whole leaf is `parts` equal slices along its first axis and this rank holds slice
        `index`; `axes` are the mesh axes of the cut), (1, 0, ()) when every rank holds all
        of it, None when it is split another way (tensor parallelism, or two kinds at once)."""
        if self.tensor_group is not None and name in self.tensor_layout:
            return None
        by_expert = self.expert_group is not None and ("experts_gate_up" in name or "experts_down" in name)
        by_fsdp = self.fsdp is not None and name in self.fsdp.sharded
        if by_expert and by_fsdp:
            return None
        if by_fsdp:
            if rows * self.fsdp.world != self.fsdp.sharded[name] and rows != self.fsdp.sharded[name]:
                return None
            return self.fsdp.world, self.fsdp.rank, tuple(self.fsdp.axes)
        if by_expert:
            return self.shape["expert"], dist.get_rank(self.expert_group), ("expert",)
        return 1, 0, ()

    def leaf_placement(self, key: str, t):
        """For a writer that lets every rank write its own rows: (parts, index, writer), where
        `writer` says whether this rank is the one among its replicas that writes slice `index`
        (`t` is this rank's part). None when the leaf has to be put together first."""
        if getattr(self, "pipeline", None) is not None:
            return None
        if not isinstance(t, torch.Tensor) or t.dim() == 0:
            return 1, 0, self.rank == 0
        name = key.split("/", 1)[1] if "/" in key else key     # ``kind/name`` for a moment
        split = self._row_split(name, t.shape[0])
        if split is None:
            return None
        parts, index, axes = split
        if parts > 1 and self.fsdp is not None and name in self.fsdp.sharded \
                and t.shape[0] * parts != self.fsdp.sharded[name]:
            return None        # this rank holds the whole of a leaf its axes would cut: put it together
        first_replica = all(self.coords[a] == 0 for a in M.AXES if a not in axes)
        return parts, index, first_replica

    def restore_rows(self, trainer):
        """``f(name, shape of the whole leaf)`` giving the (lo, hi) rows this rank holds when
        rows are all the leaf is cut by on this mesh, else None (`restore_leaf` then cuts the
        whole leaf). Lets a restore read from disk only what the rank keeps."""
        known = {n for n, _ in trainer.model.named_parameters()} | {n for n, _ in trainer.model.named_buffers()}
        piped = getattr(self, "pipeline", None) is not None

        def rows(name: str, shape):
            if piped or not shape or name not in known:
                return None
            split = self._row_split(name, shape[0])
            if split is None:
                return None
            parts, index, _ = split
            if parts == 1 or shape[0] % parts:
                return None
            if self.fsdp is not None and name in self.fsdp.sharded and shape[0] != self.fsdp.sharded[name]:
                return None
            per = shape[0] // parts
            return index * per, (index + 1) * per

        return rows

    def restore_tree(self, trainer, tree: dict) -> dict:
        """The inverse of `checkpoint_tree`: from a tree of whole leaves (every rank read it),
        what this rank holds. In the reverse order of the gathers: a pipeline stage keeps its
        own layers' leaves, an expert rank its experts, a tensor rank its columns or rows of
        every split parameter, and the sharding axes this rank's rows. Optimizer leaves have
        their parameter's shape in a checkpoint, so one rule serves both."""
        return _restore(self, trainer, tree)

    def restore_leaf(self, trainer):
        """`restore_tree` for one leaf at a time: returns ``f(name, whole tensor)`` giving this
        rank's part (None for a leaf of another pipeline stage)."""
        return _mine(self, trainer)


def _mine(par: "Parallel", trainer):
    """name, tensor → this rank's part of a whole leaf (None: another stage's leaf)."""
    params = dict(trainer.model.named_parameters())
    known = set(params) | {n for n, _ in trainer.model.named_buffers()}
    piped = getattr(par, "pipeline", None) is not None
    ep_world = dist.get_world_size(par.expert_group) if par.expert_group is not None else 1
    ep_rank = dist.get_rank(par.expert_group) if par.expert_group is not None else 0
    tp_world = par.shape["tensor"]
    tp_rank = par.coords["tensor"]

    def mine(name: str, t):
        if not isinstance(t, torch.Tensor) or t.dim() == 0:
            return t
        if name not in known:
            return None if piped else t      # another stage's leaf; otherwise `load` reports it
        if ep_world > 1 and ("experts_gate_up" in name or "experts_down" in name) and t.dim() >= 1:
            t = t.chunk(ep_world, dim=0)[ep_rank]
        lay = par.tensor_layout.get(name)
        if lay is not None and t.dim() > lay[0] and t.shape[lay[0]] == sum(lay[1]):
            from . import tensor

            t = tensor.shard_of(t, lay[0], lay[1], tp_rank, tp_world)
        if par.fsdp is not None and name in par.fsdp.sharded and t.dim() >= 1 \
                and t.shape[0] == par.fsdp.sharded[name]:
            t = t.chunk(par.fsdp.world, dim=0)[par.fsdp.rank]
        return t.contiguous()

    return mine


def _restore(par: "Parallel", trainer, tree: dict) -> dict:
    """This rank's part of every leaf of a tree of whole leaves (see `Parallel.restore_tree`)."""
    mine = _mine(par, trainer)

    def walk(node: dict) -> dict:
        out = {}
        for key, value in node.items():
            if isinstance(value, dict):
                out[key] = walk(value)
            else:
                kept = mine(key.replace("/", "."), value)
                if kept is not None:
                    out[key] = kept
        return out

    return {part: walk(node) if isinstance(node, dict) else node for part, node in tree.items()}


def _gather_experts(tree: dict, group) -> dict:
    world = dist.get_world_size(group)
    for part in tree.values():
        for name in list(part):
            if "experts_gate_up" in name or "experts_down" in name:
                t = part[name]
                full = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(full, t.contiguous(), group=group)
                part[name] = torch.cat(full, dim=0) if t.dim() >= 3 else torch.cat(full)
    return tree


def init_distributed(device: Optional[torch.device] = None) -> bool:
    """Join the job the environment describes (torchrun / SLURM / Open MPI variables).
    Returns whether there is more than one process."""
    env = os.environ
    from .. import runtime

    world = runtime.world_size()
    if world <= 1:
        return False
    if not dist.is_initialized():
        from .. import runtime

        rank = runtime.rank()
        env.setdefault("MASTER_ADDR", "127.0.0.1")
        env.setdefault("MASTER_PORT", "29500")
        backend = "nccl" if device is not None and device.type == "cuda" else "gloo"
        kw = {"device_id": device} if backend == "nccl" else {}
        dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return True
