"""Sharded parameters over the ``fsdp`` axis: ZeRO-3 per block, ZeRO-1/2 per step, HSDP.

Every parameter whose first dimension divides by the axis size keeps only its rows
``[rank*R/n, (rank+1)*R/n)`` (whole rows, like the reference's layout rule,
``parallel/layout.py:95``); the optimizer, the checkpoint and the gradient clip see that
shard under the parameter's own name and shape rank. A *unit* is one block of a repeat
(or the root for what is outside every block). Around a unit's forward the shards of
all its parameters travel in ONE all-gather (``parallel/gather.py:94``), the whole
tensors shadow the module attributes, and they are dropped after the forward; the
gradient of the gather is ONE reduce-scatter per unit (``parallel/gather.py:103``), so
the sharded parameter's ``.grad`` is already this rank's rows of the sum. With
activation checkpointing the replay of a block gathers again (true ZeRO-3: a whole
block lives only while it runs). ``layout(zero=1|2)`` and ``methods(gather="step")``
keep the gathered tensors for all microbatches of a step.

The next unit's all-gather is issued before the current unit runs (forward order in
the forward, reverse order in a replay), so it overlaps the unit's kernels on NCCL's
stream.
"""

from __future__ import annotations

from contextlib import contextmanager

import torch
import torch.distributed as dist
from torch import nn


def _reduce_scatter(out: torch.Tensor, flat: torch.Tensor, group) -> None:
    """out = this rank's slice of the sum of `flat` over the group."""
    if flat.is_cuda:
        dist.reduce_scatter_tensor(out, flat, group=group)
        return
    dist.all_reduce(flat, group=group)  # gloo has no reduce-scatter
    r, n = dist.get_rank(group), out.numel()
    out.copy_(flat[r * n:(r + 1) * n])


class _Gather(torch.autograd.Function):
    """(shards…) → (whole tensors…): one all-gather forward, one reduce-scatter backward."""

    @staticmethod
    def forward(ctx, unit, *shards):
        ctx.unit = unit
        # fresh tensor objects: kept buffers are returned more than once in a step
        return tuple(w.view(w.shape) for w in unit.gather(shards))

    @staticmethod
    def backward(ctx, *grads):
        return (None, *ctx.unit.scatter(grads))


class Unit:
    def __init__(self, module: nn.Module, entries: list, group, reduce_dtype):
        self.module = module
        self.entries = entries            # (owner module, attribute, shard parameter)
        self.group = group
        self.world = dist.get_world_size(group)
        self.reduce_dtype = reduce_dtype
        self.pending = None               # (handle, buffers) of a prefetched all-gather
        self.kept = None                  # whole tensors kept for the step
        self.root = False
        self.shadowed = False

    # -- the collective halves
    def _by_dtype(self, tensors) -> dict:
        groups: dict = {}
        for i, t in enumerate(tensors):
            groups.setdefault(t.dtype, []).append(i)
        return groups

    def start_gather(self, shards=None):
        shards = [e[2].data for e in self.entries] if shards is None else [s.detach() for s in shards]
        work = []
        for dtype, idx in self._by_dtype(shards).items():
            send = torch.cat([shards[i].reshape(-1) for i in idx])
            recv = torch.empty(self.world * send.numel(), dtype=dtype, device=send.device)
            h = dist.all_gather_into_tensor(recv, send, group=self.group, async_op=True)
            work.append((h, recv, idx, send.numel()))
        return work, shards

    def finish_gather(self, work, shards) -> list:
        out = [None] * len(shards)
        for h, recv, idx, per in work:
            h.wait()
            table = recv.view(self.world, per)
            off = 0
            for i in idx:
                n = shards[i].numel()
                rows = shards[i].shape[0]
                out[i] = table[:, off:off + n].reshape(self.world * rows, *shards[i].shape[1:])
                off += n
        return out

    def gather(self, shards) -> list:
        if self.kept is not None:
            return self.kept
        if self.pending is not None:
            work, mine = self.pending
            self.pending = None
        else:
            work, mine = self.start_gather(shards)
        return self.finish_gather(work, mine)

    def scatter(self, grads) -> list:
        shapes = [e[2].shape for e in self.entries]
        out = [None] * len(grads)
        live = [i for i, g in enumerate(grads) if g is not None]
        by: dict = {}
        for i in live:
            by.setdefault(grads[i].dtype, []).append(i)
        for dtype, idx in by.items():
            rd = self.reduce_dtype or dtype
            # [rank][parameter] order, so each rank's slice is contiguous
            parts = [grads[i].reshape(self.world, -1).to(rd) for i in idx]
            flat = torch.cat(parts, dim=1).reshape(-1)
            mine = torch.empty(flat.numel() // self.world, dtype=rd, device=flat.device)
            _reduce_scatter(mine, flat, self.group)
            off = 0
            for i in idx:
                n = grads[i].numel() // self.world
                out[i] = mine[off:off + n].view(shapes[i]).to(dtype)
                off += n
        return out

    # -- shadowing the module attributes with the whole tensors
    def shadow(self, keep: bool) -> None:
        if self.shadowed:
            return
        params = [e[2] for e in self.entries]
        if torch.is_grad_enabled() and any(p.requires_grad for p in params):
            whole = _Gather.apply(self, *params)
        else:
            whole = self.gather([p.data for p in params])
        if keep and self.kept is None:
            self.kept = [w.detach() for w in whole]
        for (owner, attr, _), w in zip(self.entries, whole):
            owner.__dict__[attr] = w
        self.shadowed = True

    def unshadow(self) -> None:
        if not self.shadowed:
            return
        for owner, attr, _ in self.entries:
            owner.__dict__.pop(attr, None)
        self.shadowed = False


class FSDP:
    def __init__(self, model: nn.Module, par, skip=(), axes=("fsdp",)):
        t = par.train
        self.axes = tuple(axes)
        self.group = par.group(self.axes)
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.keep = t.layout.zero < 3 or getattr(t.methods, "gather", "layer") == "step"
        reduce = getattr(t.precision, "reduce", None)
        self.reduce_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}.get(reduce)
        self.sharded: dict = {}           # parameter name → rows of the whole parameter
        skip = {id(p) for p in skip}
        blocks = self._blocks(model)
        self.units: list = []
        taken: set = set()
        for block in (*blocks, model):
            entries = []
            for owner in block.modules():
                for attr, p in list(owner._parameters.items()):
                    if p is None or id(p) in taken or id(p) in skip:
                        continue
                    if block is model and any(owner is m for b in blocks for m in b.modules()):
                        continue
                    taken.add(id(p))
                    if p.dim() == 0 or p.shape[0] % self.world != 0 or p.shape[0] < self.world:
                        continue  # stays whole on every rank (replicated, all-reduced)
                    rows = p.shape[0] // self.world
                    local = nn.Parameter(p.data[self.rank * rows:(self.rank + 1) * rows].clone(),
                                         requires_grad=p.requires_grad)
                    for k, v in p.__dict__.items():
                        setattr(local, k, v)
                    local._bux_sharded = True
                    local._bux_rows = p.shape[0]
                    owner._parameters[attr] = local
                    entries.append((owner, attr, local))
            if entries:
                unit = Unit(block, entries, self.group, self.reduce_dtype)
                unit.root = block is model
                self.units.append(unit)
                self._hook(unit, len(self.units) - 1, root=block is model)
        for name, p in model.named_parameters():
            if getattr(p, "_bux_sharded", False):
                self.sharded[name] = p._bux_rows

    @staticmethod
    def _blocks(model: nn.Module) -> list:
        from ..models.graph import Repeated

        out = []
        for m in model.modules():
            if isinstance(m, Repeated) and not any(m is c for b in out for c in b.modules()):
                out.extend(m.items)
        return out

    def _hook(self, unit: Unit, index: int, root: bool) -> None:
        def pre(module, args, kwargs=None):
            unit.shadow(self.keep)
            if root:
                return
            # the neighbour that runs next: after this one in a forward, before it in a replay
            nxt = index - 1 if torch.is_grad_enabled() and self._replaying(args) else index + 1
            if 0 <= nxt < len(self.units):
                other = self.units[nxt]
                if other.pending is None and other.kept is None and not other.shadowed and not other.root:
                    other.pending = other.start_gather()

        def post(module, args, output):
            unit.unshadow()

        unit.module.register_forward_pre_hook(pre)
        unit.module.register_forward_hook(post)

    @staticmethod
    def _replaying(args) -> bool:
        x = args[0] if args else None
        return isinstance(x, torch.Tensor) and x.is_leaf and x.requires_grad

    # ------------------------------------------------------------------ the step
    @contextmanager
    def microbatch(self, last: bool):
        yield

    def finish(self) -> None:
        for u in self.units:
            u.kept = None
            u.pending = None
            u.unshadow()

    # ------------------------------------------------------------------ checkpoints
    def gather_tree(self, tree: dict) -> dict:
        """Whole leaves from shards, for the rank that writes (every rank takes part)."""
        for part in tree.values():
            for key in list(part):
                name = key.split("/", 1)[1] if "/" in key else key
                rows = self.sharded.get(name)
                t = part[key]
                if rows is None or not isinstance(t, torch.Tensor) or t.dim() == 0 or t.shape[0] * self.world != rows:
                    continue
                t = t.contiguous()
                whole = torch.empty(self.world * t.numel(), dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(whole, t.reshape(-1), group=self.group)
                part[key] = whole.view(rows, *t.shape[1:])
        return tree

    def shard_tree(self, tree: dict) -> dict:
        """The inverse for a restore: this rank's rows of every sharded leaf."""
        for part in tree.values():
            for key in list(part):
                name = key.split("/", 1)[1] if "/" in key else key
                rows = self.sharded.get(name)
                t = part[key]
                if rows is None or not hasattr(t, "shape") or len(t.shape) == 0 or t.shape[0] != rows:
                    continue
                n = rows // self.world
                part[key] = t[self.rank * n:(self.rank + 1) * n]
        return tree
