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

``compiler(options="--fsdp=fused")`` replaces both collectives by this library's own kernels
over NVLink peer memory (`FusedComm`; bf16 parameters on GPUs):

* the all-gather becomes peer stores: every owner writes its rows of each parameter into
  every rank's staging buffer (`tp_push_block`) on a side stream, one unit ahead, and raises
  a flag; a GEMM that takes a gathered weight as its B operand waits *in its TMA producer
  warp*, per tile of output columns, for the flag of the rank that owns those rows
  (``wait_on_n``), so the gather is part of the first GEMM that consumes it, and whatever
  else reads a gathered parameter waits for the flags on the stream;
* the reduce-scatter becomes peer loads: a unit's whole gradients are written into this
  rank's staging buffer, a flag is raised, and each rank sums its own rows out of every
  rank's buffer in fp32 (`tp_pull_reduce`), casts and hands the result to autograd, on a side
  stream, beside the backward of the unit before it.

Staging buffers come in two slots per direction; a slot is written again only after every
rank has flagged that it is done with what the slot held (bounded waits, as everywhere).
Reference: ``parallel/gather.py:94-114`` and the overlap pass ``train/reorder.py:46`` there.
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


SLOT_ROOT = 2                                   # slots 0 and 1 alternate between the blocks
CH_GATHER, CH_READ, CH_GRAD, CH_PULLED, CH_SMALL = 0, 3, 6, 9, 12   # + slot


class FusedComm:
    """Symmetric staging memory, flags and the side stream of the in-kernel all-gather and
    reduce-scatter. Two slots per direction alternate between the repeated blocks; what is
    outside every block (embedding, head: gathered once and used through the whole forward)
    has a slot of its own."""

    def __init__(self, group, device, units: list):
        import torch.distributed._symmetric_memory as symm

        self.group, self.device = group, device
        self.world, self.me = dist.get_world_size(group), dist.get_rank(group)
        # per unit: (offset, bytes) of each parameter's whole tensor in its slot, 256-byte aligned
        self.layout: dict = {}
        sizes = {False: 0, True: 0}
        for u in units:
            at, pieces = 0, []
            for _, _, p in u.entries:
                size = p.numel() * self.world * p.element_size()
                pieces.append((at, size))
                at += -(-size // 256) * 256
            self.layout[id(u)] = pieces
            sizes[u.root] = max(sizes[u.root], at)
        block, root = sizes[False], sizes[True]
        per_kind = 2 * block + root
        self.slot_at = {0: 0, 1: block, SLOT_ROOT: 2 * block}
        self.kind_at = {0: 0, 1: per_kind}            # 0: gathered parameters, 1: whole gradients
        flags_at = 2 * per_kind
        heap = symm.empty(flags_at + 15 * self.world * 4, dtype=torch.uint8, device=device)
        hdl = symm.rendezvous(heap, group.group_name)
        heap.zero_()
        self.heap = heap
        self.bases = [int(b) for b in hdl.buffer_ptrs]
        self.flags = heap[flags_at:].view(torch.int32).view(15, self.world)
        self.peer_flags = torch.tensor([b + flags_at for b in self.bases], dtype=torch.int64, device=device)
        self.epoch = [0] * 15
        self.side = torch.cuda.Stream(device=device)
        self._tables: dict = {}
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def region(self, kind: int, slot: int, offset: int, size: int) -> torch.Tensor:
        start = self.kind_at[kind] + self.slot_at[slot] + offset
        return self.heap[start:start + size]

    def table(self, kind: int, slot: int, offset: int) -> torch.Tensor:
        key = (kind, slot, offset)
        if key not in self._tables:
            start = self.kind_at[kind] + self.slot_at[slot] + offset
            self._tables[key] = torch.tensor([b + start for b in self.bases], dtype=torch.int64, device=self.device)
        return self._tables[key]

    def signal(self, ch: int) -> int:
        from ..ops import kernels as K

        self.epoch[ch] += 1
        K.ep_signal(self.peer_flags, ch, self.world, self.me, self.epoch[ch])
        return self.epoch[ch]

    def wait(self, ch: int, epoch: int) -> None:
        from ..ops import kernels as K

        if epoch > 0:
            K.ep_wait(self.flags[ch], epoch)


class _Gather(torch.autograd.Function):
    """(shards…) → (whole tensors…): one all-gather forward, one reduce-scatter backward."""

    @staticmethod
    def forward(ctx, unit, *shards):
        ctx.unit = unit
        ctx.releases = unit.fused is not None and unit.release_in_backward
        # fresh tensor objects: kept buffers are returned more than once in a step
        return tuple(w.view(w.shape) for w in unit.gather(shards))

    @staticmethod
    def backward(ctx, *grads):
        if ctx.releases:
            # the unit's backward read the gathered weights where they arrived: the slot is free now
            ctx.unit._fused_release()
        return (None, *ctx.unit.scatter(grads))


class _Copy(torch.autograd.Function):
    """A copy out of a staging slot that autograd sees through."""

    @staticmethod
    def forward(ctx, w):
        return w.clone()

    @staticmethod
    def backward(ctx, g):
        return g


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
        self.fused = None                 # a `FusedComm`: the collectives by this library's kernels
        self.in_kernel_wait = False       # GEMMs wait for their gathered weight themselves (bf16 matmuls)
        self.gemm_weights: list = []      # per entry: whether only `ops.linear` reads the parameter
        self.arrivals: list = []
        self.reading = None
        self.release_in_backward = False
        self.index = 0
        self.pending_grads: list = []     # (event, sources) of reductions still running on the side stream
        self.hold = False                 # keep this microbatch's whole gradients here, reduce later
        self.held: list = []              # whole gradients of the step's earlier microbatches

    # -- the collective halves
    def _by_dtype(self, tensors) -> dict:
        groups: dict = {}
        for i, t in enumerate(tensors):
            groups.setdefault(t.dtype, []).append(i)
        return groups

    # -- the same two halves by this library's kernels over peer memory
    def _slot(self) -> int:
        return SLOT_ROOT if self.root else self.index % 2

    def _fused_start(self, shards):
        """Push this rank's rows of every parameter of the unit into every rank's staging slot,
        on the side stream. Returns (slot, epoch) for `_fused_finish`."""
        from ..ops import kernels as K

        fc, slot = self.fused, self._slot()
        main = torch.cuda.current_stream(fc.device)
        fc.side.wait_stream(main)
        with torch.cuda.stream(fc.side):
            # every rank must have finished reading what the slot held before
            fc.wait(CH_READ + slot, fc.epoch[CH_READ + slot])
            # what no GEMM waits for in its own kernel goes first, under a flag of its own
            small = None
            for late in (False, True):
                for (off, size), shard, gemm in zip(fc.layout[id(self)], shards, self.gemm_weights):
                    if (gemm and self.in_kernel_wait) != late:
                        continue
                    flat = shard.contiguous().view(-1).view(torch.bfloat16)
                    mine = fc.region(0, slot, off, size).view(torch.bfloat16).view(fc.world, flat.numel())
                    mine[fc.me].copy_(flat)
                    K.tp_push_block(flat.view(1, -1), fc.table(0, slot, off), fc.me)
                if not late:
                    small = fc.signal(CH_SMALL + slot)
            epoch = fc.signal(CH_GATHER + slot)
        return slot, small, epoch

    def _fused_finish(self, work, shards) -> list:
        """The whole parameters as views of the staging slot, and for each the flags a GEMM
        that takes it as its B operand can wait on (`arrivals`); the stream itself waits only
        if something other than such a GEMM reads the unit's parameters."""
        fc = self.fused
        slot, small, epoch = work
        out, self.arrivals = [], []
        for (off, size), shard, gemm in zip(fc.layout[id(self)], shards, self.gemm_weights):
            rows = shard.shape[0]
            whole = fc.region(0, slot, off, size).view(shard.dtype).view(fc.world * rows, *shard.shape[1:])
            waits_itself = gemm and self.in_kernel_wait
            self.arrivals.append((fc.flags[CH_GATHER + slot], epoch, rows) if waits_itself else None)
            out.append(whole)
        fc.wait(CH_SMALL + slot, small)
        if not self.in_kernel_wait:
            fc.wait(CH_GATHER + slot, epoch)
        self.reading = slot
        return out

    def _fused_release(self) -> None:
        """Tell every rank that this rank no longer reads the slot: after a forward without a
        backward to come, or after the backward of the unit that was run from the slot."""
        slot = getattr(self, "reading", None)
        if slot is not None:
            self.fused.signal(CH_READ + slot)
            self.reading = None

    def _fused_scatter(self, grads) -> list:
        """Whole gradients → this rank's rows of their sum over the ranks, by peer loads on the
        side stream, beside the backward of the unit that comes next."""
        from ..ops import kernels as K

        fc, slot = self.fused, self._slot()
        main = torch.cuda.current_stream(fc.device)
        self.pending_grads = [(ev, src) for ev, src in self.pending_grads if not ev.query()]
        shapes = [e[2].shape for e in self.entries]
        out = [None] * len(grads)
        live = [i for i, g in enumerate(grads) if g is not None]
        # outputs come from the main stream's pool: the side stream is made to wait for the main
        # one below, so whatever used their memory before has finished by then
        for i in live:
            out[i] = torch.empty(shapes[i], dtype=grads[i].dtype, device=fc.device)
        fc.side.wait_stream(main)
        with torch.cuda.stream(fc.side):
            fc.wait(CH_PULLED + slot, fc.epoch[CH_PULLED + slot])   # every rank pulled what the slot held
            for i in live:
                off, size = fc.layout[id(self)][i]
                fc.region(1, slot, off, size).view(grads[i].dtype).view(grads[i].shape).copy_(grads[i])
            epoch = fc.signal(CH_GRAD + slot)
            fc.wait(CH_GRAD + slot, epoch)
            for i in live:
                off, size = fc.layout[id(self)][i]
                K.tp_pull_reduce(fc.table(1, slot, off), fc.me, out[i].view(1, -1))
            fc.signal(CH_PULLED + slot)
            done = torch.cuda.Event()
            done.record(fc.side)
        # the sources stay alive until the side stream has copied them
        self.pending_grads.append((done, [grads[i] for i in live]))
        if any(self.entries[i][2].grad is not None for i in live):
            main.wait_event(done)   # a later microbatch: autograd adds to .grad on the main stream at once
        return out

    def start_gather(self, shards=None):
        shards = [e[2].data for e in self.entries] if shards is None else [s.detach() for s in shards]
        if self.fused is not None:
            return self._fused_start(shards), shards
        work = []
        for dtype, idx in self._by_dtype(shards).items():
            send = torch.cat([shards[i].reshape(-1) for i in idx])
            recv = torch.empty(self.world * send.numel(), dtype=dtype, device=send.device)
            h = dist.all_gather_into_tensor(recv, send, group=self.group, async_op=True)
            work.append((h, recv, idx, send.numel()))
        return work, shards

    def finish_gather(self, work, shards) -> list:
        if self.fused is not None:
            return self._fused_finish(work, shards)
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
        if self.hold or self.held:
            # gradients stay whole on this rank until the step's last microbatch
            if not self.held:
                self.held = [None] * len(grads)
            for i, g in enumerate(grads):
                if g is not None:
                    self.held[i] = g.clone() if self.held[i] is None else self.held[i].add_(g)
            if self.hold:
                return [None] * len(grads)
            grads, self.held = self.held, []
        if self.fused is not None and all(g is None or (g.dtype == torch.bfloat16 and g.is_cuda) for g in grads):
            return self._fused_scatter([None if g is None else g.contiguous() for g in grads])
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
    def shadow(self, keep: bool, replay: bool = False) -> None:
        if self.shadowed:
            return
        params = [e[2] for e in self.entries]
        grad_mode = torch.is_grad_enabled() and any(p.requires_grad for p in params)
        fused_now = self.fused is not None and self.kept is None
        # gathered weights live in a staging slot that the next-but-one unit overwrites: a
        # forward whose backward comes much later (no checkpointing), or weights kept for the
        # whole step, are copied out; a checkpointed replay reads them in place and frees the
        # slot after its backward; a forward without gradients frees it when the unit is left
        copy_out = fused_now and (keep or (grad_mode and not replay))
        self.release_in_backward = fused_now and grad_mode and not copy_out
        if grad_mode:
            whole = _Gather.apply(self, *params)
        else:
            whole = self.gather([p.data for p in params])
        arrivals = self.arrivals if fused_now else []
        if copy_out:
            if any(a is not None for a in arrivals):   # nothing waited for the GEMM weights yet
                slot = self._slot()
                self.fused.wait(CH_GATHER + slot, self.fused.epoch[CH_GATHER + slot])
            whole = [w.clone() for w in whole] if not grad_mode else [_Copy.apply(w) for w in whole]
            arrivals = []
            self._fused_release()
        if keep and self.kept is None:
            self.kept = [w.detach() for w in whole]
        for k, ((owner, attr, _), w) in enumerate(zip(self.entries, whole)):
            if k < len(arrivals) and arrivals[k] is not None:
                w._bux_arrival = arrivals[k]
            owner.__dict__[attr] = w
        self.shadowed = True

    def unshadow(self) -> None:
        if not self.shadowed:
            return
        for owner, attr, _ in self.entries:
            owner.__dict__.pop(attr, None)
        self.shadowed = False
        if self.fused is not None and not self.release_in_backward:
            self._fused_release()


class FSDP:
    def __init__(self, model: nn.Module, par, skip=(), axes=("fsdp",)):
        t = par.train
        self.axes = tuple(axes)
        self.group = par.group(self.axes)
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.keep = t.layout.zero < 3 or getattr(t.methods, "gather", "layer") == "step"
        # accumulate="unreduced": whole gradients are summed on this rank over the microbatches
        # of a step and reduce-scattered once, with the last microbatch (the reference's
        # `_unreduced` path, ``train/trainer.py:844``); "reduced" and "auto": every microbatch
        self.unreduced = getattr(t.methods, "accumulate", "auto") == "unreduced"
        reduce = getattr(t.precision, "reduce", None)
        self.reduce_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}.get(reduce)
        self.sharded: dict = {}           # parameter name → rows of the whole parameter
        options = getattr(getattr(t, "compiler", None), "options", "") or ""
        self.fused_comm = None
        fused = "--fsdp=fused" in options.split() and par.device.type == "cuda"
        if fused:
            from .. import runtime

            if not runtime.on_one_node(self.group):   # peer-memory kernels: one machine only
                import warnings

                warnings.warn("compiler(options=\"--fsdp=fused\"): the sharding axes span machines; taking NCCL")
                fused = False
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
                    if getattr(p, "placed_whole", None) is not None:
                        # built as this rank's rows already (`models.placement`): adopted as it is
                        p._bux_sharded, p._bux_rows = True, p.placed_whole
                        entries.append((owner, attr, p))
                        continue
                    if p.dim() == 0 or p.shape[0] % self.world != 0 or p.shape[0] < self.world:
                        continue  # stays whole on every rank (replicated, all-reduced)
                    if fused and (p.dtype != torch.bfloat16 or (p.numel() // self.world * 2) % 16):
                        continue  # the peer-memory kernels move bf16 in 16-byte pieces: the rest stays whole
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
        if fused and self.units:
            from ..models.layers.basic import Linear

            # only with bf16 matmuls does a GEMM read the gathered weight itself; a block-scaled
            # linear quantises it first, so there the stream waits for the whole unit
            roles = {k: v for k, v in t.precision.roles.model_dump().items() if k != "type" and v is not None}
            plain = t.precision.matmuls in ("compute", None) and not roles
            self.fused_comm = FusedComm(self.group, par.device, self.units)
            for i, u in enumerate(self.units):
                u.fused, u.index = self.fused_comm, i
                u.in_kernel_wait = plain and not u.root
                u.gemm_weights = [isinstance(owner, Linear) and attr == "weight" and p.dim() == 2
                                  for owner, attr, p in u.entries]

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
            replay = torch.is_grad_enabled() and self._replaying(args)
            unit.shadow(self.keep, replay)
            if root:
                return
            # the neighbour that runs next: after this one in a forward, before it in a replay
            nxt = index - 1 if replay else index + 1
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
        for u in self.units:
            u.hold = self.unreduced and not last
        yield

    def finish(self) -> None:
        if self.fused_comm is not None:
            # the last reductions run on the side stream: the optimizer comes after them
            torch.cuda.current_stream(self.fused_comm.device).wait_stream(self.fused_comm.side)
        for u in self.units:
            if u.pending is not None and u.fused is not None:
                # a prefetched gather that nothing consumed: take it and free its slot
                u.finish_gather(*u.pending)
                u._fused_release()
            u.kept = None
            u.pending = None
            u.pending_grads = []
            u.held = []
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
