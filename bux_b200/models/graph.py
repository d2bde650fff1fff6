"""IR graph → module tree. One module class per node kind; layers come from the
registry. Attribute names (``items``, ``body``, ``terms``, ``factors``) follow the IR so
that parameter paths read like the graph (``graph.items.1.items.0.body.items.1.q``).

Reference counterparts: ``architecture/graph.py:37-241`` and the repeat builders in
``architecture/repeats/repeat.py:38-141``.
"""

from __future__ import annotations

import copy
from typing import Optional

import torch
from torch import nn

from ..lang import ir
from .registry import BuildContext, Context, build_layer


class Sequence(nn.Module):
    def __init__(self, items):
        super().__init__()
        self.items = nn.ModuleList(items)

    def forward(self, x, ctx: Context):
        for item in self.items:
            x = item(x, ctx)
        return x


class ResidualBranch(nn.Module):
    """``[body]``: x + body(x), or whatever the residual algebra makes of a branch."""

    def __init__(self, body, algebra: Optional[nn.Module] = None, name: str = "branch"):
        super().__init__()
        self.body = body
        self.name = name   # what observed values of this branch are filed under
        if algebra is not None:
            self.algebra = algebra

    def forward(self, x, ctx: Context):
        algebra = getattr(self, "algebra", None)
        ctx.branch_index += 1
        outer = ctx.branch_depth == 0
        if outer:   # precision(first=..., last=...) counts these
            ctx.precision.branch = ctx.top_branch
            ctx.top_branch += 1
        observing = outer and ctx.observing
        if observing:   # values observed inside are filed under gqa.00, moe.03, ...
            from . import observe

            count = ctx.branch_names.get(self.name, 0)
            ctx.branch_names[self.name] = count + 1
            ctx.observed_branch = f"{self.name}.{count:02d}"
        ctx.branch_depth += 1
        try:
            y = algebra(x, self.body, ctx) if algebra is not None else x + self.body(x, ctx)
            if observing:
                observe.stream(ctx, x, y)
            return y
        finally:
            ctx.branch_depth -= 1
            if outer:
                ctx.precision.branch = -1
                ctx.observed_branch = None


class Parallel(nn.Module):
    def __init__(self, terms, product: bool):
        super().__init__()
        name = "factors" if product else "terms"
        setattr(self, name, nn.ModuleList(terms))
        self.product = product

    def forward(self, x, ctx: Context):
        parts = self.factors if self.product else self.terms
        out = None
        for part in parts:
            y = part(x, ctx)
            if out is None:
                out = y
            else:
                out = out * y if self.product else out + y
        return out


class Negate(nn.Module):
    def __init__(self, body):
        super().__init__()
        self.body = body

    def forward(self, x, ctx):
        return -self.body(x, ctx)


class Constant(nn.Module):
    def __init__(self, value: float):
        super().__init__()
        self.value = value

    def forward(self, x, ctx):
        return self.value


class Identity(nn.Module):
    def forward(self, x, ctx):
        return x


class TapWrite(nn.Module):
    def __init__(self, name: str):
        super().__init__()
        self.name = name

    def forward(self, x, ctx: Context):
        ctx.push(self.name, x)
        return x


class TapRead(nn.Module):
    def __init__(self, name: str, pop: bool):
        super().__init__()
        self.name, self.pop = name, pop

    def forward(self, x, ctx: Context):
        return ctx.read(self.name, self.pop)


class Repeated(nn.Module):
    """``body^n``: n copies with their own parameters, run in order. `remat` wraps each
    pass in activation checkpointing (only its input is kept for the backward)."""

    def __init__(self, items, shared_body: bool = False):
        super().__init__()
        self.items = nn.ModuleList(items)
        self.remat = False
        self.offload = False  # keep each pass's input in pinned host memory
        # keep attention outputs too, so the replay skips that kernel: True for every pass, or
        # a count for the last so many passes only (what the device has room for)
        self.keep_attention = False
        self.kept_to_host = False  # with `offload`, kept outputs follow the inputs to pinned host memory
        self.first = None          # checkpoint only the first so many passes; the rest keep everything

    def forward(self, x, ctx: Context):
        for i, item in enumerate(self.items):
            if (self.remat and ctx.training and torch.is_grad_enabled() and isinstance(x, torch.Tensor)
                    and x.requires_grad and (self.first is None or i < self.first)):
                keep, to_host = self.keep_attention, self.kept_to_host
                if keep is not True and keep is not False:
                    on_device = i >= len(self.items) - int(keep)
                    # the last `keep` passes hold their outputs on the device; with `kept_to_host`
                    # the earlier ones send theirs after their inputs to pinned host memory
                    keep, to_host = (on_device or to_host), (to_host and not on_device)
                x = _checkpointed(item, x, ctx, self.offload, (id(self), i), keep, to_host)
            else:
                x = item(x, ctx)
        return x


_OFFLOADED: list = []   # blocks whose inputs sit in host memory, in forward order
_SIDE: dict = {}
_IN_FLIGHT: list = []   # (event, tensors) of device → host copies whose sources are still held


def _hold_until_copied(event, tensors) -> None:
    """Keep `tensors` alive until the side-stream copy that reads them is done.

    Their memory goes back to the allocator only after the main stream has been made to
    wait for the copy, so the allocator's own stream order covers the reuse. (Marking the
    tensors as used by the side stream instead would leave each freed block unusable until
    the host sees the copy finished; a host that runs a step ahead of the device then
    holds every block's input twice.)"""
    _IN_FLIGHT.append((event, tensors))


def _release_copied(device, keep_last: int = 0) -> None:
    """Let go of the sources of all but the newest `keep_last` copies in flight."""
    while len(_IN_FLIGHT) > keep_last:
        event, tensors = _IN_FLIGHT.pop(0)
        torch.cuda.current_stream(device).wait_event(event)
        del tensors


def _side_stream(device):
    key = torch.device(device).index
    if key not in _SIDE:
        _SIDE[key] = torch.cuda.Stream(device=device)
    return _SIDE[key]


class _Remat(torch.autograd.Function):
    """Activation checkpointing of one block: the forward keeps only the block's input
    (optionally in pinned host memory), the backward reruns the block and differentiates
    it. Auxiliary losses the block reports are outputs of the function, so their
    gradients reach the block's parameters too."""

    @staticmethod
    def forward(fctx, x, holder, *outside):
        # `outside`: tensors on the taps when the block starts (written by earlier layers) that
        # carry gradients. They are inputs of this function, so what the block's replay sends
        # back to them goes on through the graph that made them, once, with everything else.
        fctx.holder = holder
        fctx.set_materialize_grads(False)   # an output nobody read has no gradient: skip it, do not make zeros
        fctx.cuda_rng = torch.cuda.get_rng_state(x.device) if x.is_cuda else None
        fctx.cpu_rng = torch.get_rng_state()
        fctx.host = None
        if holder.offload and x.is_cuda:
            # the copy runs on a side stream so the block's kernels do not wait for PCIe; the
            # copy of the block before this one has had a whole block's time to finish
            _release_copied(x.device)
            host = holder.pinned(x)
            side = _side_stream(x.device)
            side.wait_stream(torch.cuda.current_stream(x.device))
            with torch.cuda.stream(side):
                host.copy_(x, non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(side)
            _hold_until_copied(copied, (x,))
            fctx.host = host
            fctx.device = x.device
            fctx.fetched = None
            _OFFLOADED.append(fctx)
            fctx.save_for_backward(*outside)
        else:
            fctx.save_for_backward(x, *outside)
        with torch.no_grad():
            y, aux = holder.run(x, replay=False)
        if fctx.host is not None and holder.kept and holder.kept_to_host:
            # kept attention outputs follow the block's input to the host
            side = _side_stream(x.device)
            side.wait_stream(torch.cuda.current_stream(x.device))
            hosted, sources = [], []
            with torch.cuda.stream(side):
                for i, pair in enumerate(holder.kept):
                    on_host = []
                    for j, t in enumerate(pair):
                        h = holder.pinned(t, slot=(i, j))
                        h.copy_(t, non_blocking=True)
                        sources.append(t)
                        on_host.append(h)
                    hosted.append(tuple(on_host))
                copied = torch.cuda.Event()
                copied.record(side)
            _hold_until_copied(copied, tuple(sources))
            holder.kept = hosted
        # what the block pushed onto taps leaves as outputs too: a later reader's gradient
        # comes back to this block instead of stopping at a tensor made without a graph
        return (y, *aux, *holder.pushed)

    @staticmethod
    def _fetch(fctx) -> None:
        """Start the host → device copies of a block's input (and of the attention
        outputs kept with it) on the side stream."""
        main = torch.cuda.current_stream(fctx.device)
        side = _side_stream(fctx.device)
        buf = torch.empty(fctx.host.shape, dtype=fctx.host.dtype, device=fctx.device)
        kept = fctx.holder.kept if fctx.holder.kept_to_host else None
        back = None
        if kept:
            back = [tuple(torch.empty(h.shape, dtype=h.dtype, device=fctx.device) for h in pair) for pair in kept]
        side.wait_stream(main)  # the buffers' previous owners ran on the main stream
        with torch.cuda.stream(side):
            buf.copy_(fctx.host, non_blocking=True)
            if back is not None:
                for pair, dst in zip(kept, back):
                    for h, d in zip(pair, dst):
                        d.copy_(h, non_blocking=True)
            done = torch.cuda.Event()
            done.record(side)
        if back is not None:
            fctx.holder.kept = back
        fctx.fetched = (buf, done)

    @staticmethod
    def backward(fctx, dy, *daux):
        holder = fctx.holder
        if fctx.host is not None:
            _release_copied(fctx.device)
            if fctx.fetched is None:
                _Remat._fetch(fctx)
            x, done = fctx.fetched
            fctx.fetched = None
            torch.cuda.current_stream(fctx.device).wait_event(done)
            if _OFFLOADED and _OFFLOADED[-1] is fctx:
                _OFFLOADED.pop()
            # the block that goes backward next: its input travels while this one computes
            if _OFFLOADED and _OFFLOADED[-1].fetched is None:
                _Remat._fetch(_OFFLOADED[-1])
            outside = fctx.saved_tensors
        else:
            x, *outside = fctx.saved_tensors
        x = x.detach().requires_grad_(True)
        # the replay reads detached stand-ins for the tensors other layers wrote: its backward
        # stops at them, and their gradients leave through this function's return
        stand_ins = [t.detach().requires_grad_(True) for t in outside]
        devices = [x.device] if x.is_cuda else []
        with torch.random.fork_rng(devices=devices):
            torch.set_rng_state(fctx.cpu_rng)
            if fctx.cuda_rng is not None:
                torch.cuda.set_rng_state(fctx.cuda_rng, x.device)
            with torch.enable_grad():
                y, aux = holder.run(x, replay=True, stand_ins={id(t): r for t, r in zip(outside, stand_ins)})
        outs, grads = [], []
        for o, g in zip((y, *aux, *holder.pushed), (dy, *daux)):
            if o.requires_grad and g is not None:
                outs.append(o)
                grads.append(g)
        if outs:
            torch.autograd.backward(outs, grads)
        # The forward's context reaches this node (context -> heads -> hidden states -> their
        # graph -> this node) and this node reached the context through the holder: a cycle
        # through autograd's C++ edges, which Python's collector cannot see. Cut it here, or
        # every step's context (its hidden states, tables, positions) stays alive for good.
        fctx.holder = None
        holder.ctx = holder.block = None
        holder.taps = holder.ports = None
        holder.pushed = []
        return (x.grad, None, *(r.grad for r in stand_ins))


class _BlockRun:
    """Runs a block for `_Remat`: the first run records taps / metrics as usual and
    returns the auxiliary losses it reported; the replay records nothing."""

    _pinned: dict = {}

    def __init__(self, block, ctx: Context, offload: bool, key, keep_attention: bool = False,
                 kept_to_host: bool = False):
        self.block, self.ctx, self.offload, self.key = block, ctx, offload, key
        self.kept = [] if keep_attention else None
        self.kept_to_host = kept_to_host
        self.names: list = []
        self.taps = {k: list(v) for k, v in ctx.taps.items()}
        self.ports = dict(ctx.ports)
        self.branches = (ctx.branch_index, ctx.top_branch)   # where the block's first run starts counting
        self.pushed: list = []   # tensors the block's last run left on the taps (its own writes)

    def outside(self) -> list:
        """Tensors on the taps at the block's start that carry gradients (each once)."""
        seen, out = set(), []
        for stack in self.taps.values():
            for value in stack:
                for t in _tensors_of(value):
                    if t.requires_grad and id(t) not in seen:
                        seen.add(id(t))
                        out.append(t)
        return out

    def pinned(self, x, slot=None):
        k = (self.key, slot, tuple(x.shape), x.dtype)
        buf = _BlockRun._pinned.get(k)
        if buf is None:
            buf = torch.empty(x.shape, dtype=x.dtype, device="cpu", pin_memory=True)
            _BlockRun._pinned[k] = buf
        return buf

    def run(self, x, replay: bool, stand_ins=None):
        ctx = self.ctx
        before = {id(t) for stack in self.taps.values() for value in stack for t in _tensors_of(value)}
        saved = (ctx.taps, ctx.losses, ctx.metrics, ctx.ports, ctx.branch_index, ctx.top_branch)
        ctx.losses = {}
        was_observing = ctx.observing
        if replay:
            ctx.observing = False   # the first run observed
            ctx.branch_index, ctx.top_branch = self.branches   # the branches count as in the first run
            ctx.taps = {k: [_swapped(value, stand_ins) for value in v] for k, v in self.taps.items()}
            ctx.metrics, ctx.ports = {}, dict(self.ports)
            ctx.tail_values_unused = _ends_in_plain_moe_branch(self.block)
        from ..ops import functional as OF

        if self.kept is not None:
            OF.attention_replay = ("load", iter(self.kept)) if replay else ("save", self.kept)
        try:
            y = self.block(x, ctx)
            reported = ctx.losses
            # what this run left on the taps that was not there before (a tap pushed and popped
            # inside the block never shows): in the order the stacks hold them, so the first run
            # and the replay list the same writes
            swapped = {id(r) for r in (stand_ins or {}).values()}
            self.pushed = [t for stack in ctx.taps.values() for value in stack for t in _tensors_of(value)
                           if id(t) not in before and id(t) not in swapped and t.is_floating_point()]
        finally:
            OF.attention_replay = None
            ctx.tail_values_unused = False
            ctx.observing = was_observing
            if replay:
                self.kept = None
            if replay:
                ctx.taps, ctx.losses, ctx.metrics, ctx.ports, ctx.branch_index, ctx.top_branch = saved
            else:
                ctx.losses = saved[1]
        if not replay:
            self.names = list(reported)
        return y, [reported[n] for n in self.names]


def _tensors_of(value) -> tuple:
    """The tensors of a tap's entry: the entry itself, or the members of a tuple or list."""
    if isinstance(value, torch.Tensor):
        return (value,)
    if isinstance(value, (tuple, list)):
        return tuple(t for t in value if isinstance(t, torch.Tensor))
    return ()


def _swapped(value, stand_ins):
    """`value` with every tensor that has a stand-in replaced by it."""
    if not stand_ins:
        return value
    if isinstance(value, torch.Tensor):
        return stand_ins.get(id(value), value)
    if isinstance(value, (tuple, list)):
        return type(value)(stand_ins.get(id(t), t) if isinstance(t, torch.Tensor) else t for t in value)
    return value


def _ends_in_plain_moe_branch(block) -> bool:
    """Whether the block's last op is ``x + moe(...)``: in a replay nothing reads that sum's
    values (the add's backward needs none), so the experts' combine can skip moving them."""
    from .layers.moe import MoE

    last = block.items[-1] if isinstance(block, Sequence) and len(block.items) else block
    if not isinstance(last, ResidualBranch) or getattr(last, "algebra", None) is not None:
        return False
    body = last.body
    tail = body.items[-1] if isinstance(body, Sequence) and len(body.items) else body
    return isinstance(tail, MoE)


def _checkpointed(block, x, ctx: Context, offload: bool = False, key=None, keep_attention: bool = False,
                  kept_to_host: bool = False):
    holder = _BlockRun(block, ctx, offload, key, keep_attention, kept_to_host)
    y, *rest = _Remat.apply(x, holder, *holder.outside())
    aux, pushed = rest[:len(holder.names)], rest[len(holder.names):]
    for name, value in zip(holder.names, aux):
        prev = ctx.losses.get(name)
        ctx.losses[name] = value if prev is None else prev + value
    # the taps hold the function's outputs (which carry its graph), not the tensors the run
    # under no_grad made
    raw = holder.pushed
    if pushed:
        as_output = {id(t): o for t, o in zip(raw, pushed)}
        for name, stack in ctx.taps.items():
            ctx.taps[name] = [_swapped(value, as_output) for value in stack]
    return y


def count_outer_branches(node: nn.Module) -> int:
    """Residual branches that are inside no other, in the order they run, up to the first head:
    what ``precision(first=..., last=...)`` counts."""
    from .layers.basic import Head

    total = 0

    def walk(m) -> bool:   # True once a head was reached
        nonlocal total
        if isinstance(m, Head):
            return True
        if isinstance(m, ResidualBranch):
            total += 1
            return False
        children = list(m.items) if isinstance(m, (Sequence, Repeated)) else list(m.children())
        for child in children:
            if walk(child):
                return True
        return False

    walk(node)
    return total


class GraphBuilder:
    def __init__(self, arch: ir.Architecture, dtype: torch.dtype):
        self.arch = arch
        self.dtype = dtype
        self.shared: dict = {}
        self.embedding = None
        self.layer_count = 0
        self.num_layers = sum(1 for _ in arch.layers())
        self.depth = 0      # residual branches around the node being built
        self.branches = 0   # top-level branches built so far: the algebra numbers them

    def build(self, node):
        if node.share is not None:
            if node.share not in self.shared:
                self.shared[node.share] = self._build(node)
            return self.shared[node.share]
        return self._build(node)

    def _build(self, node):
        if isinstance(node, ir.Layer):
            bctx = BuildContext(d_model=self.arch.d_model, vocab_size=self.arch.vocab_size,
                                residual=self.arch.residual, init=self.arch.init, width=node.width,
                                ports=node.ports, embedding=self.embedding, dtype=self.dtype,
                                layer_index=self.layer_count, num_layers=self.num_layers)
            self.layer_count += 1
            module = build_layer(node.config, bctx)
            if node.config.type == "embed" and self.embedding is None:
                self.embedding = module
            if node.ports:
                module.ports = node.ports
            return module
        if isinstance(node, ir.Seq):
            return Sequence([self.build(n) for n in node.items])
        if isinstance(node, ir.Residual):
            # only a branch outside any other goes through the residual algebra
            algebra = None
            if self.arch.residual is not None and self.depth == 0:
                from . import residual

                algebra = residual.build(self.arch.residual, self.arch.d_model, self.branches)
                for name in getattr(algebra, "no_weight_decay", ()):
                    if hasattr(algebra, name):
                        getattr(algebra, name).no_weight_decay = True
                self.branches += 1
            self.depth += 1
            try:
                body = self.build(node.body)
            finally:
                self.depth -= 1
            from . import observe

            return ResidualBranch(body, algebra, observe.branch_name(node))
        if isinstance(node, ir.Sum):
            return Parallel([self.build(n) for n in node.terms], product=False)
        if isinstance(node, ir.Prod):
            return Parallel([self.build(n) for n in node.factors], product=True)
        if isinstance(node, ir.Neg):
            return Negate(self.build(node.body))
        if isinstance(node, ir.Const):
            return Constant(node.value)
        if isinstance(node, ir.Identity):
            return Identity()
        if isinstance(node, ir.Repeat):
            if node.body.share is not None:
                body = self.build(node.body)
                return Repeated([body] * node.times)
            return Repeated([self.build(node.body) for _ in range(node.times)])
        if isinstance(node, ir.Tap):
            return TapWrite(node.name)
        if isinstance(node, ir.Ref):
            return TapRead(node.name, node.pop)
        raise AssertionError(node)
