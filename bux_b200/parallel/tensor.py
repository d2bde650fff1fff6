"""Tensor parallelism over the ``tensor`` axis (Megatron column / row splits).

Each attention, MLP and MoE layer keeps a 1/n slice of its heads or hidden units:
the first projection (q/k/v, gate/up, the experts' gate/up) is split by output rows
(whole heads, whole hidden units), the last (o, down) by input columns, so the layer's
output is a partial sum that ONE all-reduce per layer completes. The two collectives
of a layer are autograd functions placed by hooks around the module: `_Copy` at its
input (identity forward, all-reduce of the input gradient in the backward) and
`_Reduce` at its output (all-reduce forward, identity backward). Reference:
``parallel/tensor.py:92-114`` (the GSPMD method places the same two collectives),
``architecture/common/sharding.py:56-74``.

Parameters that stay whole but see only the local heads (per-head q/k norms) get a
partial gradient; `partial` lists them and the engine sums them over the axis.
``layout(stream=tensor)`` (sequence parallelism) additionally keeps the residual stream
split by position between the layers: the input hook becomes an all-gather along the
sequence and the output hook a reduce-scatter.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _reduce_scatter_seq(x: torch.Tensor, group) -> torch.Tensor:
    n, r = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    if x.is_cuda:
        parts = x.transpose(0, 1).contiguous()  # [t, b, d]: this rank's positions are contiguous
        out = torch.empty(parts.shape[0] // n, *parts.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, parts, group=group)
        return out.transpose(0, 1).contiguous()
    dist.all_reduce(x, group=group)
    per = x.shape[1] // n
    return x[:, r * per:(r + 1) * per].contiguous()


def _all_gather_seq(x: torch.Tensor, group) -> torch.Tensor:
    n = dist.get_world_size(group)
    parts = x.transpose(0, 1).contiguous()
    out = torch.empty(n * parts.shape[0], *parts.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, parts, group=group)
    return out.transpose(0, 1).contiguous()


class _GatherSeq(torch.autograd.Function):
    """[b, t/n, d] → [b, t, d]; backward reduce-scatters (the layer after it is split by
    heads, so every rank holds a partial gradient for every position)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_seq(g, ctx.group), None


class _ScatterSeq(torch.autograd.Function):
    """partial [b, t, d] → summed [b, t/n, d]; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_seq(g, ctx.group), None


class _SliceSeq(torch.autograd.Function):
    """whole, identical on every rank → this rank's positions; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = dist.get_world_size(group), dist.get_rank(group)
        per = x.shape[1] // n
        return x[:, r * per:(r + 1) * per].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_seq(g.contiguous(), ctx.group), None


class _WholeSeq(torch.autograd.Function):
    """this rank's positions → whole sequence for a replicated tail (final norm, head);
    every rank then computes the same gradient, of which it keeps its own positions."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        per = g.shape[1] // n
        return g[:, r * per:(r + 1) * per].contiguous(), None


def split(module: nn.Module, name: str, dim: int, pieces: list, r: int, n: int, layout: dict):
    """Keep this rank's 1/n of every consecutive group of `pieces` along `dim`."""
    old = module._parameters.get(name)
    if old is None:
        return None
    parts, off = [], 0
    for size in pieces:
        per = size // n
        parts.append(old.data.narrow(dim, off + r * per, per))
        off += size
    new = nn.Parameter(torch.cat(parts, dim=dim).contiguous(), requires_grad=old.requires_grad)
    for k, v in old.__dict__.items():   # what the optimizer reads off a parameter (no_weight_decay, no_muon)
        setattr(new, k, v)
    module._parameters[name] = new
    layout[id(new)] = (dim, list(pieces))
    return new


def shard_of(whole_tensor: torch.Tensor, dim: int, pieces: list, r: int, n: int) -> torch.Tensor:
    """What `split` keeps of a whole tensor on rank r of n (the inverse of `whole`)."""
    parts, off = [], 0
    for size in pieces:
        per = size // n
        parts.append(whole_tensor.narrow(dim, off + r * per, per))
        off += size
    return torch.cat(parts, dim=dim).contiguous()


def whole(shard: torch.Tensor, dim: int, pieces: list, group) -> torch.Tensor:
    """Inverse of `split` (every rank of the group calls it): the whole tensor."""
    n = dist.get_world_size(group)
    got = [torch.empty_like(shard) for _ in range(n)]
    dist.all_gather(got, shard.contiguous(), group=group)
    out, off = [], 0
    for size in pieces:
        per = size // n
        out.extend(g.narrow(dim, off, per) for g in got)
        off += per
    return torch.cat(out, dim=dim)


def _need(cond: bool, what: str) -> None:
    if not cond:
        raise ValueError(f"tensor parallelism: {what}")


def shard_model(model: nn.Module, par) -> None:
    from ..models.layers.attention import GQA
    from ..models.layers.basic import MLP
    from ..models.layers.moe import MoE

    group = par.tensor_group
    n, r = dist.get_world_size(group), dist.get_rank(group)
    sequence = "tensor" in _axes(par.train.layout.stream)
    # the collectives run inside the GEMM kernels (NVLink peers, bf16, sequence-parallel stream)
    fused = (par.train.methods.tensor == "fused" and sequence and par.device.type == "cuda")
    if fused:
        from .. import runtime

        if not runtime.on_one_node(par.tensor_group):   # peer-memory kernels: one machine only
            import warnings

            warnings.warn("methods(tensor=fused): the tensor axis spans machines; taking the NCCL collectives")
            fused = False
    par.tensor_partial = []
    layout: dict = {}
    done: set = set()

    def mlp(m):
        f = m.c.intermediate_size
        _need(f % n == 0, f"hidden size {f} does not divide by tensor={n}")
        first = m.gate_up if m.gated else m.up
        pieces = [f, f] if m.gated else [f]
        split(first, "weight", 0, pieces, r, n, layout)
        split(first, "bias", 0, pieces, r, n, layout)
        split(m.down, "weight", 1, [f], r, n, layout)
        if m.down.bias is not None and r != 0:
            m.down.bias = None  # the bias joins the partial sums once: the first rank adds it
        m.f_local = f // n

    for m in model.modules():
        if isinstance(m, GQA):
            _need(m.h % n == 0 and m.g % n == 0, f"{m.h} heads / {m.g} kv heads do not divide by tensor={n}")
            _need(not (m.c.qk_norm is not None and m.c.qk_norm_all_heads), "qk_norm over all heads is not split")
            extras = [name for name in ("lambda_proj", "xsa_alpha", "k_conv", "rel_proj", "gate_up", "gate_bias",
                                        "output_gate_down", "cross_gate", "ve_gate", "v_norm") if hasattr(m, name)]
            _need(not extras, f"gqa with {', '.join(extras)} is not split over tensor ranks yet")
            _need(not m.c.paired, "gqa(paired=true) is not split over tensor ranks yet")
            pieces = [m.q_rows, m.k_rows, m.v_rows]
            split(m.qkv, "weight", 0, pieces, r, n, layout)
            split(m.qkv, "bias", 0, pieces, r, n, layout)
            split(m.o, "weight", 1, [m.h * m.dv], r, n, layout)
            if m.o.bias is not None and r != 0:
                m.o.bias = None
            if hasattr(m, "gate"):
                split(m.gate, "weight", 0, [m.gate.weight.shape[0]], r, n, layout)
                split(m.gate, "bias", 0, [m.gate.weight.shape[0] * n], r, n, layout)
            split(m, "sinks", 0, [m.h], r, n, layout)
            m.h, m.g, m.hq = m.h // n, m.g // n, m.hq // n
            m.q_rows, m.k_rows, m.v_rows = m.q_rows // n, m.k_rows // n, m.v_rows // n
            for name in ("q_norm", "k_norm", "out_norm"):
                if hasattr(m, name):
                    par.tensor_partial.extend(getattr(m, name).parameters())
            if fused and not hasattr(m, "gate") and m.qkv.bias is None and m.o.bias is None:
                m.qkv.tp_fused, m.o.tp_fused = ("gather", group, True), ("scatter", group, True)
            else:
                _hook(m, group, sequence)
            done.add(id(m))
        elif isinstance(m, MoE):
            f = m.f
            _need(f % n == 0, f"experts' hidden size {f} does not divide by tensor={n}")
            split(m, "experts_gate_up", 1, [f, f], r, n, layout)
            split(m, "experts_down", 2, [f], r, n, layout)
            m.f = f // n
            m.tp_share = 1.0 / n
            if hasattr(m, "shared"):
                mlp(m.shared)
                done.add(id(m.shared))
            # the picks are weighted before the all-reduce, so the router's gradient (through
            # the weights) is a partial sum like the outputs
            par.tensor_partial.extend(m.router.parameters())
            if hasattr(m, "shared_gate"):
                par.tensor_partial.extend(m.shared_gate.parameters())
            _hook(m, group, sequence)
            done.add(id(m))
    for m in model.modules():
        if isinstance(m, MLP) and id(m) not in done:
            mlp(m)
            first = m.gate_up if m.gated else m.up
            if fused and first.bias is None and m.down.bias is None and m.c.up_softcap is None:
                # rows stay in the kernels' (rank, batch, position) order between the two GEMMs
                first.tp_fused, m.down.tp_fused = ("gather", group, False), ("scatter", group, False)
            else:
                _hook(m, group, sequence)
            done.add(id(m))
    par.tensor_inside = {id(p) for m in model.modules() if id(m) in done for p in m.parameters()}
    par.tensor_layout = {name: layout[id(p)] for name, p in model.named_parameters() if id(p) in layout}
    par.tensor_sharded = set(layout)
    if sequence:
        _sequence_hooks(model, par, group)


def gather_tree(tree: dict, par) -> dict:
    """Whole leaves from tensor-parallel shards, for the rank that writes a checkpoint."""
    for part in tree.values():
        for key in list(part):
            name = key.split("/", 1)[1] if "/" in key else key
            lay = par.tensor_layout.get(name)
            t = part[key]
            if lay is None or not isinstance(t, torch.Tensor) or t.dim() <= lay[0]:
                continue
            part[key] = whole(t, lay[0], lay[1], par.tensor_group)
    return tree


def _axes(value) -> tuple:
    if value is None:
        return ()
    return (value,) if isinstance(value, str) else tuple(value)


def _hook(module: nn.Module, group, sequence: bool) -> None:
    enter = _GatherSeq if sequence else _Copy
    leave = _ScatterSeq if sequence else _Reduce

    def pre(mod, args):
        return (enter.apply(args[0], group), *args[1:])

    def post(mod, args, out):
        return leave.apply(out, group)

    module.register_forward_pre_hook(pre)
    module.register_forward_hook(post)


def _sequence_hooks(model: nn.Module, par, group) -> None:
    """Sequence parallelism: the stream is split by position after the embedding and whole
    again before the tail (final norm and head run replicated). Whole parameters between
    the two see only this rank's positions, so their gradients are partial."""
    from ..models.layers.basic import Embedding
    from ..models.graph import Repeated

    for m in model.modules():
        if isinstance(m, Embedding):
            # `_SliceSeq` gathers the gradient of every position: the table's gradient is whole
            m.register_forward_hook(lambda mod, args, out: _SliceSeq.apply(out, group))
        elif isinstance(m, Repeated):
            m.register_forward_hook(lambda mod, args, out: _WholeSeq.apply(out, group))
            for p in m.parameters():
                if id(p) not in par.tensor_inside and not any(p is q for q in par.tensor_partial):
                    par.tensor_partial.append(p)
