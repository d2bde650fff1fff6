"""Context (sequence) parallelism of softmax attention over the ``context`` axis.

Every rank holds ``t / c`` consecutive positions of each row; everything per-position
(norms, MLPs, experts, the loss) runs on those alone. Attention is where positions
meet, by one of (``methods(attention=...)``; reference ``parallel/context.py:406-600``,
``parallel/ring.py:58-190``):

* ``ulysses``: all-to-all [b, t/c, h, d] → [b, t, h/c, d] around a whole-row kernel call
  and back (needs c | kv heads); 4 all-to-alls forward, 4 backward.
* ``gathered`` / ``ring``: K and V are all-gathered once; rank r's queries see the keys
  of chunks 0..r (the kernel's causal mask with more keys than queries), and the
  backward reduce-scatters dK, dV.
* ``auto``: ulysses when c divides the kv heads, else gathered.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


class _ToHeads(torch.autograd.Function):
    """[b, t/c, h, d] → [b, t, h/c, d]"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _to_heads(x, group)

    @staticmethod
    def backward(ctx, g):
        return _to_positions(g.contiguous(), ctx.group), None


class _ToPositions(torch.autograd.Function):
    """[b, t, h/c, d] → [b, t/c, h, d]"""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _to_positions(x, group)

    @staticmethod
    def backward(ctx, g):
        return _to_heads(g.contiguous(), ctx.group), None


def _to_heads(x, group):
    c = dist.get_world_size(group)
    b, tl, h, d = x.shape
    # send head-group j to rank j: [c, b, tl, h/c, d]
    send = x.reshape(b, tl, c, h // c, d).permute(2, 0, 1, 3, 4).contiguous()
    got = _a2a(send, group)
    # got[i] = rank i's positions of my heads → concatenate along t
    return got.permute(1, 0, 2, 3, 4).reshape(b, c * tl, h // c, d)


def _to_positions(x, group):
    c = dist.get_world_size(group)
    b, t, hl, d = x.shape
    send = x.reshape(b, c, t // c, hl, d).permute(1, 0, 2, 3, 4).contiguous()
    got = _a2a(send, group)
    # got[j] = my positions of head-group j → concatenate along heads
    return got.permute(1, 2, 0, 3, 4).reshape(b, t // c, c * hl, d)


class _GatherKV(torch.autograd.Function):
    """Local [b, t/c, g, d] → the first (r+1) chunks [b, (r+1)·t/c, g, d]; the backward
    sums every rank's gradient of this rank's chunk (reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        c, r = dist.get_world_size(group), dist.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(c)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.shape = x.shape
        return torch.cat(parts[: r + 1], dim=1)

    @staticmethod
    def backward(ctx, g):
        c, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        tl = ctx.shape[1]
        full = g.new_zeros(c, *ctx.shape)
        full[: r + 1] = g.reshape(g.shape[0], r + 1, tl, *g.shape[2:]).transpose(0, 1)
        if g.is_cuda:
            mine = torch.empty(ctx.shape, dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(mine, full, group=ctx.group)
        else:
            dist.all_reduce(full, group=ctx.group)
            mine = full[r]
        return mine.contiguous(), None


def method_for(name: str, kv_heads: int, heads: int, world: int) -> str:
    if name in ("auto", "cudnn", "fa4", "tokamax", "xla"):
        return "ulysses" if kv_heads % world == 0 and heads % world == 0 else "gathered"
    if name in ("ring", "gathered", "allgather"):
        return "gathered"
    if name == "ulysses":
        if kv_heads % world or heads % world:
            raise ValueError(f"ulysses needs the context size {world} to divide the heads ({heads}/{kv_heads})")
        return "ulysses"
    raise ValueError(f"methods(attention={name!r}) is not a context-parallel method")


def attend(attention, q, k, v, group, method: str, **kw):
    """`attention(q, k, v, **kw)` is the whole-row kernel call; this wraps it for rows
    split by position over `group`."""
    if kw.get("segments") is not None:
        raise NotImplementedError("context parallelism of packed rows (document masks) is not built yet")
    c = dist.get_world_size(group)
    how = method_for(method, k.shape[2], q.shape[2], c)
    if how == "ulysses":
        qh, kh, vh = (_ToHeads.apply(x.contiguous(), group) for x in (q, k, v))
        sinks = kw.get("sinks")
        if sinks is not None:  # this rank's heads
            r, per = dist.get_rank(group), q.shape[2] // c
            kw = dict(kw, sinks=sinks[r * per:(r + 1) * per])
        out = attention(qh, kh, vh, **kw)
        return _ToPositions.apply(out.contiguous(), group)
    kg, vg = _GatherKV.apply(k, group), _GatherKV.apply(v, group)
    return attention(q, kg, vg, **kw)
