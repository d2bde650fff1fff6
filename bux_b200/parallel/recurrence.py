"""Context parallelism of recurrent token mixers: each rank holds a stretch of positions and
needs the state the ranks before it leave behind.

The recurrence is affine in its state: over a rank's stretch, S_end = M S_start + B with a
transition M [dk, dk] and an offset B [dk, dv] that depend only on the stretch's own tokens,
and every output is o_t = o_t(from a zero state) + S_start^T r_t with r_t [dk] a read-out
vector of the stretch. All three come out of ONE local scan over values widened by dk zero
columns and started from the state [0 | I]: the recurrence acts on a state's columns
independently, so the widened state ends as [B | M] and the widened outputs are [o_t | r_t].
The (M, B) pairs are then all-gathered (dk x (dk + dv) numbers per head and rank), every
rank folds the pairs of the ranks before it into its own S_start, and adds S_start^T r_t to
its outputs. One scan per rank, one small collective, no serial hand-over between ranks
(the reference's ``pass_state``, ``parallel/recurrence.py:82-156`` there, after LASP-2).

Convolutions and token shifts only need the few positions before a rank's first one: `halo`.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class _AllGather(torch.autograd.Function):
    """x → stack of every rank's x ([world, ...]); the backward sums the ranks' gradients of
    this rank's slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def gathered(x: torch.Tensor, group) -> torch.Tensor:
    return _AllGather.apply(x, group)


def pass_state(scan, q, k, v, g, a, b, starts, group):
    """`scan(q, k, v, g, a, b, starts, state)` over rows whose positions are split over
    `group`, in order of rank. Returns (outputs of this rank's positions, this rank's last state)."""
    world, me = dist.get_world_size(group), dist.get_rank(group)
    bsz, t, h, dk = k.shape
    dv = v.shape[-1]
    wide_v = torch.cat([v.float(), torch.zeros(bsz, t, h, dk, device=v.device)], dim=-1)
    eye = torch.eye(dk, device=v.device).expand(bsz, h, dk, dk)
    start = torch.cat([torch.zeros(bsz, h, dk, dv, device=v.device), eye], dim=-1)
    wide_o, wide_s = scan(q, k, wide_v, g, a, b, starts, start)
    o_zero, readout = wide_o[..., :dv].float(), wide_o[..., dv:].float()      # [b, t, h, dv], [b, t, h, dk]
    offset, transition = wide_s[..., :dv], wide_s[..., dv:]                   # [b, h, dk, dv], [b, h, dk, dk]
    every = gathered(torch.cat([offset, transition], dim=-1), group)           # [world, b, h, dk, dv + dk]
    # every rank's graph must hold the gathered pairs, or the ranks would disagree on which
    # collectives the backward runs (the first rank reads none of them)
    state = torch.zeros(bsz, h, dk, dv, device=v.device) + every.sum() * 0.0
    for r in range(me):
        state = every[r, ..., dv:] @ state + every[r, ..., :dv]
    out = o_zero + torch.einsum("bthk,bhkv->bthv", readout, state)
    last = transition @ state + offset
    return out.to(v.dtype), last


def halo(x: torch.Tensor, width: int, group) -> torch.Tensor:
    """The last `width` positions of the rank before this one ([b, width, ...]; zeros on the
    first rank): what a causal convolution or a token shift reads before its first position."""
    me = dist.get_rank(group)
    tails = gathered(x[:, -width:].contiguous(), group)
    # the first rank takes a tail too (times zero): every rank's backward then runs the same collectives
    return tails[me - 1] * (0.0 if me == 0 else 1.0)
