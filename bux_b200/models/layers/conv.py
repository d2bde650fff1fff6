"""Causal depthwise convolutions over the tokens: the ``conv`` and ``short_conv`` layers
and the short convs inside the recurrent mixers (reference: ``architecture/layers/conv.py``,
``architecture/recurrent/ssm.py:324``).

Weights are [channels, taps]; tap j multiplies the token j positions back. Taps that
would reach across a document start are dropped (packed rows).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ..registry import BuildContext, Context, register
from .basic import Linear


class CausalDepthwise(nn.Module):
    """y[t] = sum_j w[:, j] x[t-j] (+ bias)."""

    def __init__(self, d: int, taps: int, zero: bool = False, bias: bool = False):
        super().__init__()
        w = torch.zeros(d, taps) if zero else torch.empty(d, taps).uniform_(-1, 1) / math.sqrt(taps)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(d)) if bias else None

    def forward(self, x, ctx: Optional[Context] = None):
        t = x.shape[1]
        pos = None
        if ctx is not None and getattr(ctx, "segments", None) is not None:
            pos = ctx.positions
        w = self.weight.to(x.dtype)
        taps = w.shape[1]
        cache = getattr(ctx, "cache", None) if ctx is not None else None
        if cache is not None and taps > 1:
            return self._continued(x, ctx, cache, pos)
        y = x * w[:, 0]
        cp = getattr(ctx.parallel, "context_group", None) if ctx is not None and getattr(ctx, "parallel", None) else None
        if cp is None or taps == 1:
            from ... import ops

            return ops.causal_conv(x, self.weight, self.bias, pos)   # the kernel on a GPU, the same sum elsewhere
        before = None
        if cp is not None and taps > 1:
            # positions split over ranks: the taps before this rank's first position read the
            # last positions of the rank before it
            from ...parallel import recurrence

            before = recurrence.halo(x, min(taps - 1, t), cp)
        for j in range(1, min(taps, t + (before.shape[1] if before is not None else 0))):
            if before is not None:
                joined = torch.cat([before, x], dim=1)
                shifted = joined[:, before.shape[1] - j: before.shape[1] - j + t]
            else:
                shifted = nn.functional.pad(x[:, : t - j], (0, 0, j, 0))
            if pos is not None:
                shifted = shifted * (pos >= j).unsqueeze(-1).to(x.dtype)
            y = y + shifted * w[:, j]
        return y if self.bias is None else y + self.bias.to(y.dtype)


    def _continued(self, x, ctx, cache, pos):
        """Incremental decoding: the taps reach back into the inputs of earlier calls, which the
        cache holds (the last ``taps - 1`` of them; padding and what lies before a row's first
        token count as zeros)."""
        from ... import ops

        t, keep = x.shape[1], self.weight.shape[1] - 1
        tail = cache.tails.get(id(self))
        real = cache.new_real.unsqueeze(-1).to(x.dtype)
        if tail is None:       # the prompt: the usual sum (taps that would cross a row's start are dropped)
            y = ops.causal_conv(x, self.weight, self.bias, pos)
            joined = nn.functional.pad(x * real, (0, 0, keep, 0))
        else:
            joined = torch.cat([tail, x * real], dim=1)
            y = ops.causal_conv(joined, self.weight, self.bias, None)[:, -t:]
        cache.tails[id(self)] = joined[:, -keep:]
        return y


class Conv(nn.Module):
    """``conv``: a causal depthwise conv of the stream."""

    def __init__(self, c, b: BuildContext):
        super().__init__()
        width = b.width if isinstance(b.width, int) else b.d_model
        self.conv = CausalDepthwise(width, c.size, bias=c.bias)

    def forward(self, x, ctx: Context):
        return self.conv(x, ctx)


class ShortConv(nn.Module):
    """``short_conv`` (LFM2): B, C, u from the input; C * conv(B * u), projected back."""

    def __init__(self, c, b: BuildContext):
        super().__init__()
        width = b.width if isinstance(b.width, int) else b.d_model
        self.in_proj = Linear(width, 3 * width, c.bias, b)
        self.conv = CausalDepthwise(width, c.conv_size, bias=c.bias)
        self.out_proj = Linear(width, width, c.bias, b, init_role="out")

    def forward(self, x, ctx: Context):
        bb, cc, u = self.in_proj(x, ctx).chunk(3, -1)
        return self.out_proj(cc * self.conv(bb * u, ctx), ctx)


@register("conv")
def _conv(c, b):
    return Conv(c, b)


@register("short_conv")
def _short_conv(c, b):
    return ShortConv(c, b)
