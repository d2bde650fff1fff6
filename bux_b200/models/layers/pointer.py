"""The copy pointer of a head (CPLM): the next token's probability is the head's softmax
mixed with a pointer over the earlier tokens of the document,

    p(y) = p_lm(y) · (1 − a·(1 − a_sink)) + a · p_copy(y)

where a is the softmax's mass on the ``<copy>`` row (a row of the vocabulary that no token
is), p_lm the softmax over the other rows, p_copy(y) the attention of one pointer head on
the earlier positions of the document whose token is y, and a_sink its attention on a
learned sink. Everything is kept in log space and in fp32.

Reference: ``architecture/copy.py:52-436`` (`Pointer`, `mixture_nll`, `CopyPointer`).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ...config import layers as L
from ..registry import BuildContext, Context
from .basic import Linear

QUERY_CHUNK = 512
_NEG = float("-inf")


def logadd(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """log(eᵃ + eᵇ) whose gradient stays finite where one of them is −inf."""
    top = torch.maximum(a, b).detach()
    top = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    return top + torch.log(torch.exp(a - top) + torch.exp(b - top))


def masked_lse(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """logsumexp of the scores the mask keeps; −inf (with a zero gradient) where it keeps none."""
    some = mask.any(-1)
    top = scores.masked_fill(~mask, _NEG).amax(-1).detach()
    top = torch.where(some, top, torch.zeros_like(top))
    e = torch.where(mask, torch.exp(torch.where(mask, scores, top[..., None]) - top[..., None]),
                    torch.zeros_like(scores))
    total = e.sum(-1)
    return torch.where(some, top + torch.log(torch.where(some, total, torch.ones_like(total))),
                       torch.full_like(total, _NEG))


def rms_normed(x: torch.Tensor) -> torch.Tensor:
    y = x.float()
    return (y * torch.rsqrt(y.square().mean(-1, keepdim=True) + torch.finfo(torch.float32).eps)).to(x.dtype)


def mixture_nll(logits: torch.Tensor, targets: torch.Tensor, copy: int, log_copy: torch.Tensor,
                log_sink: torch.Tensor):
    """−log of the mixture's probability of each target, and the log of the softmax's
    normaliser (``<copy>`` in it). logits [n, vocab]; targets, log_copy, log_sink [n]."""
    lf = logits.float()
    target = lf.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    gate = lf[..., copy]
    left = torch.zeros_like(lf, dtype=torch.bool).scatter_(-1, targets.long().unsqueeze(-1), True)
    left[..., copy] = True
    others = masked_lse(lf, ~left)
    log_lm = -nn.functional.softplus(others - target)   # log p_lm(y): the softmax without <copy>
    lse_lm = logadd(target, others)
    lse = logadd(lse_lm, gate)
    log_gate = gate - lse
    kept = logadd(lse_lm - lse, log_gate + log_sink)     # log(1 − a + a·a_sink)
    return -logadd(log_lm + kept, log_gate + log_copy), lse


class PointerView:
    """What a head's pointer leaves for the loss at each position of the pass."""

    def __init__(self, query, key, sink, tokens, docs, copy: int, window: Optional[int]):
        self.query, self.key, self.sink = query, key, sink
        self.tokens, self.docs, self.copy, self.window = tokens, docs, copy, window

    def logs(self, targets: torch.Tensor):
        """(log p_copy of each position's target, −inf where no earlier position of its
        document within the window holds it; log a_sink). Scores q·k/√c in fp32, a chunk
        of queries at a time against every key of the row."""
        b, t, c = self.query.shape
        at = torch.arange(t, device=targets.device)
        out_copy, out_sink = [], []
        for start in range(0, t, QUERY_CHUNK):
            stop = min(t, start + QUERY_CHUNK)
            q = self.query[:, start:stop].float()
            scores = torch.einsum("bnc,btc->bnt", q, self.key.float()) * c ** -0.5
            behind = at[start:stop, None] - at[None, :]
            valid = behind > 0
            if self.window is not None:
                valid = valid & (behind <= self.window)
            valid = valid[None] & (self.docs[:, start:stop, None] == self.docs[:, None, :])
            match = valid & (targets[:, start:stop, None] == self.tokens[:, None, :])
            sink = self.sink[:, start:stop]
            every = logadd(masked_lse(scores, valid), sink)
            out_copy.append(masked_lse(scores, match) - every)
            out_sink.append(sink - every)
        return torch.cat(out_copy, 1), torch.cat(out_sink, 1)

    def sums(self, head, targets: torch.Tensor, mask: torch.Tensor, z_weight: float = 0.0,
             chunk: int = 8192):
        """(Σ over kept positions of the mixture's −log-likelihood (+ z·lse²), count):
        the head's logits a chunk of positions at a time."""
        log_copy, log_sink = self.logs(targets)
        h = head.hidden.reshape(-1, head.hidden.shape[-1])
        tg, mk = targets.reshape(-1), mask.reshape(-1).float()
        lc, ls = log_copy.reshape(-1), log_sink.reshape(-1)
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        for start in range(0, h.shape[0], chunk):
            sl = slice(start, start + chunk)
            logits = nn.functional.linear(h[sl], head.weight.to(h.dtype),
                                          None if head.bias is None else head.bias.to(h.dtype)).float()
            if head.softcap:
                logits = head.softcap * torch.tanh(logits / head.softcap)
            nll, lse = mixture_nll(logits, tg[sl], self.copy, lc[sl], ls[sl])
            if z_weight:
                nll = nll + z_weight * lse.square()
            total = total + (nll * mk[sl]).sum()
        return total, mk.sum()


class CopyPointer(nn.Module):
    """Query and key projections of the head's input, the query's gain and the sink's key."""

    def __init__(self, c: L.CopyPointerConfig, width: int, vocab: int, b: BuildContext):
        super().__init__()
        self.q = Linear(width, c.dim, False, b, role="head")
        self.k = Linear(width, c.dim, False, b, role="head")
        if b.init is None:  # LeCun uniform unless the model's init says otherwise
            bound = math.sqrt(3.0 / width)
            for lin in (self.q, self.k):
                nn.init.uniform_(lin.weight, -bound, bound)
        self.gain = nn.Parameter(torch.ones(()))
        self.sink = nn.Parameter(torch.randn(c.dim) * c.dim ** -0.5)
        self.copy = vocab - 1 if c.token is None else c.token
        if not 0 <= self.copy < vocab:
            raise ValueError(f"copy_pointer(token={self.copy}) is no row of {vocab}")
        self.window = c.window

    def forward(self, x, ctx: Context) -> PointerView:
        q = rms_normed(self.q(x, ctx)) * self.gain.to(x.dtype)
        k = rms_normed(self.k(x, ctx))
        sink = torch.einsum("btc,c->bt", q.float(), self.sink.float()) * q.shape[-1] ** -0.5
        docs = ctx.segments if getattr(ctx, "segments", None) is not None else torch.ones_like(ctx.input_ids)
        return PointerView(q, k, sink, ctx.input_ids, docs, self.copy, self.window)
