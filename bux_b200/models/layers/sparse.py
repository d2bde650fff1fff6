"""DeepSeek sparse attention's lightning indexer (``gqa(indexer=indexer(...))``).

For every query it scores every key it may see, ``I[t,s] = Σ_j w_j ReLU(q_j·k_s)`` with
a few small heads, keeps the ``top_k`` best, and the layer's softmax runs over the kept
keys only. The indexer reads a detached copy of the layer's input and is trained only by
its own loss, ``KL(p || softmax(I))`` over the kept keys, where p is the layer's attention
summed over heads and normalised over them (DeepSeek-V3.2, eq. 4); that loss trains
nothing else. The kept keys travel between layers through the ``index`` port.

This is the dense statement (scores and attention as [t, s] matrices, the CPU oracle of a
future top-k + gather kernel): single keys (``block_size=1``), one pick for all heads.
Reference: ``architecture/attention/indexer.py:269-620``, ``sparse.py``.
"""

from __future__ import annotations

import torch
from torch import nn

from ...config import layers as L
from ...ops import reference as ref
from ..registry import BuildContext, Context
from . import rope as rope_lib
from .basic import Linear, Norm


def top_mask(scores: torch.Tensor, seen: torch.Tensor, k: int) -> torch.Tensor:
    """The k highest scores of those `seen` in each row (the first of equal ones)."""
    k = min(k, scores.shape[-1])
    ranked = scores.float().masked_fill(~seen, float("-inf"))
    best = ranked.sort(dim=-1, descending=True, stable=True).indices[..., :k]
    return torch.zeros_like(seen).scatter(-1, best, True) & seen


class Indexer(nn.Module):
    def __init__(self, c: L.SparseIndexerConfig, width: int, rope, rope_dims: int, b: BuildContext):
        super().__init__()
        if c.block_size != 1 or c.per_group:
            raise NotImplementedError("indexer: blocks of keys and per-group picks are not built yet")
        self.c = c
        h, i = c.num_heads, c.head_dim
        self.q = Linear(width, h * i, False, b, role="q")
        self.k = Linear(width, i, False, b, role="q")
        if c.weighted:
            self.weights = Linear(width, h, False, b, role="router")
        if c.norm is not None:
            self.q_norm = Norm(c.norm, i)
        self.k_norm = Norm(c.norm or L.NormalizationConfig(type="layernorm", bias=True), i)
        n = min(rope_dims, i) // 2 * 2
        if rope is not None and n:
            own = rope.model_copy(update={"fraction": 1.0, "layout": c.rope_layout})
            inv, gain = rope_lib.inverse_frequencies(own, n)
            self.register_buffer("inv_freq", inv, persistent=False)
            self.rope_gain, self.interleaved = gain, c.rope_layout == "interleaved"

    def _rotate(self, x, ctx: Context):
        if not hasattr(self, "inv_freq"):
            return x
        cos, sin = rope_lib.tables(ctx.positions, self.inv_freq, self.rope_gain)
        return ref.rope(x, cos, sin, interleaved=self.interleaved)

    def scores(self, x, ctx: Context) -> torch.Tensor:
        """[b, t, s] from a detached input."""
        c = self.c
        x = x.detach()
        bsz, t, _ = x.shape
        q = self.q(x, ctx).view(bsz, t, c.num_heads, c.head_dim)
        if hasattr(self, "q_norm"):
            q = self.q_norm(q, ctx)
        q = self._rotate(q, ctx)
        k = self._rotate(self.k_norm(self.k(x, ctx), ctx).unsqueeze(2), ctx)[:, :, 0]
        scale = c.head_dim ** -0.5
        if hasattr(self, "weights"):
            w = self.weights(x, ctx).float() * (scale * c.num_heads ** -0.5)
        else:
            w = torch.full((bsz, t, c.num_heads), scale, device=x.device)
        dots = torch.einsum("bthi,bsi->bths", q.float(), k.float())
        if c.relu:
            dots = dots.relu()
        return torch.einsum("bths,bth->bts", dots, w)


def seen_mask(ctx: Context, t: int, window) -> torch.Tensor:
    """[b, t, s]: causal, inside the query's document, inside the window."""
    pos = torch.arange(t, device=ctx.positions.device)
    seen = (pos[None, :, None] >= pos[None, None, :]).expand(ctx.positions.shape[0], t, t)
    if window:
        seen = seen & (pos[None, :, None] - pos[None, None, :] < window)
    if getattr(ctx, "segments", None) is not None:
        seen = seen & (ctx.segments[:, :, None] == ctx.segments[:, None, :])
    return seen


def attend_kept(q, k, v, kept, scale, sinks=None, softcap=None):
    """Softmax attention over the kept keys: (out [b,t,h,dv], p summed over heads [b,t,s],
    detached). q [b,t,h,d], k/v [b,s,g,d]; kept [b,t,s] bool."""
    bsz, t, h, d = q.shape
    g = k.shape[2]
    kk = k.repeat_interleave(h // g, dim=2)
    vv = v.repeat_interleave(h // g, dim=2)
    logits = torch.einsum("bthd,bshd->bhts", q.float(), kk.float()) * (scale if scale is not None else d ** -0.5)
    if softcap:
        logits = softcap * torch.tanh(logits / softcap)
    logits = logits.masked_fill(~kept[:, None], float("-inf"))
    if sinks is not None:
        sink = sinks.float().view(1, h, 1, 1).expand(bsz, h, t, 1)
        probs = torch.softmax(torch.cat([logits, sink], -1), -1)[..., :-1]
    else:
        probs = torch.softmax(logits, -1)
    probs = torch.nan_to_num(probs)
    out = torch.einsum("bhts,bshd->bthd", probs, vv.float()).to(q.dtype)
    return out, probs.sum(1).detach()


def indexer_loss(scores: torch.Tensor, kept: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """mean over queries of KL(p || softmax(I)) over the kept keys."""
    p = target.masked_fill(~kept, 0.0)
    p = p / p.sum(-1, keepdim=True).clamp_min(torch.finfo(p.dtype).tiny)
    log_q = torch.log_softmax(scores.float().masked_fill(~kept, float("-inf")), -1)
    log_p = torch.log(torch.where(p > 0, p, torch.ones_like(p)))
    terms = torch.where(p > 0, p * (log_p - torch.where(kept, log_q, torch.zeros_like(log_q))), torch.zeros_like(p))
    return terms.sum(-1).mean()
