"""DeepSeek sparse attention's lightning indexer (``gqa(indexer=indexer(...))``).

For every query it scores every key it may see, ``I[t,s] = Σ_j w_j ReLU(q_j·k_s)`` with
a few small heads, keeps the ``top_k`` best, and the layer's softmax runs over the kept
keys only. The indexer reads a detached copy of the layer's input and is trained only by
its own loss, ``KL(p || softmax(I))`` over the kept keys, where p is the layer's attention
summed over heads and normalised over them (DeepSeek-V3.2, eq. 4); that loss trains
nothing else. The kept keys travel between layers through the ``index`` port.

Variants (all here): ``per_group`` (MiniMax MSA: each indexer head picks for the query heads
that share one kv head, by its own unweighted scores); ``block_size > 1`` keeps whole blocks
of keys, counted from each document's first key: mean-pooled (Qwen3.8 QSA: a block's key is
the mean of its keys as projected, normalised, rotated to its first key's position; a query
picks among the blocks it sees all of and also keeps the keys of its own unfinished block;
the loss's target of a block is its most attended key's) or max-pooled (MSA: a block scores
the best of its keys the query sees, the query's own block is always among the
``top_k // block_size`` kept, the loss runs over the kept keys).

This is the dense statement (scores and attention as [t, s] matrices, the CPU oracle of a
future top-k + gather kernel). Reference: ``architecture/attention/indexer.py:262-790``,
``sparse.py``.
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


def block_ids(positions: torch.Tensor, size: int) -> torch.Tensor:
    """[b, s] which block of `size` keys each key is in, blocks counted from each document's
    first key (a document starts where the position is 0) and numbered along the row."""
    return (positions % size == 0).long().cumsum(-1) - 1


def per_block(values: torch.Tensor, block: torch.Tensor, blocks: int, how: str) -> torch.Tensor:
    """[b, t, (g,) s] → [b, t, (g,) blocks]: the sum or the maximum of each block's keys
    (-inf for the maximum of a block with none)."""
    index = block.view(block.shape[0], *([1] * (values.dim() - 2)), -1).expand_as(values)
    shape = (*values.shape[:-1], blocks)
    if how == "sum":
        return torch.zeros(shape, dtype=values.dtype, device=values.device).scatter_add(-1, index, values)
    out = torch.full(shape, float("-inf"), dtype=values.dtype, device=values.device)
    return out.scatter_reduce(-1, index, values, reduce="amax", include_self=True)


def kl_over(target: torch.Tensor, scores: torch.Tensor, over: torch.Tensor) -> torch.Tensor:
    """Every query's KL(p || softmax(scores)) over the entries `over` keeps, p = target normalised
    over them; 0 for a query with none."""
    p = target.masked_fill(~over, 0.0)
    p = p / p.sum(-1, keepdim=True).clamp_min(torch.finfo(p.dtype).tiny)
    log_q = torch.log_softmax(scores.float().masked_fill(~over, float("-inf")), -1)
    log_p = torch.log(torch.where(p > 0, p, torch.ones_like(p)))
    terms = torch.where(p > 0, p * (log_p - torch.where(over, log_q, torch.zeros_like(log_q))), torch.zeros_like(p))
    return terms.sum(-1)


class Picked:
    """What an indexer kept for a chunk of queries, and what its loss scores again."""

    def __init__(self, kept, scores, over, block=None, blocks=0):
        self.kept = kept        # [b, t, (g,) s] the keys attention runs over
        self.scores = scores    # [b, t, (g,) s] per key, or [b, t, blocks] per block (mean-pooled)
        self.over = over        # what the loss runs over, shaped like `scores`
        self.block, self.blocks = block, blocks   # [b, s] block of each key when the loss is per block


class Indexer(nn.Module):
    """`width`: the layer's input (the heads' weights come from it). `query_width`: what the
    queries are projected from (the input, or a query latent). `key_width`: what the keys are
    projected from; None when the keys come ready from another layer (through a ``kv`` port).
    `key_norm`: the keys' norm unless the config names one."""

    def __init__(self, c: L.SparseIndexerConfig, width: int, rope, rope_dims: int, b: BuildContext,
                 query_width: int = None, key_width="input", key_norm=None):
        super().__init__()
        self.c = c
        h, i = c.num_heads, c.head_dim
        self.q = Linear(query_width or width, h * i, False, b, role="q")
        if key_width is not None:
            self.k = Linear(width if key_width == "input" else key_width, i, False, b, role="q")
        if c.weighted:
            self.weights = Linear(width, h, False, b, role="router")
        if c.norm is not None:
            self.q_norm = Norm(c.norm, i)
        if key_width is not None:
            self.k_norm = Norm(c.norm or key_norm or L.NormalizationConfig(type="layernorm", bias=True), i)
        n = min(rope_dims, i) // 2 * 2
        if rope is not None and n:
            own = rope.model_copy(update={"fraction": 1.0, "layout": c.rope_layout})
            inv, gain = rope_lib.inverse_frequencies(own, n)
            self.register_buffer("inv_freq", inv, persistent=False)
            self.rope_gain, self.interleaved = gain, c.rope_layout == "interleaved"

    def _rotate(self, x, ctx: Context, positions=None):
        if not hasattr(self, "inv_freq"):
            return x
        cos, sin = rope_lib.tables(ctx.positions if positions is None else positions, self.inv_freq, self.rope_gain)
        return ref.rope(x, cos, sin, interleaved=self.interleaved)

    def keys_of(self, source, positions, ctx: Context) -> torch.Tensor:
        """The indexer's keys [b, s, head_dim] of `source` [b, s, key_width] (detached),
        normalised and rotated to `positions`."""
        k = self.k_norm(self.k(source.detach(), ctx), ctx)
        return self._rotate(k.unsqueeze(2), ctx, positions)[:, :, 0]

    def scores_of(self, x, query, keys, ctx: Context) -> torch.Tensor:
        """Scores [b, t, s] of ready keys [b, s, head_dim] for queries projected from `query`
        (the heads' weights from `x`); both detached."""
        q = self._queries(query.detach(), ctx)
        return self._combine(torch.einsum("bthi,bsi->bths", q.float(), keys.detach().float()), x.detach(), ctx)

    def _queries(self, x, ctx: Context):
        c = self.c
        bsz, t, _ = x.shape
        q = self.q(x, ctx).view(bsz, t, c.num_heads, c.head_dim)
        if hasattr(self, "q_norm"):
            q = self.q_norm(q, ctx)
        return self._rotate(q, ctx)

    def _combine(self, dots: torch.Tensor, x, ctx: Context) -> torch.Tensor:
        """[b, t, h, n] dot products → [b, t, n] (the heads weighed and summed), or
        [b, t, g, n] with ``per_group`` (each head is its group's score)."""
        c = self.c
        scale = c.head_dim ** -0.5
        if c.relu:
            dots = dots.relu()
        if c.per_group:
            return dots * scale
        if hasattr(self, "weights"):
            w = self.weights(x, ctx).float() * (scale * c.num_heads ** -0.5)
        else:
            w = torch.full(dots.shape[:3], scale, device=x.device)
        return torch.einsum("bthn,bth->btn", dots, w)

    def scores(self, x, ctx: Context) -> torch.Tensor:
        """Every key's score for every query, from a detached input: [b, t, s], or
        [b, t, g, s] with ``per_group``."""
        x = x.detach()
        q = self._queries(x, ctx)
        k = self._rotate(self.k_norm(self.k(x, ctx), ctx).unsqueeze(2), ctx)[:, :, 0]
        return self._combine(torch.einsum("bthi,bsi->bths", q.float(), k.float()), x, ctx)

    def block_scores(self, x, ctx: Context, block: torch.Tensor, blocks: int) -> torch.Tensor:
        """[b, t, blocks]: mean-pooled blocks. A block's key is the mean of its keys as
        projected, normalised, then rotated to the position of the block's first key."""
        c = self.c
        x = x.detach()
        q = self._queries(x, ctx)
        raw = self.k(x, ctx).float()                                          # [b, s, i]
        index = block.unsqueeze(-1).expand_as(raw)
        sums = torch.zeros(raw.shape[0], blocks, raw.shape[-1], device=raw.device).scatter_add(1, index, raw)
        keys = self.k_norm((sums / c.block_size).to(x.dtype), ctx)
        if hasattr(self, "inv_freq"):
            first = torch.zeros(block.shape[0], blocks, dtype=ctx.positions.dtype, device=block.device)
            starts = ctx.positions % c.block_size == 0
            first = first.scatter_add(1, block, torch.where(starts, ctx.positions, torch.zeros_like(ctx.positions)))
            cos, sin = rope_lib.tables(first, self.inv_freq, self.rope_gain)
            keys = ref.rope(keys.unsqueeze(2), cos, sin, interleaved=self.interleaved)[:, :, 0]
        return self._combine(torch.einsum("bthi,bni->bthn", q.float(), keys.float()), x, ctx)

    def pick(self, x, ctx: Context, seen: torch.Tensor, top_k: int = None) -> Picked:
        """The keys each query keeps of those it sees (`seen` [b, t, s]); `top_k` overrides the
        config's."""
        c = self.c
        top_k = c.top_k if top_k is None else top_k
        size = c.block_size
        if size == 1:
            scores = self.scores(x, ctx)
            mask = seen.unsqueeze(2).expand_as(scores) if c.per_group else seen
            kept = top_mask(scores, mask, top_k)
            return Picked(kept, scores, kept)
        block = block_ids(ctx.positions, size)
        blocks = int(block.max().item()) + 1
        member = torch.nn.functional.one_hot(block, blocks).bool()            # [b, s, blocks]
        newest = torch.where(seen, torch.arange(seen.shape[-1], device=seen.device), -1).amax(-1)   # [b, t]
        own = torch.where(newest >= 0, block.gather(1, newest.clamp_min(0)), -1)                     # [b, t]
        is_own = torch.arange(blocks, device=seen.device) == own.unsqueeze(-1)                       # [b, t, blocks]
        keep = max(top_k // size, 1)
        if c.pool == "mean":
            scores = self.block_scores(x, ctx, block, blocks)                                        # [b, t, blocks]
            whole = per_block(seen.float(), block, blocks, "sum") == size     # blocks the query sees all of
            picked = top_mask(scores, whole, keep)
            chosen = picked | is_own                                          # and its own unfinished block's keys
            kept = torch.einsum("btn,bsn->bts", chosen.float(), member.float()).bool() & seen
            return Picked(kept, scores, picked, block, blocks)
        scores = self.scores(x, ctx)                                          # per key; [b, t, (g,) s]
        mask = seen.unsqueeze(2).expand_as(scores) if c.per_group else seen
        best = per_block(scores.masked_fill(~mask, float("-inf")), block, blocks, "max")
        any_seen = best > float("-inf")
        own_b = is_own.unsqueeze(2).expand_as(best) if c.per_group else is_own
        # the query's own block always, then the best of the others
        ranked = torch.where(own_b, torch.full_like(best, float("inf")), best)
        chosen = top_mask(ranked, any_seen, keep)
        kept = torch.einsum("bt...n,bsn->bt...s", chosen.float(), member.float()).bool() & mask
        return Picked(kept, scores, kept)

    def loss(self, picked: Picked, target: torch.Tensor) -> torch.Tensor:
        """KL(p || softmax(I)) over what was kept, averaged over the queries (and the groups):
        p is the layer's attention (`target`, shaped like the kept mask); a mean-pooled
        block's p is its most attended key's."""
        if picked.block is not None:
            target = per_block(target, picked.block, picked.blocks, "max").clamp_min(0.0)
        return kl_over(target, picked.scores, picked.over).mean()


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
    """Softmax attention over the kept keys: (out [b,t,h,dv], p summed over heads, detached:
    [b,t,s], or [b,t,g,s] summed over each group's heads when `kept` is per group).
    q [b,t,h,d], k/v [b,s,g,d]; kept [b,t,s] or [b,t,g,s] bool."""
    bsz, t, h, d = q.shape
    g = k.shape[2]
    kk = k.repeat_interleave(h // g, dim=2)
    vv = v.repeat_interleave(h // g, dim=2)
    logits = torch.einsum("bthd,bshd->bhts", q.float(), kk.float()) * (scale if scale is not None else d ** -0.5)
    if softcap:
        logits = softcap * torch.tanh(logits / softcap)
    per_group = kept.dim() == 4
    heads_kept = kept.transpose(1, 2).repeat_interleave(h // g, dim=1) if per_group else kept[:, None]
    logits = logits.masked_fill(~heads_kept, float("-inf"))
    if sinks is not None:
        sink = sinks.float().view(1, h, 1, 1).expand(bsz, h, t, 1)
        probs = torch.softmax(torch.cat([logits, sink], -1), -1)[..., :-1]
    else:
        probs = torch.softmax(logits, -1)
    probs = torch.nan_to_num(probs)
    out = torch.einsum("bhts,bshd->bthd", probs, vv.float()).to(q.dtype)
    if per_group:
        return out, probs.view(bsz, g, h // g, t, -1).sum(2).transpose(1, 2).detach()
    return out, probs.sum(1).detach()


def indexer_loss(scores: torch.Tensor, kept: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """mean over queries of KL(p || softmax(I)) over the kept keys."""
    return kl_over(target, scores, kept).mean()


def candidate_pool(scores: torch.Tensor, seen: torch.Tensor, block: torch.Tensor, blocks: int, keep: int) -> torch.Tensor:
    """A coarse pool for a later layer's indexer (DeepSeek-V4.1): the `keep` blocks of keys whose
    best seen key scores highest for each query, as a mask over the keys [b, t, s]."""
    best = per_block(scores.float().masked_fill(~seen, float("-inf")), block, blocks, "max")
    chosen = top_mask(best, best > float("-inf"), keep)
    member = torch.nn.functional.one_hot(block, blocks)
    return torch.einsum("btn,bsn->bts", chosen.float(), member.float()).bool()
