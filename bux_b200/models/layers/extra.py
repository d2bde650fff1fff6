"""Less common layers: multi-head latent attention (``mla``), value embeddings
(``value_embed``), multi-token prediction's input (``nextn``), n-gram hash memory
(``engram``) and the document-local copy feature (``doc_copy``).

Reference: ``architecture/attention/mla.py``, ``architecture/layers/embedding.py:123,251``,
``architecture/layers/engram.py``, ``architecture/layers/doc_copy.py``.
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...config import layers as L
from ...ops import reference as ref
from ..registry import BuildContext, Context, register
from . import rope as rope_lib
from .basic import Linear, Norm, init_weight
from .conv import CausalDepthwise


# ------------------------------------------------------------------ MLA
class MLA(nn.Module):
    """Every head's keys and values are projected up from one normalised latent per token,
    its queries from another (or from the input at full rank), plus `qk_rope_head_dim`
    key dims shared by all heads, the only ones rotated. The softmax runs on the
    attention kernel when the head dims allow (q/k of n+r dims, v padded to them)."""

    def __init__(self, c: L.MLAConfig, b: BuildContext):
        super().__init__()
        self.c = c
        width = b.width if isinstance(b.width, int) else b.d_model
        h, n, r, dv = c.num_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
        self.ports = tuple(b.ports or ())
        if c.indexer is not None and not any(p.name == "index" and p.mode != "write" for p in self.ports):
            from .sparse import Indexer

            # DeepSeek sparse attention on MLA: a lightning indexer of its own picks the keys,
            # unless the layer reads another layer's picks through the `index` port
            self.indexer = Indexer(c.indexer, width, c.rope, r, b)
        self.h, self.n, self.r, self.dv, self.rank = h, n, r, dv, c.kv_lora_rank
        latent = c.q_lora_rank
        rms = L.NormalizationConfig(type="rmsnorm")
        if latent:
            self.q_a = Linear(width, latent, False, b, role="q")
            self.q_a_norm = Norm(rms, latent)
        self.q = Linear(latent or width, h * (n + r), False, b, role="q")
        self.kv_a = Linear(width, self.rank + r, False, b, role="q")
        self.kv_a_norm = Norm(rms, self.rank)
        self.kv_b = Linear(self.rank, h * (n + dv), False, b, role="q")
        self.o = Linear(h * dv, width, False, b, role="o", init_role="out")
        if c.qk_norm is not None:
            self.q_norm, self.k_norm = Norm(c.qk_norm, n + r), Norm(c.qk_norm, n + r)
        if c.rope is not None:
            inv, gain = rope_lib.inverse_frequencies(c.rope, r)
            self.register_buffer("inv_freq", inv, persistent=False)
            self.rope_gain = gain

    def _rotate(self, x, ctx: Context):
        if self.c.rope is None:
            return x
        cos, sin = rope_lib.tables(ctx.positions, self.inv_freq, self.rope_gain)
        rot = ref.rope(x[..., self.n:], cos, sin, interleaved=self.c.rope.layout == "interleaved")
        return torch.cat([x[..., : self.n], rot], -1)

    def forward(self, x, ctx: Context):
        c = self.c
        bsz, t, _ = x.shape
        h, n, r, dv = self.h, self.n, self.r, self.dv
        query = self.q_a_norm(self.q_a(x, ctx), ctx) if hasattr(self, "q_a") else x
        q = self.q(query, ctx).view(bsz, t, h, n + r)
        kv_latent, k_rope = self.kv_a(x, ctx).split([self.rank, r], -1)
        kv = self.kv_b(self.kv_a_norm(kv_latent, ctx), ctx).view(bsz, t, h, n + dv)
        k_nope, v = kv.split([n, dv], -1)
        k = torch.cat([k_nope, k_rope.unsqueeze(2).expand(bsz, t, h, r)], -1)
        if hasattr(self, "q_norm"):
            q, k = self.q_norm(q, ctx), self.k_norm(k, ctx)
        q, k = self._rotate(q, ctx), self._rotate(k, ctx)
        scale = c.scale if c.scale is not None else (n + r) ** -0.5
        if c.indexer is not None:
            out = self._sparse(x, q, k, v, scale, ctx)
        elif getattr(ctx, "cache", None) is not None:
            # incremental decoding: the expanded keys and values join the layer's cache (the plain
            # statement; a serving stack caches the latent and absorbs the expansion instead)
            k_all, v_all = ctx.cache.extend(self, k, v)
            out, _ = ref.attention(q, k_all, v_all, causal=True, window=c.sliding_window_size, sinks=None,
                                   softcap=c.softcap, scale=scale, segments=ctx.cache.segments())
        else:
            out = ops.attention(q, k, v, causal=True, window=c.sliding_window_size, sinks=None,
                                softcap=c.softcap, scale=scale, segments=ctx.segments)
        return self.o(out.reshape(bsz, t, h * dv), ctx)

    def _sparse(self, x, q, k, v, scale, ctx: Context):
        """Attention over the keys the indexer kept (its own, or another layer's through the
        ``index`` port), and the indexer's distillation loss: the dense statement, as `gqa`'s."""
        from . import sparse as S

        c = self.c
        t = q.shape[1]
        seen = S.seen_mask(ctx, t, c.sliding_window_size)
        reads = [p for p in self.ports if p.name == "index" and p.mode != "write"]
        picked = None
        if reads:
            kept = ctx.read(reads[0].tap, reads[0].mode == "pop")
            kept = kept & (seen.unsqueeze(2) if kept.dim() == 4 else seen)
        else:
            picked = self.indexer.pick(x, ctx, seen, c.indexer.top_k)
            kept = picked.kept
        for p in self.ports:
            if p.name == "index" and p.mode == "write":
                ctx.push(p.tap, kept)
        out, target = S.attend_kept(q, k, v, kept, scale, None, c.softcap)
        if picked is not None and ctx.training and c.indexer.loss_weight:
            ctx.report("indexer_loss", self.indexer.loss(picked, target), c.indexer.loss_weight)
        return out


@register("mla")
def _mla(c, b):
    return MLA(c, b)


# ------------------------------------------------------------------ value embeddings
class ValueEmbedding(nn.Module):
    """A row per token, pushed to the ``ve`` port for an attention layer to add to its
    values; the stream goes on as it is."""
    no_muon = True


    def __init__(self, c: L.ValueEmbeddingConfig, b: BuildContext):
        super().__init__()
        self.table = nn.Parameter(torch.randn(b.vocab_size, c.features, dtype=b.dtype) * c.std)
        self.ports = b.ports or ()

    def forward(self, x, ctx: Context):
        rows = self.table[ctx.input_ids]
        for p in self.ports:
            if p.mode == "write":
                ctx.push(p.tap, rows)
        return x


@register("value_embed")
def _value_embed(c, b):
    return ValueEmbedding(c, b)


# ------------------------------------------------------------------ nextn
class NextN(nn.Module):
    """The stream mixed with the embedding of the token k positions ahead, W [norm(e);
    norm(h)], for the k-th nextn of the pass; the last k positions embed token 0."""

    def __init__(self, c: L.NextNConfig, b: BuildContext):
        super().__init__()
        from ..residual import widening

        d = b.d_model
        copies = widening(b.residual)
        self.streams = b.width == "streams"
        if self.streams:
            self.hidden_norm = Norm(c.norm, copies * d)
            width = d
            self.copies = None
        else:
            width = b.width if isinstance(b.width, int) else d
            self.hidden_norm = Norm(c.norm, width)
            self.copies = copies
        self.embed_norm = Norm(c.norm, d)
        self.proj = Linear(d + width, width, False, b)
        object.__setattr__(self, "embedding", b.embedding)
        if b.embedding is None:
            raise ValueError("nextn needs an embedding before it")

    def forward(self, x, ctx: Context):
        ctx.nextn_runs = getattr(ctx, "nextn_runs", 0) + 1
        k, tokens = ctx.nextn_runs, ctx.input_ids
        ahead = F.pad(tokens[:, k:], (0, min(k, tokens.shape[1])))
        e = self.embedding.embed_tokens(ahead, ctx).to(x.dtype)   # scaled and normalised as the embedding's rows are
        e = self.embed_norm(e, ctx)
        if x.dim() == 4:
            hdn = self.hidden_norm(x.reshape(*x.shape[:2], -1), ctx).reshape(x.shape)
            e = e.unsqueeze(2).expand(x.shape)
        else:
            hdn = self.hidden_norm(x, ctx)
        y = self.proj(torch.cat([e, hdn], -1), ctx)
        if self.copies is not None and y.dim() == 3:
            y = y.unsqueeze(2).expand(-1, -1, self.copies, -1).contiguous()
        return y


@register("nextn")
def _nextn(c, b):
    return NextN(c, b)


# ------------------------------------------------------------------ engram
def _is_prime(n: int) -> bool:
    if n < 2:
        return False
    if n % 2 == 0:
        return n == 2
    i = 3
    while i * i <= n:
        if n % i == 0:
            return False
        i += 2
    return True


def next_primes(start: int, count: int, taken: set) -> list:
    """The `count` smallest primes >= start not taken yet; takes them."""
    out, n = [], max(2, start)
    while len(out) < count:
        if n not in taken and _is_prime(n):
            out.append(n)
            taken.add(n)
        n += 1
    return out


_ENGRAMS: dict = {}  # per-model bookkeeping: id(embedding) → (taken primes, engrams built)


class Engram(nn.Module):
    """Every n-gram of 2..max_ngram_size tokens ending at a position is hashed by
    `num_heads` heads into tables of distinct prime sizes; with e the looked-up rows,
    a = <norm(x), norm(W_k e)>/sqrt(d), it adds u = sigmoid(sign(a) sqrt|a|) W_v e and,
    with a conv, silu(conv(norm(u)))."""
    no_weight_decay = ("table",)


    def __init__(self, c: L.EngramConfig, b: BuildContext):
        super().__init__()
        self.c = c
        d, n, heads = b.d_model, c.max_ngram_size, c.num_heads
        key = id(b.embedding)
        taken, built = _ENGRAMS.setdefault(key, (set(), [0]))
        primes = next_primes(c.table_size, (n - 1) * heads, taken)
        built[0] += 1
        odd = np.random.default_rng(10007 * built[0]).integers(0, 2 ** 31, n)
        self.register_buffer("multipliers", torch.tensor(odd * 2 + 1, dtype=torch.int64), persistent=False)
        self.register_buffer("primes", torch.tensor(primes, dtype=torch.int64).view(n - 1, heads), persistent=False)
        offs = np.concatenate([[0], np.cumsum(primes[:-1])])
        self.register_buffer("offsets", torch.tensor(offs, dtype=torch.int64).view(n - 1, heads), persistent=False)
        self.streams = b.width == "streams"
        copies = (getattr(b.residual, "expansion", 1) if self.streams else 1)
        self.copies = copies
        self.table = nn.Parameter(torch.empty(sum(primes), c.head_dim, dtype=b.dtype))
        init_weight(self.table, b.init, "embed")
        self.kv = Linear((n - 1) * heads * c.head_dim, (copies + 1) * d, False, b)
        self.q_gain = nn.Parameter(torch.ones(copies, d))
        self.k_gain = nn.Parameter(torch.ones(copies, d))
        self.eps = c.norm.eps
        if c.conv_size:
            self.conv = CausalDepthwise(copies * d, c.conv_size, zero=True)
            self.conv_gain = nn.Parameter(torch.ones(copies, d))
            self.dilation = n

    def rows(self, ids: torch.Tensor, starts: torch.Tensor) -> torch.Tensor:
        """Table rows [b, t, (n-1)*heads] of the n-grams ending at each position: the
        n-gram of the last j+1 ids hashes to XOR_{i<=j} ids[t-i]*m_i in wrapping uint32
        arithmetic; ids before the row's / document's start or at or before the last
        boundary token count as the boundary's (or 0's)."""
        c = self.c
        bsz, t = ids.shape
        pos = torch.arange(t, device=ids.device)
        zero = torch.zeros(bsz, t, dtype=torch.long, device=ids.device)
        start = zero
        if starts is not None:  # a document start begins a span
            start = torch.cummax(torch.where(starts, pos.expand(bsz, t), zero), 1).values
        if c.boundary_token is not None:  # positions after a boundary token do not reach it
            after = torch.where(ids == c.boundary_token, (pos + 1).expand(bsz, t), zero)
            start = torch.maximum(start, F.pad(torch.cummax(after, 1).values[:, :-1], (1, 0)))
        pad = c.boundary_token or 0
        if c.vocab_classes:
            ids, pad = ids % c.vocab_classes, pad % c.vocab_classes
        h = torch.zeros_like(ids)
        rows = []
        for i in range(c.max_ngram_size):
            back = pos - i
            prev = torch.where(back.unsqueeze(0) >= start, ids[:, back.clamp(min=0)], torch.full_like(ids, pad))
            h = h ^ ((prev * self.multipliers[i]) & 0xFFFFFFFF)
            if i:
                rows.append(h.unsqueeze(-1) % self.primes[i - 1] + self.offsets[i - 1])
        return torch.cat(rows, -1)

    @staticmethod
    def _norm(x, gain, eps):
        y = x.float()
        return y * torch.rsqrt(y.square().mean(-1, keepdim=True) + eps) * gain.float()

    def forward(self, x, ctx: Context):
        ids = ctx.input_ids
        starts = None
        if getattr(ctx, "segments", None) is not None:
            starts = ctx.positions == 0
        memory = self.table[self.rows(ids, starts)].flatten(2).to(x.dtype)
        hdn = x if self.streams else x.unsqueeze(2)
        bsz, t, n, d = hdn.shape
        kv = self.kv(memory, ctx)
        key, value = kv[..., : n * d].reshape(bsz, t, n, d), kv[..., n * d:]
        a = (self._norm(hdn, self.q_gain, self.eps) * self._norm(key, self.k_gain, self.eps)).sum(-1) / math.sqrt(d)
        gate = torch.sigmoid(torch.sign(a) * torch.sqrt(a.abs().clamp(min=1e-6)))
        u = gate.unsqueeze(-1) * value.float().unsqueeze(2)
        if hasattr(self, "conv"):
            cu = self._norm(u, self.conv_gain, self.eps).reshape(bsz, t, n * d)
            u = u + F.silu(self.conv(cu, ctx)).reshape(u.shape)
        y = hdn + u.to(hdn.dtype)
        return y if self.streams else y[:, :, 0]


@register("engram")
def _engram(c, b):
    return Engram(c, b)


# ------------------------------------------------------------------ doc_copy
_BASE, _MIX = 0x9E3779B97F4A7C15, 0x2545F4914F6CDD1D


def _i64(n: int) -> int:
    n &= 2 ** 64 - 1
    return n - 2 ** 64 if n >= 2 ** 63 else n


def copy_candidates(tokens, within, doc, lengths, counts):
    """For each position, the token after the latest earlier occurrence (in the same
    document) of the longest context of `lengths` ending here, and a bucket
    (0 = none; else (rank of the length) * counts + min(occurrences, counts))."""
    bsz, t = tokens.shape
    dev = tokens.device
    pos = torch.arange(t, device=dev)
    best_len = torch.zeros(bsz, t, dtype=torch.long, device=dev)
    best_prev = torch.zeros(bsz, t, dtype=torch.long, device=dev)
    best_seen = torch.zeros(bsz, t, dtype=torch.long, device=dev)
    tok = tokens.long() + 1
    base = _i64(_BASE)
    for rank, length in enumerate(lengths, start=1):
        if length > t:
            break
        # wrapping 64-bit polynomial hash of the window, keyed by the document
        h = torch.zeros_like(tok)
        for i in range(length):
            shifted = F.pad(tok[:, : t - i], (i, 0))
            h = h * base + shifted
        h = h ^ (doc.long() * _i64(_MIX)) ^ _i64(length * _MIX * 3)
        valid = within >= length - 1
        unique = -(pos + 1).expand(bsz, t) - (rank << 40)   # keys of invalid windows match nothing
        key = torch.where(valid, h, unique)
        order = torch.sort(key, dim=1, stable=True).indices
        sk = key.gather(1, order)
        same = sk[:, 1:] == sk[:, :-1]
        prev_sorted = torch.full((bsz, t), -1, dtype=torch.long, device=dev)
        prev_sorted[:, 1:] = torch.where(same, order[:, :-1], torch.full_like(order[:, 1:], -1))
        run_start = torch.cummax(torch.where(F.pad(~same, (1, 0), value=True), pos.expand(bsz, t),
                                             torch.zeros_like(order)), 1).values
        seen_sorted = pos.expand(bsz, t) - run_start
        prev = torch.empty_like(prev_sorted).scatter_(1, order, prev_sorted)
        seen = torch.empty_like(seen_sorted).scatter_(1, order, seen_sorted)
        found = valid & (prev >= 0)
        # exactness: the windows must really match (a hash collision finds nothing)
        ok = found.clone()
        for i in range(length):
            a = tokens.gather(1, (pos - i).clamp(min=0).expand(bsz, t))
            bb = tokens.gather(1, (prev - i).clamp(min=0))
            ok &= a == bb
        best_len = torch.where(ok, torch.full_like(best_len, rank), best_len)
        best_prev = torch.where(ok, prev, best_prev)
        best_seen = torch.where(ok, seen, best_seen)
    after = tokens.gather(1, (best_prev + 1).clamp(max=t - 1))
    candidate = torch.where(best_len > 0, after, torch.zeros_like(after))
    bucket = torch.where(best_len > 0, (best_len - 1) * counts + best_seen.clamp(1, counts),
                         torch.zeros_like(best_len))
    return candidate, bucket


class DocCopy(nn.Module):
    """Adds gain·(E[c]·s[b] + e[b]) of each position's candidate c and bucket b to the
    stream (every copy of a widened one). With its ``copy`` port it pushes the vector,
    or reads it instead and adds it by its own gain."""
    no_weight_decay = ("gain", "scale", "bucket_embed")
    no_muon = True


    def __init__(self, c: L.DocCopyConfig, b: BuildContext):
        super().__init__()
        self.c = c
        self.ports = b.ports or ()
        self.gain = nn.Parameter(torch.tensor(float(c.gain)))
        self.reads = any(p.name == "copy" and p.mode != "write" for p in self.ports)
        object.__setattr__(self, "embedding", b.embedding)
        if not self.reads:
            buckets = 1 + len(c.lengths) * c.counts
            self.scale = nn.Parameter(torch.zeros(buckets))
            self.bucket_embed = nn.Parameter(torch.zeros(buckets, b.d_model))

    def vector(self, ctx: Context):
        tokens = ctx.input_ids
        seg = ctx.segments if getattr(ctx, "segments", None) is not None else torch.zeros_like(tokens)
        within = ctx.positions if getattr(ctx, "segments", None) is not None else \
            torch.arange(tokens.shape[1], device=tokens.device).expand_as(tokens)
        cand, bucket = copy_candidates(tokens, within, seg, list(self.c.lengths), self.c.counts)
        live = (torch.arange(self.scale.shape[0], device=bucket.device) > 0).float()
        rows = self.embedding.tokens.embedding[cand]
        scale = (self.scale * live)[bucket].unsqueeze(-1)
        return rows * scale.to(rows.dtype) + (self.bucket_embed * live[:, None])[bucket].to(rows.dtype)

    def forward(self, x, ctx: Context):
        if self.reads:
            port = next(p for p in self.ports if p.name == "copy" and p.mode != "write")
            v = ctx.read(port.tap, port.mode == "pop")
        else:
            v = self.vector(ctx)
        for p in self.ports:
            if p.name == "copy" and p.mode == "write":
                ctx.push(p.tap, v)
        add = (self.gain * v.float()).to(x.dtype)
        return x + (add.unsqueeze(2) if x.dim() == 4 else add)


@register("doc_copy")
def _doc_copy(c, b):
    return DocCopy(c, b)
