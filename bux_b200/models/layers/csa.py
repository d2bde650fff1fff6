"""Compressed sparse attention (``csa``, DeepSeek-V4's layer).

A *latent* is a ``head_dim`` wide RMS-normalised projection of a token: the key and the
value, at once, of a single KV head that every query head shares. A query attends, in ONE
softmax, to (a) the latents of a sliding window of tokens and (b) *compressed* latents:
every ``compress_ratio`` tokens of a document pooled into one, per channel under a softmax
gate learned from the tokens, RMS-normalised, rotated to the position of the group's first
token and visible from the group's last token on. Queries come from a ``q_lora_rank``
latent (or the input); the first ``rope.fraction`` dims of queries and latents are
rotated, and since the values were rotated with the keys the head outputs are rotated
back by their query's position. ``o_lora_rank`` makes the output projection grouped and
low-rank. Reference: ``architecture/attention/csa.py:50-377`` there.

An indexer (``indexer=indexer(...)``) keeps the ``top_k`` compressed latents of each query
(its queries from the query latent, its keys projected from the compressed latents); without
one a query attends to every compressed latent it may see. Ports: ``kv`` written pushes the
compressed latents with the indexer's keys, read reuses them (the layer then has no
compression of its own, and an indexer it runs scores the keys that came); ``index`` written
pushes the kept latents, read reuses them (no indexer); ``candidates`` written pushes a coarse
pool (blocks of ``candidate_block_size`` latents, ``candidate_top_k`` latents in all), read
confines the indexer's picks to it.

This is the layer's dense statement (all t x (t + t) logits), like the other sparse layers here.
"""

from __future__ import annotations


import torch
from torch import nn

from ...config import layers as L
from ...ops import reference as ref
from ..registry import BuildContext, Context, register
from . import rope as rope_lib
from .basic import Linear, Norm, init_weight


class CSA(nn.Module):
    def __init__(self, c: L.CSAConfig, b: BuildContext):
        super().__init__()
        self.c = c
        self.ports = list(b.ports or ())
        width = b.width if isinstance(b.width, int) else b.d_model
        h, d, r = c.num_heads, c.head_dim, c.compress_ratio
        if r is None and (c.indexer is not None or self.ports):
            raise ValueError("csa: an indexer, and the kv, index and candidates ports, are for compressed "
                             "latents; set compress_ratio")
        reads = {p.name for p in self.ports if p.mode != "write"}
        compresses = r is not None and "kv" not in reads
        runs_indexer = c.indexer is not None and "index" not in reads
        if not runs_indexer and any(p.name == "candidates" for p in self.ports):
            raise ValueError("csa: the candidates port is its indexer's: the layer runs none")
        rank, groups = c.o_lora_rank, c.o_groups
        if rank and h % groups:
            raise ValueError(f"csa: {h} heads do not split into {groups} o_groups")
        self.h, self.d, self.ratio = h, d, r
        latent = c.q_lora_rank
        if latent:
            self.q_a = Linear(width, latent, False, b, role="q")
            self.q_a_norm = Norm(c.latent_norm, latent)
        self.q = Linear(latent or width, h * d, False, b, role="q")
        self.kv = Linear(width, d, False, b, role="kv")
        self.kv_norm = Norm(c.latent_norm, d)
        if compresses:
            self.compress_kv = Linear(width, d, False, b, role="kv")
            self.compress_norm = Norm(c.latent_norm, d)
            if r > 1:
                self.compress_gate = Linear(width, d, False, b, role="kv")
        if rank:
            self.o_a = nn.Parameter(torch.empty(groups, h * d // groups, rank, dtype=b.dtype))
            init_weight(self.o_a, b.init)
        self.o = Linear(groups * rank if rank else h * d, width, False, b, role="o", init_role="out")
        if c.qk_norm is not None:
            self.q_norm = Norm(c.qk_norm, d)
        if c.sinks:
            self.sinks = nn.Parameter(torch.zeros(h))
            self.sinks.no_weight_decay = True
        if c.rope is not None:
            self.rotated = rope_lib.rotated_dims(d, c.rope.fraction)
            inv, gain = rope_lib.inverse_frequencies(c.rope, d)
            self.register_buffer("inv_freq", inv, persistent=False)
            self.rope_gain = gain
        if runs_indexer:
            from .sparse import Indexer

            self.indexer = Indexer(c.indexer, width, c.rope, getattr(self, "rotated", 0), b,
                                   query_width=latent or width, key_width=d if compresses else None,
                                   key_norm=c.latent_norm)

    # ---- rotation of the first `rotated` dims
    def _rotate(self, x, positions, back: bool = False):
        if self.c.rope is None or self.rotated == 0:
            return x
        cos, sin = rope_lib.tables(-positions if back else positions, self.inv_freq, self.rope_gain)
        out = ref.rope(x, cos, sin, interleaved=self.c.rope.layout == "interleaved")
        if back and self.rope_gain != 1.0:
            # rotating back multiplies by the gain again: take it out twice
            out = torch.cat([out[..., : self.rotated] / self.rope_gain ** 2, out[..., self.rotated:]], -1)
        return out

    def _compressed(self, x, ctx: Context, within):
        """(latents [b, t, d] one slot per token, valid [b, t]): slot i holds the latent of the
        group of `ratio` tokens of its document that ends at token i, where one does."""
        r = self.ratio
        t = x.shape[1]
        kv = self.compress_kv(x, ctx).float()
        if r > 1:
            gate = self.compress_gate(x, ctx).float()
            pad_kv = torch.nn.functional.pad(kv, (0, 0, r - 1, 0))
            pad_gate = torch.nn.functional.pad(gate, (0, 0, r - 1, 0), value=float("-inf"))
            stack_kv = torch.stack([pad_kv[:, i:i + t] for i in range(r)], dim=2)       # [b, t, r, d]
            stack_gate = torch.stack([pad_gate[:, i:i + t] for i in range(r)], dim=2)
            kv = (stack_kv * torch.softmax(stack_gate, dim=2)).sum(2)
        latent = self.compress_norm(kv.to(x.dtype), ctx)
        valid = (within + 1) % r == 0
        # rotated to the position of the group's first token
        first = torch.gather(ctx.positions, 1, (torch.arange(t, device=x.device) - (r - 1)).clamp_min(0)
                             .unsqueeze(0).expand_as(ctx.positions))
        return self._rotate(latent.unsqueeze(2), first)[:, :, 0], valid, latent, first

    def _port(self, name: str, write: bool):
        for p in self.ports:
            if p.name == name and (p.mode == "write") == write:
                return p
        return None

    def forward(self, x, ctx: Context):
        c = self.c
        bsz, t, _ = x.shape
        h, d = self.h, self.d
        pos = ctx.positions
        seg = ctx.segments if getattr(ctx, "segments", None) is not None else torch.ones_like(pos)
        within = pos
        if getattr(ctx, "segments", None) is None:
            within = torch.arange(t, device=x.device).unsqueeze(0).expand(bsz, t)
        query = self.q_a_norm(self.q_a(x, ctx), ctx) if hasattr(self, "q_a") else x
        q = self.q(query, ctx).view(bsz, t, h, d)
        if hasattr(self, "q_norm"):
            q = self.q_norm(q, ctx)
        q = self._rotate(q, pos)
        kv = self._rotate(self.kv_norm(self.kv(x, ctx), ctx).unsqueeze(2), pos)[:, :, 0]      # [b, t, d]
        scale = c.scale if c.scale is not None else d ** -0.5
        qi = torch.arange(t, device=x.device)
        same = seg.unsqueeze(2) == seg.unsqueeze(1)                                           # [b, t, s]
        causal = (qi.unsqueeze(1) >= qi.unsqueeze(0)).unsqueeze(0)
        window = causal & same
        if c.sliding_window_size:
            window = window & ((qi.unsqueeze(1) - qi.unsqueeze(0)) < c.sliding_window_size).unsqueeze(0)
        keys, mask = [kv], [window]
        picked_scores = kept = None
        if self.ratio is not None:
            from . import sparse as S

            port = self._port("kv", write=False)
            if port is not None:
                latents, valid, index_keys = ctx.read(port.tap, port.mode == "pop")
            else:
                latents, valid, plain, first = self._compressed(x, ctx, within)
                index_keys = None
                if hasattr(self, "indexer") and hasattr(self.indexer, "k"):
                    index_keys = self.indexer.keys_of(plain, first, ctx)
            port = self._port("kv", write=True)
            if port is not None:
                ctx.push(port.tap, (latents, valid, index_keys))
            seen = causal & same & valid.unsqueeze(1)           # from its group's last token on
            kept = seen
            port = self._port("index", write=False)
            if port is not None:
                kept = ctx.read(port.tap, port.mode == "pop") & seen
            elif hasattr(self, "indexer"):
                if index_keys is None:
                    raise ValueError("csa: the latents that came through the kv port carry no indexer keys "
                                     "(the layer that wrote them runs no indexer)")
                ic = c.indexer
                picked_scores = self.indexer.scores_of(x, query, index_keys, ctx)
                allowed = seen
                port = self._port("candidates", write=False)
                if port is not None:
                    allowed = allowed & ctx.read(port.tap, port.mode == "pop")
                kept = S.top_mask(picked_scores, allowed, ic.top_k)
                port = self._port("candidates", write=True)
                if port is not None:
                    order = valid.long().cumsum(-1) - 1          # the latents of a row, counted in order
                    block = (order.clamp_min(0) // ic.candidate_block_size)
                    blocks = int(block.max().item()) + 1
                    pool = S.candidate_pool(picked_scores, seen, block, blocks,
                                            max(ic.candidate_top_k // ic.candidate_block_size, 1))
                    ctx.push(port.tap, pool & valid.unsqueeze(1))
            port = self._port("index", write=True)
            if port is not None:
                ctx.push(port.tap, kept)
            keys.append(latents)
            mask.append(kept)
        k_all = torch.cat(keys, dim=1).float()                                                 # [b, S, d]
        m_all = torch.cat(mask, dim=2)                                                        # [b, t, S]
        logits = torch.einsum("bthd,bsd->bhts", q.float(), k_all) * scale
        if c.softcap:
            logits = c.softcap * torch.tanh(logits / c.softcap)
        logits = logits.masked_fill(~m_all.unsqueeze(1), float("-inf"))
        if hasattr(self, "sinks"):
            sink = self.sinks.float().view(1, h, 1, 1).expand(bsz, h, t, 1)
            probs = torch.softmax(torch.cat([logits, sink], dim=-1), dim=-1)[..., :-1]
        else:
            probs = torch.softmax(logits, dim=-1)
        if picked_scores is not None and ctx.training and c.indexer.loss_weight:
            # the indexer's own loss: KL(attention over the kept latents || softmax of its scores)
            from . import sparse as S

            target = probs[..., t:].sum(1).detach()
            ctx.report("indexer_loss", S.indexer_loss(picked_scores, kept, target), c.indexer.loss_weight)
        out = torch.einsum("bhts,bsd->bthd", probs, k_all).to(x.dtype)
        out = self._rotate(out, pos, back=True)
        if hasattr(self, "o_a"):
            groups = self.o_a.shape[0]
            low = torch.einsum("btgi,gir->btgr", out.reshape(bsz, t, groups, -1), self.o_a.to(out.dtype))
            return self.o(low.reshape(bsz, t, -1), ctx)
        return self.o(out.reshape(bsz, t, h * d), ctx)


@register("csa")
def _csa(c, b):
    return CSA(c, b)
