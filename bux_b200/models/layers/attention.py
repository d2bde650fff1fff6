"""Grouped-query softmax attention (``gqa``).

One fused QKV projection ([(H + 2G)·D, d], one GEMM), per-head QK-norm fused with RoPE
in one kernel, the tcgen05 attention kernel (causal, GQA, sliding window, sinks), an
optional output gate, then the output projection.

Reference: ``architecture/attention/gqa.py:79-833`` (`SoftmaxAttention`, `Attention`).
Parameter names there are ``q / k / v / o`` (+ ``q_norm / k_norm``, ``sinks``); here
``qkv`` holds q, k, v stacked along the output rows in that order, and the checkpoint
layer splits / joins them.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ... import ops
from ...config import layers as L
from ...ops import reference as ref
from ..registry import BuildContext, Context, register
from . import rope as rope_lib
from .basic import Linear, Norm, init_weight

def power_scale(pos: torch.Tensor, power: float, length: int) -> torch.Tensor:
    """(1 + n / length) ** power at position n counted from 1 (``attention/gqa.py:817-823`` there)."""
    return torch.exp(power * torch.log1p((pos.float() + 1) / length))


def length_scale(pos: torch.Tensor, log_scale: float, floor: int) -> torch.Tensor:
    """1 + log_scale · ln(max(n / floor, 1)) at position n counted from 1 (``:826-832`` there)."""
    return 1 + log_scale * torch.log(((pos.float() + 1) / floor).clamp_min(1.0))


def exclusive(out: torch.Tensor, v: torch.Tensor, strength: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exclusive self-attention: each head's output y less its part along its query's own
    value, y − s (y·u) u with u = v / |v|, in fp32 (``attention/gqa.py:700-728`` there)."""
    h, g = out.shape[2], v.shape[2]
    y = out.float()
    u = v.float().repeat_interleave(h // g, dim=2)
    u = u * torch.rsqrt(u.square().sum(-1, keepdim=True).clamp_min(1e-24))
    along = (y * u).sum(-1, keepdim=True) * u
    if strength is not None:
        along = along * strength.float()[:, None]
    return (y - along).to(out.dtype)


def relative_bias(r: torch.Tensor, table: torch.Tensor, t: int) -> torch.Tensor:
    """[b, h, t, s] bias <r[b, t, h], table[:, t − s]>; keys ahead of the query, or `extent`
    or more behind, get none (``attention/gqa.py:802-814`` there)."""
    extent = table.shape[-1]
    index = torch.arange(t, device=r.device)
    offset = index[:, None] - index[None, :]
    per_offset = torch.einsum("bthr,re->bhte", r.float(), table.float())      # [b, h, t, extent]
    picked = per_offset.gather(-1, offset.clamp(0, extent - 1).expand(r.shape[0], r.shape[2], t, t))
    return picked * ((offset >= 0) & (offset < extent))


class GQA(nn.Module):
    def __init__(self, c: L.GQAConfig, b: BuildContext):
        super().__init__()
        self.c = c
        width = b.width if isinstance(b.width, int) else b.d_model
        ports = tuple(b.ports or ())
        reads = {p.name for p in ports if p.mode != "write"}
        self.h, self.g = c.num_heads, c.num_kv_heads
        self.hq = 2 * self.h if c.differential else self.h  # differential: a pair of query heads per output
        self.d = c.head_dim or width // c.num_heads
        self.dv = c.v_head_dim or self.d
        self.q_rows, self.k_rows = self.hq * self.d, self.g * self.d
        self.v_rows = 0 if c.k_eq_v else self.g * self.dv       # k_eq_v: values are the normalised keys
        from .. import placement

        out_bias = c.bias if c.output_bias is None else c.output_bias
        # the mimetic initialisation writes V's and O's rows by index: those two are built whole
        with placement.whole_parameters() if c.mimetic_vo is not None else placement.placing(placement._experts, placement._rows):
            self.qkv = Linear(width, self.q_rows + self.k_rows + self.v_rows, c.bias, b, role="q")
            self.o = Linear(self.h * self.dv, width, out_bias, b, role="o", init_role="out")
            if c.mimetic_vo is not None:
                self._mimetic_vo(width, c.mimetic_vo, c.mimetic_noise)
        if c.qk_norm is not None:
            per = self.d
            self.q_norm = Norm(c.qk_norm, self.hq * per if c.qk_norm_all_heads else per)
            self.k_norm = Norm(c.qk_norm, self.g * per if c.qk_norm_all_heads else per)
        if c.k_eq_v:
            eps = c.qk_norm.eps if c.qk_norm is not None else 1e-6
            self.v_norm = Norm(L.NormalizationConfig(type="rmsnorm", affine=False, eps=eps), self.d)
        if c.kv_conv_size and "kv" not in reads:
            from .conv import CausalDepthwise

            self.k_conv = CausalDepthwise(self.k_rows, c.kv_conv_size)
            if self.v_rows:
                self.v_conv = CausalDepthwise(self.v_rows, c.kv_conv_size)
        if c.sinks:
            self.sinks = nn.Parameter(torch.zeros(self.h))
        if c.differential:
            self.lambda_proj = Linear(width, self.h, False, b, role="q")
        if c.exclusive == "learned":
            self.xsa_alpha = nn.Parameter(torch.zeros(self.h))
        if "v" in reads and c.value_residual != "fixed":
            self.v_mix = nn.Parameter(torch.full((2,) if c.value_residual == "learned" else (), 0.5))
        if "ve" in reads and c.value_embed_gate is not None:
            self.ve_gate = Linear(2 * c.value_embed_gate, self.g, False, b, role="q")
            nn.init.zeros_(self.ve_gate.weight)
        if c.relative_bias is not None:
            self.rel_proj = Linear(width, self.h * c.relative_bias.rank, c.bias, b, role="q")
            self.rel_table = nn.Parameter(torch.zeros(c.relative_bias.rank, c.relative_bias.extent))
        if c.gated:
            # the gate: act(x W + b_h); HyGA's parts make W low-rank (per-head up projection),
            # add the head's own output to the logits, and multiply by a gate from all heads
            gate_dims = c.gate_input_rank or self.dv
            gate_out = self.h if c.gate_per_head else self.h * gate_dims
            self.gate = Linear(width, gate_out, c.bias, b, role="q")
            if c.gate_head_bias:
                self.gate_bias = nn.Parameter(torch.zeros(self.h))
            if c.gate_input_rank:
                self.gate_up = nn.Parameter(torch.empty(self.h, c.gate_input_rank, self.dv))
                init_weight(self.gate_up, b.init)
            if c.gate_output_rank:
                self.output_gate_down = nn.Parameter(torch.empty(self.h, self.dv, c.gate_output_rank))
                self.output_gate_up = nn.Parameter(torch.empty(self.h, c.gate_output_rank, self.dv))
                init_weight(self.output_gate_down, b.init)
                init_weight(self.output_gate_up, b.init)
            if c.gate_cross_head:
                self.cross_gate = Linear(self.h * self.dv, self.h, c.bias, b, role="q")
        if c.output_norm is not None:
            self.out_norm = Norm(c.output_norm, self.dv)
        self.ports = ()
        if c.indexer is not None and not any(p.name == "index" and p.mode != "write" for p in (b.ports or ())):
            from .sparse import Indexer

            rot = rope_lib.rotated_dims(self.d, c.rope.fraction) if c.rope is not None else 0
            self.indexer = Indexer(c.indexer, width, c.rope, rot, b)
        if c.rope is not None:
            inv, gain = rope_lib.inverse_frequencies(c.rope, self.d)
            self.register_buffer("inv_freq", inv, persistent=False)
            self.rope_gain = gain

    # -- pieces
    def _tables(self, ctx: Context):
        key = (id(self.c.rope), self.d)
        return ctx.rope_tables(key, lambda: rope_lib.tables(ctx.positions, self.inv_freq, self.rope_gain))

    def _norm_rope(self, x, norm: Optional[Norm], ctx: Context):
        c = self.c
        has_rope = c.rope is not None
        fused = (has_rope and c.rope.layout == "half" and not c.qk_norm_all_heads
                 and rope_lib.rotated_dims(self.d, c.rope.fraction) == self.d
                 and (norm is None or (norm.c.type == "rmsnorm" and norm.bias is None
                                       and not norm.c.scale_input)))
        if fused:
            cos, sin = self._tables(ctx)
            w = None
            if norm is not None:
                w = norm.scale + 1.0 if (norm.c.zero_centered and norm.scale is not None) else norm.scale
                if w is None:
                    w = torch.ones(self.d, device=x.device)
                return ops.rmsnorm_rope(x, w, cos, sin, norm.c.eps)
            return ops.rope(x, cos, sin)
        if norm is not None:
            x = norm(x.flatten(-2), ctx).view_as(x) if c.qk_norm_all_heads else norm(x, ctx)
        if has_rope:
            cos, sin = self._tables(ctx)
            x = ref.rope(x, cos, sin, interleaved=c.rope.layout == "interleaved")
        return x

    def _norm_rope_paired(self, x, norm: Optional[Norm], ctx: Context):
        """Paired heads: head i of the token at position p is turned at 2p + (i mod 2)
        (``attention/gqa.py:664-681`` there); the norm is each head's own, as without pairs."""
        c = self.c
        if norm is not None:
            x = norm(x.flatten(-2), ctx).view_as(x) if c.qk_norm_all_heads else norm(x, ctx)
        if c.rope is None:
            return x
        bsz, t, n, d = x.shape
        halves = x.reshape(bsz, t, n // 2, 2, d)
        turned = []
        for i in (0, 1):
            cos, sin = rope_lib.tables(2 * ctx.positions + i, self.inv_freq, self.rope_gain)
            turned.append(ref.rope(halves[..., i, :], cos, sin, interleaved=c.rope.layout == "interleaved"))
        return torch.stack(turned, 3).reshape(bsz, t, n, d)

    def _attend_paired(self, q, k, v, ctx: Context):
        """Heads j and j + n/2 interleaved along the sequence into one of twice the length
        (position 2p: the first half of the heads of token p, 2p + 1: the second half), so a
        query sees both heads' keys in one softmax; a window counts interleaved positions
        (``attention/gqa.py:731-747`` there)."""
        c = self.c
        bsz, t, h, _ = q.shape

        def pair(a):
            return a.reshape(bsz, 2 * t, a.shape[2] // 2, a.shape[3])

        segments = None
        if ctx.segments is not None:
            segments = ctx.segments.repeat_interleave(2, dim=1)
        out = ops.attention(pair(q), pair(k), pair(v), causal=True, window=c.sliding_window_size,
                            softcap=c.softcap, scale=c.scale, segments=segments)
        return out.reshape(bsz, t, h, -1)

    def forward(self, x, ctx: Context):
        c = self.c
        qkv = self.qkv(x, ctx)
        bsz, t = qkv.shape[:2]  # with the sequence gathered inside the projection, longer than x
        if c.k_eq_v:
            q, k = qkv.split((self.q_rows, self.k_rows), dim=-1)
            v = None
        else:
            q, k, v = qkv.split((self.q_rows, self.k_rows, self.v_rows), dim=-1)  # backward: one cat
        if hasattr(self, "k_conv"):  # k + conv(k), v + conv(v): before the heads split
            k = k + self.k_conv(k, ctx)
            if v is not None:
                v = v + self.v_conv(v, ctx)
        q = q.reshape(bsz, t, self.hq, self.d)
        k = k.reshape(bsz, t, self.g, self.d)
        if c.k_eq_v:  # each head's projected key, normalised without a gain and not rotated
            v = self.v_norm(k, ctx)
        else:
            v = v.reshape(bsz, t, self.g, self.dv)
        for port in self.ports:  # value embeddings, then value residual / kv sharing, through taps
            if port.name == "ve" and port.mode != "write":
                v = self._add_value_embedding(x, v, ctx.read(port.tap, port.mode == "pop"), ctx)
        for port in self.ports:
            if port.name == "v" and port.mode != "write":
                v = self._mix_values(v, ctx.read(port.tap, port.mode == "pop"))
            elif port.name == "kv" and port.mode != "write":
                k, v = ctx.read(port.tap, port.mode == "pop")
        rotate = self._norm_rope_paired if c.paired else self._norm_rope
        q = rotate(q, getattr(self, "q_norm", None), ctx)
        if c.power_scale is not None:
            q = (q.float() * power_scale(ctx.positions, c.power_scale, c.power_scale_length)[..., None, None]).to(q.dtype)
        kv_shared = any(p.name == "kv" and p.mode != "write" for p in self.ports)
        if not kv_shared:
            k = rotate(k, getattr(self, "k_norm", None), ctx)
        for port in self.ports:
            if port.mode == "write":
                ctx.push(port.tap, v if port.name == "v" else (k, v))
        if c.paired:
            return self._finish(self._attend_paired(q, k, v, ctx), x, v, bsz, t, ctx)
        if c.indexer is not None:
            out = self._sparse(x, q, k, v, ctx)
            return self._finish(out, x, v, bsz, t, ctx)
        if c.relative_bias is not None or (c.attention_dropout and ctx.training):
            out = self._full_logits(x, q, k, v, ctx)
            return self._finish(out, x, v, bsz, t, ctx)
        if c.log_scale is not None:
            # the length scale multiplies a query's logits, so it is put on the query
            # (sinks keep their logit; a softcap applies after it, as there)
            q = (q.float() * length_scale(ctx.positions, c.log_scale, c.log_scale_floor)[..., None, None]).to(q.dtype)
        sinks = getattr(self, "sinks", None)
        if sinks is not None and c.differential:
            sinks = sinks.repeat_interleave(2)
        kw = dict(causal=True, window=c.sliding_window_size, sinks=sinks,
                  softcap=c.softcap, scale=c.scale, segments=ctx.segments)
        cp = getattr(ctx.parallel, "context_group", None) if ctx.parallel is not None else None
        if ctx.observing and cp is None:
            from .. import observe

            observe.attention_sample(ctx, q, k, c.scale)
        if ctx.cache is not None:
            # incremental decoding: the new keys and values join the layer's cache and the new
            # queries (the last t positions) attend over all of it; padding is never read
            from ...ops import reference as ref

            k_all, v_all = ctx.cache.extend(self, k, v)
            out, _ = ref.attention(q, k_all, v_all, **{**kw, "segments": ctx.cache.segments()})
            return self._finish(out, x, v, bsz, t, ctx)
        if cp is not None:
            from ...parallel import context

            out = context.attend(ops.attention, q, k, v, cp, ctx.methods.attention, **kw)
        else:
            out = ops.attention(q, k, v, **kw)
        return self._finish(out, x, v, bsz, t, ctx)

    def _mimetic_vo(self, width: int, beta: float, noise: float) -> None:
        """Mimetic V-O init (modded-nanogpt's, after Trockman & Kolter 2023): value head j reads the
        stream's channels j·dv .. (j+1)·dv times sqrt(beta), every query head of its group writes its
        output back onto them times -sqrt(beta) / group, so a head that attends to itself subtracts
        beta / group of those channels; both matrices take noise of std `noise` in place of their
        own draws. Reference: ``initializers.py:140`` (`mimetic_vo`)."""
        values, group = self.g * self.dv, self.h // self.g
        if values > width:
            raise ValueError(f"mimetic_vo maps {self.g} value heads of {self.dv} onto the stream's channels: "
                             f"{values} of them do not fit in a width of {width}")
        root = beta ** 0.5
        with torch.no_grad():
            w = self.qkv.weight
            v = torch.randn(values, width) * noise + root * torch.eye(values, width)
            w[self.q_rows + self.k_rows:] = v.to(w.dtype)
            read = torch.arange(self.h * self.dv)
            channel = (read // self.dv) // group * self.dv + read % self.dv   # query head i's dim r → its value head's dim r
            o = torch.randn(width, self.h * self.dv) * noise
            o[channel, read] -= root / group
            self.o.weight.copy_(o.to(self.o.weight.dtype))

    def _add_value_embedding(self, x, v, e, ctx: Context):
        """v + 2·sigmoid(W [x[:n], e[:n]])·e with a gate per kv head (W starts at 0, so the
        rows are added whole at first); without the gate, v + e."""
        bsz, t, g, dv = v.shape
        e = e.reshape(bsz, t, g * dv).to(v.dtype)
        rows = e.view(bsz, t, g, dv)
        if not hasattr(self, "ve_gate"):
            return v + rows
        n = self.ve_gate.weight.shape[1] // 2
        gate = self.ve_gate(torch.cat([x[..., :n], e[..., :n]], -1), ctx)
        return v + (2 * torch.sigmoid(gate.float())).unsqueeze(-1).to(v.dtype) * rows

    def _mix_values(self, v, v1):
        """The value residual a·v + b·v1: a = b = 0.5 fixed, both learned, or a learned, b = 1 − a."""
        if not hasattr(self, "v_mix"):
            return 0.5 * (v + v1)
        w = self.v_mix.to(v.dtype)
        if self.c.value_residual == "learned":
            return w[0] * v + w[1] * v1
        return w * v + (1 - w) * v1

    def _full_logits(self, x, q, k, v, ctx: Context):
        """Attention through all t × s logits, for what needs them: the relative position
        bias and dropout of the probabilities (``attention/gqa.py:834-936`` there). Scaled
        logits plus bias, times the length scale, soft-capped, masked, softmax with sinks."""
        from . import sparse as S

        c = self.c
        bsz, t, h, d = q.shape
        g = k.shape[2]
        kk = k.repeat_interleave(h // g, dim=2)
        vv = v.repeat_interleave(h // g, dim=2)
        logits = torch.einsum("bthd,bshd->bhts", q.float(), kk.float()) * (c.scale if c.scale is not None else d ** -0.5)
        if c.relative_bias is not None:
            r = self.rel_proj(x, ctx).view(bsz, t, h, -1)
            logits = logits + relative_bias(r, self.rel_table, t)
        if c.log_scale is not None:
            logits = logits * length_scale(ctx.positions, c.log_scale, c.log_scale_floor)[:, None, :, None]
        if c.softcap:
            logits = c.softcap * torch.tanh(logits / c.softcap)
        seen = S.seen_mask(ctx, t, c.sliding_window_size)
        logits = logits.masked_fill(~seen[:, None], float("-inf"))
        if hasattr(self, "sinks"):
            sink = self.sinks.float().view(1, h, 1, 1).expand(bsz, h, t, 1)
            probs = torch.softmax(torch.cat([logits, sink], -1), -1)[..., :-1]
        else:
            probs = torch.softmax(logits, -1)
        if c.attention_dropout and ctx.training:
            probs = nn.functional.dropout(probs, c.attention_dropout)
        return torch.einsum("bhts,bshd->bthd", probs, vv.float()).to(q.dtype)

    def _sparse(self, x, q, k, v, ctx: Context):
        """Attention over the keys an indexer kept (its own, or another layer's through
        the ``index`` port), and the indexer's distillation loss."""
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
        out, target = S.attend_kept(q, k, v, kept, c.scale, getattr(self, "sinks", None), c.softcap)
        if picked is not None and ctx.training and c.indexer.loss_weight:
            ctx.report("indexer_loss", self.indexer.loss(picked, target), c.indexer.loss_weight)
        return out

    def _finish(self, out, x, v, bsz, t, ctx: Context):
        c = self.c
        if c.differential:  # a1 − sigmoid(x W)·a2 of each pair of query heads, side by side
            pairs = out.reshape(bsz, t, self.h, 2, self.dv)
            lam = torch.sigmoid(self.lambda_proj(x, ctx).float()).to(out.dtype).unsqueeze(-1)
            out = pairs[..., 0, :] - lam * pairs[..., 1, :]
        if c.exclusive:
            if any(p.name == "kv" and p.mode != "write" for p in self.ports):
                raise ValueError("gqa(exclusive=...) takes the values the layer makes: not with its kv port read")
            out = exclusive(out, v, torch.tanh(self.xsa_alpha) if hasattr(self, "xsa_alpha") else None)
        if c.output_norm is not None:
            out = self.out_norm(out, ctx)
        if c.gated:
            out = (out.float() * self._gate(x, out, ctx)).to(out.dtype)
        out = out.reshape(bsz, t, self.h * self.dv)
        if c.output_dropout and ctx.training:
            out = nn.functional.dropout(out, c.output_dropout)
        return self.o(out, ctx)

    def _gate(self, x, out, ctx: Context):
        """The gate on the heads' outputs [b, t, h, dv or 1] in fp32
        (``attention/gqa.py:271-302`` there)."""
        c = self.c
        bsz, t = out.shape[:2]
        logits = self.gate(x, ctx).float().view(bsz, t, self.h, -1)
        if hasattr(self, "gate_up"):
            logits = torch.einsum("bthi,hio->btho", nn.functional.silu(logits), self.gate_up.float())
        if hasattr(self, "output_gate_down"):
            low = nn.functional.silu(torch.einsum("bthi,hio->btho", out.float(), self.output_gate_down.float()))
            logits = logits + torch.einsum("bthi,hio->btho", low, self.output_gate_up.float())
        if hasattr(self, "gate_bias"):
            logits = logits + self.gate_bias.float()[:, None]
        gate = ref.activation(logits, c.gate_activation)
        if hasattr(self, "cross_gate"):
            heads = torch.sigmoid(self.cross_gate(out.reshape(bsz, t, -1), ctx).float())
            gate = gate * heads.unsqueeze(-1)
        return gate


@register("gqa")
def _gqa(c, b):
    return GQA(c, b)
