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
from .basic import Linear, Norm

_UNSUPPORTED = ("kv_conv_size", "differential", "paired", "k_eq_v", "power_scale", "log_scale",
                "relative_bias", "gate_input_rank", "gate_output_rank", "gate_cross_head")


class GQA(nn.Module):
    def __init__(self, c: L.GQAConfig, b: BuildContext):
        super().__init__()
        for name in _UNSUPPORTED:
            v = getattr(c, name)
            if v not in (None, False):
                raise NotImplementedError(f"gqa({name}=...) is not built in this framework yet")
        if c.exclusive:
            raise NotImplementedError("gqa(exclusive=...) is not built in this framework yet")
        self.c = c
        width = b.width if isinstance(b.width, int) else b.d_model
        self.h, self.g = c.num_heads, c.num_kv_heads
        self.d = c.head_dim or width // c.num_heads
        self.dv = c.v_head_dim or self.d
        self.q_rows, self.k_rows, self.v_rows = self.h * self.d, self.g * self.d, self.g * self.dv
        self.qkv = Linear(width, self.q_rows + self.k_rows + self.v_rows, c.bias, b, role="q")
        out_bias = c.bias if c.output_bias is None else c.output_bias
        self.o = Linear(self.h * self.dv, width, out_bias, b, role="o", init_role="out")
        if c.qk_norm is not None:
            per = self.d
            self.q_norm = Norm(c.qk_norm, self.h * per if c.qk_norm_all_heads else per)
            self.k_norm = Norm(c.qk_norm, self.g * per if c.qk_norm_all_heads else per)
        if c.sinks:
            self.sinks = nn.Parameter(torch.zeros(self.h))
        if c.gated:
            gate_out = self.h if c.gate_per_head else self.h * self.dv
            self.gate = Linear(width, gate_out, c.gate_head_bias, b, role="q")
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

    def forward(self, x, ctx: Context):
        c = self.c
        qkv = self.qkv(x, ctx)
        bsz, t = qkv.shape[:2]  # with the sequence gathered inside the projection, longer than x
        q, k, v = qkv.split((self.q_rows, self.k_rows, self.v_rows), dim=-1)  # backward: one cat
        q = q.reshape(bsz, t, self.h, self.d)
        k = k.reshape(bsz, t, self.g, self.d)
        v = v.reshape(bsz, t, self.g, self.dv)
        for port in self.ports:  # value residual / kv sharing through taps
            if port.name == "v" and port.mode != "write":
                v = 0.5 * (v + ctx.read(port.tap, port.mode == "pop"))
            elif port.name == "kv" and port.mode != "write":
                k, v = ctx.read(port.tap, port.mode == "pop")
            elif port.name == "ve" and port.mode != "write":  # value embeddings join the values
                v = v + ctx.read(port.tap, port.mode == "pop").reshape(v.shape).to(v.dtype)
        q = self._norm_rope(q, getattr(self, "q_norm", None), ctx)
        kv_shared = any(p.name == "kv" and p.mode != "write" for p in self.ports)
        if not kv_shared:
            k = self._norm_rope(k, getattr(self, "k_norm", None), ctx)
        for port in self.ports:
            if port.mode == "write":
                ctx.push(port.tap, v if port.name == "v" else (k, v))
        if c.indexer is not None:
            out = self._sparse(x, q, k, v, ctx)
            return self._finish(out, x, bsz, t, ctx)
        kw = dict(causal=True, window=c.sliding_window_size, sinks=getattr(self, "sinks", None),
                  softcap=c.softcap, scale=c.scale, segments=ctx.segments)
        cp = getattr(ctx.parallel, "context_group", None) if ctx.parallel is not None else None
        if cp is not None:
            from ...parallel import context

            out = context.attend(ops.attention, q, k, v, cp, ctx.methods.attention, **kw)
        else:
            out = ops.attention(q, k, v, **kw)
        return self._finish(out, x, bsz, t, ctx)

    def _sparse(self, x, q, k, v, ctx: Context):
        """Attention over the keys an indexer kept (its own, or another layer's through
        the ``index`` port), and the indexer's distillation loss."""
        from . import sparse as S

        c = self.c
        t = q.shape[1]
        seen = S.seen_mask(ctx, t, c.sliding_window_size)
        reads = [p for p in self.ports if p.name == "index" and p.mode != "write"]
        scores = None
        if reads:
            kept = ctx.read(reads[0].tap, reads[0].mode == "pop") & seen
        else:
            scores = self.indexer.scores(x, ctx)
            kept = S.top_mask(scores, seen, c.indexer.top_k)
        for p in self.ports:
            if p.name == "index" and p.mode == "write":
                ctx.push(p.tap, kept)
        out, target = S.attend_kept(q, k, v, kept, c.scale, getattr(self, "sinks", None), c.softcap)
        if scores is not None and ctx.training and c.indexer.loss_weight:
            ctx.report("indexer_loss", S.indexer_loss(scores, kept, target), c.indexer.loss_weight)
        return out

    def _finish(self, out, x, bsz, t, ctx: Context):
        c = self.c
        if c.output_norm is not None:
            out = self.out_norm(out, ctx)
        out = out.reshape(bsz, t, self.h * self.dv)
        if c.gated:
            gate = ref.activation(self.gate(x, ctx).float(), c.gate_activation)
            if c.gate_per_head:
                gate = gate.repeat_interleave(self.dv, dim=-1)
            out = (out.float() * gate).to(out.dtype)
        if c.output_dropout and ctx.training:
            out = nn.functional.dropout(out, c.output_dropout)
        return self.o(out, ctx)


@register("gqa")
def _gqa(c, b):
    return GQA(c, b)
