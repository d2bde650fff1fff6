"""Embedding, LM head, norms, MLPs and the small elementwise layers.

Weights are stored ``[out, in]`` (what the tcgen05 GEMMs read K-major); checkpoints
and exports keep the reference's ``kernel`` orientation ``[in, out]`` by transposing at
the boundary (`bux_b200.ckpt`). Attribute names follow the reference modules
(``architecture/layers/embedding.py:39-251``, ``norm.py:25``, ``mlp.py:45``,
``elementwise.py``): ``tokens.embedding``, ``proj``, ``up / gate / down``, ``scale``.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ... import ops
from ...config import layers as L
from ...ops import reference as ref
from .. import placement
from ..registry import BuildContext, Context, register


# ------------------------------------------------------------------ init
def init_weight(t: torch.Tensor, init, role: str = "hidden", fan_in: Optional[int] = None,
                fan_out: Optional[int] = None) -> None:
    """Fill a weight in place per the model's ``init`` (None = normal(0.02)); `role` in
    embed / head / out / hidden picks a per-role override."""
    cfg = init if init is not None else L.NormalInitConfig()
    if role != "hidden" and getattr(cfg, role, None) is not None:
        cfg = getattr(cfg, role)
    with torch.no_grad():
        if cfg.type == "zeros":
            t.zero_()
        elif cfg.type == "normal":
            if cfg.truncate is None:
                t.normal_(0.0, cfg.std)
            else:
                nn.init.trunc_normal_(t, 0.0, cfg.std, -cfg.truncate * cfg.std, cfg.truncate * cfg.std)
        else:
            fi = fan_in if fan_in is not None else t.shape[-1]
            fo = fan_out if fan_out is not None else t.shape[0]
            fan = {"fan_in": fi, "fan_out": fo, "fan_avg": (fi + fo) / 2}[cfg.type]
            var = cfg.scale / max(1.0, fan)
            if cfg.distribution == "gaussian":
                t.normal_(0.0, math.sqrt(var))
            elif cfg.distribution == "uniform":
                lim = math.sqrt(3 * var)
                t.uniform_(-lim, lim)
            else:
                std = math.sqrt(var) / 0.87962566103423978
                nn.init.trunc_normal_(t, 0.0, std, -2 * std, 2 * std)


class Linear(nn.Module):
    """y = x·W^T (+ b), W [out, in]; `role` names the matmul format it multiplies in."""

    def __init__(self, fan_in: int, fan_out: int, bias: bool, bctx: BuildContext,
                 role: str = "mlp", init_role: str = "hidden"):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(fan_out, fan_in, dtype=bctx.dtype))
        init_weight(self.weight, bctx.init, init_role)
        self.weight = placement.place_dense(self.weight)   # under sharded parameters: this rank's rows only
        self.bias = nn.Parameter(torch.zeros(fan_out, dtype=bctx.dtype)) if bias else None
        self.role = role
        self.tp_fused = None  # (kind, group, reorder) when the tensor-parallel collective runs in the GEMM

    def forward(self, x, ctx: Optional[Context] = None):
        if self.tp_fused is not None and ops.kernels_on(x) and x.dtype == torch.bfloat16:
            from ...parallel import tensor_fused as TF

            kind, group, reorder = self.tp_fused
            if kind == "gather":
                return TF.gather_matmul(x, self.weight, group, reorder)
            return TF.matmul_scatter(x, self.weight, group, ctx.input_ids.shape[0] if ctx is not None else x.shape[0],
                                     reorder)
        if ctx is None:
            return ops.linear(x, self.weight, self.bias)
        return ops.linear(x, self.weight, self.bias, fmt=ctx.precision.of(self.role), passes=ctx.precision.passes)


# ------------------------------------------------------------------ norms
class Norm(nn.Module):
    def __init__(self, c: L.NormalizationConfig, width: int):
        super().__init__()
        self.c = c
        init = c.gain_init - 1.0 if c.zero_centered else c.gain_init   # the gain 1 + w starts at gain_init too
        self.scale = nn.Parameter(torch.full((width,), float(init))) if c.affine else None
        self.bias = nn.Parameter(torch.zeros(width)) if c.bias else None

    def forward(self, x, ctx: Optional[Context] = None):
        c = self.c
        if c.scale_input and self.scale is not None:
            # the gain goes on before the statistics, norm(w * x), and not after
            # (``architecture/layers/norm.py:59-67`` there)
            gain = (1.0 + self.scale.float()) if c.zero_centered else self.scale.float()
            x = (x.float() * gain).to(x.dtype)
            y = ref.rmsnorm(x, None, c.eps) if c.type == "rmsnorm" else ref.layernorm(x, None, None, c.eps)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        if c.type == "rmsnorm":
            y = ops.rmsnorm(x, self.scale, c.eps, c.zero_centered)
            return y if self.bias is None else y + self.bias.to(y.dtype)
        return ref.layernorm(x, self.scale, self.bias, c.eps, c.zero_centered)


@register("rmsnorm", "layernorm")
def _norm(c, b: BuildContext):
    return Norm(c, b.width if isinstance(b.width, int) else b.d_model)


class DyT(nn.Module):
    def __init__(self, c: L.DyTConfig, width: int):
        super().__init__()
        self.alpha = nn.Parameter(torch.tensor(float(c.alpha_init)))
        self.scale = nn.Parameter(torch.ones(width))
        self.bias = nn.Parameter(torch.zeros(width))

    def forward(self, x, ctx=None):
        y = torch.tanh(self.alpha * x.float()) * self.scale + self.bias
        return y.to(x.dtype)


@register("dyt")
def _dyt(c, b):
    return DyT(c, b.width if isinstance(b.width, int) else b.d_model)


# ------------------------------------------------------------------ embedding / head
class TokenTable(nn.Module):
    no_muon = True

    def __init__(self, vocab: int, width: int, bctx: BuildContext):
        super().__init__()
        self.embedding = nn.Parameter(torch.empty(vocab, width, dtype=bctx.dtype))
        init_weight(self.embedding, bctx.init, "embed", fan_in=width, fan_out=width)
        self.embedding = placement.place_dense(self.embedding)


class Embedding(nn.Module):
    no_muon = True

    def __init__(self, c: L.EmbeddingConfig, b: BuildContext):
        super().__init__()
        self.c = c
        self.tokens = TokenTable(b.vocab_size, b.d_model, b)
        if c.max_positions is not None:
            self.positions = nn.Parameter(torch.empty(c.max_positions, b.d_model, dtype=b.dtype))
            init_weight(self.positions, b.init, "embed")
        self.norm = Norm(c.norm, b.d_model) if c.norm is not None else None
        self.scale = math.sqrt(b.d_model) if c.scale_by_sqrt_dim else None
        self.dropout = c.dropout
        from ..residual import widening

        self.widen = widening(b.residual)

    def embed_tokens(self, ids, ctx: Context):
        """A token's row, scaled by sqrt(d) and normalised where the layer says so: what `nextn`
        reads too (``architecture/layers/embedding.py:78-81`` there)."""
        x = self.tokens.embedding[ids]
        if x.dtype != ctx.precision.compute:
            x = x.to(ctx.precision.compute)
        if self.scale is not None:
            x = x * self.scale
        return x if self.norm is None else self.norm(x, ctx)

    def forward(self, ids, ctx: Context):
        x = self.embed_tokens(ctx.input_ids, ctx)
        if self.c.max_positions is not None:   # after the norm: positions are added to the normalised rows
            x = x + self.positions[ctx.positions].to(x.dtype)
        if self.dropout and ctx.training:
            x = nn.functional.dropout(x, self.dropout)
        if self.widen is not None:  # the residual algebra's widened stream starts as copies
            x = x.unsqueeze(2).expand(-1, -1, self.widen, -1).contiguous()
        return x


@register("embed")
def _embed(c, b):
    return Embedding(c, b)


class HeadOutput:
    """What a head leaves for the objective: hidden states and the matrix that turns
    them into logits, so the loss can be computed without materialising the logits."""

    def __init__(self, hidden, weight, bias=None, softcap=None, name="head"):
        self.hidden, self.weight, self.bias, self.softcap, self.name = hidden, weight, bias, softcap, name
        self.pointer = None  # a copy pointer's view (`layers.pointer.PointerView`): the loss is then the mixture's

    def logits(self) -> torch.Tensor:
        out = nn.functional.linear(self.hidden, self.weight.to(self.hidden.dtype),
                                   None if self.bias is None else self.bias.to(self.hidden.dtype))
        if self.softcap:
            out = self.softcap * torch.tanh(out / self.softcap)
        return out


class Head(nn.Module):
    no_muon = True

    def __init__(self, c: L.LMHeadConfig, b: BuildContext):
        super().__init__()
        self.c = c
        self.tied_to = None
        if c.tied:
            if b.embedding is None:
                raise ValueError("a tied head needs an embedding before it")
            object.__setattr__(self, "tied_to", b.embedding)  # not a submodule: no duplicate path
        else:
            self.proj = Linear(b.width if isinstance(b.width, int) else b.d_model, b.vocab_size,
                               False, b, role="head", init_role="head")
        self.bias = nn.Parameter(torch.zeros(b.vocab_size)) if c.bias else None
        if c.pointer is not None:
            from .pointer import CopyPointer

            self.pointer = CopyPointer(c.pointer, b.width if isinstance(b.width, int) else b.d_model,
                                       b.vocab_size, b)

    def matrix(self) -> torch.Tensor:
        return self.tied_to.tokens.embedding if self.tied_to is not None else self.proj.weight

    def forward(self, x, ctx: Context):
        out = HeadOutput(x, self.matrix(), self.bias, self.c.softcap, name=f"head{len(ctx.heads)}")
        if hasattr(self, "pointer") and not ctx.heads:  # the pass's first head carries the pointer
            out.pointer = self.pointer(x, ctx)
        ctx.heads.append(out)
        return x  # the stream goes on (multi-token prediction stacks more heads after it)


@register("head")
def _head(c, b):
    return Head(c, b)


# ------------------------------------------------------------------ MLP
class MLP(nn.Module):
    """``mlp``: down(act(up(x))). ``gated_mlp``: down(act(gate(x)) * up(x)); gate and up
    are one fused [2f, d] matrix (gate rows first) so one GEMM feeds the GLU kernel."""

    def __init__(self, c: L.MLPConfig, width: int, b: BuildContext, role: str = "mlp"):
        super().__init__()
        self.c = c
        f = c.intermediate_size
        self.gated = c.type == "gated_mlp"
        if self.gated:
            self.gate_up = Linear(width, 2 * f, c.bias, b, role=role)
        else:
            self.up = Linear(width, f, c.bias, b, role=role)
        self.down = Linear(f, width, c.bias, b, role=role, init_role="out")

    def forward(self, x, ctx: Optional[Context] = None, hidden_scale=None):
        """`hidden_scale` ([..., f], optional) multiplies the hidden units before the down
        projection (an MoE's shared experts weighted by the router)."""
        c = self.c
        if self.gated:
            h = self.gate_up(x, ctx)
            if c.up_softcap is not None:
                # the up branch is clipped to +-limit, then soft-capped; the gate is capped from
                # above only (``architecture/layers/mlp.py:28-35`` there)
                f = getattr(self, "f_local", c.intermediate_size)
                up = h[..., f:].float()
                if c.limit is not None:
                    up = up.clamp(-c.limit, c.limit)
                up = c.up_softcap * torch.tanh(up / c.up_softcap)
                h = torch.cat((h[..., :f], up.to(h.dtype)), dim=-1)
            a = ops.glu(h, c.activation, None, c.limit, c.up_offset)
        else:
            h = self.up(x, ctx).float()
            if c.limit is not None:
                h = h.clamp(-c.limit, c.limit)
            if c.up_softcap is not None:
                h = c.up_softcap * torch.tanh(h / c.up_softcap)
            a = ref.activation(h, c.activation).to(x.dtype)
        if hidden_scale is not None:
            a = (a.float() * hidden_scale).to(a.dtype)
        y = self.down(a, ctx)
        if c.dropout and ctx is not None and ctx.training:   # of the output (``architecture/layers/mlp.py:88`` there)
            y = nn.functional.dropout(y, c.dropout)
        return y


@register("mlp", "gated_mlp")
def _mlp(c, b):
    return MLP(c, b.width if isinstance(b.width, int) else b.d_model, b)


# ------------------------------------------------------------------ elementwise
class LinearLayer(nn.Module):
    def __init__(self, c: L.LinearConfig, b: BuildContext):
        super().__init__()
        width = b.width if isinstance(b.width, int) else b.d_model
        self.proj = Linear(width, c.features, c.bias, b)

    def forward(self, x, ctx=None):
        return self.proj(x, ctx)


@register("linear")
def _linear(c, b):
    return LinearLayer(c, b)


class Act(nn.Module):
    def __init__(self, fn: str):
        super().__init__()
        self.fn = fn

    def forward(self, x, ctx=None):
        return ref.activation(x.float(), self.fn).to(x.dtype)


@register("act")
def _act(c, b):
    return Act(c.fn)


class Scale(nn.Module):
    def __init__(self, c: L.ScaleConfig, width: int):
        super().__init__()
        shape = (width,) if c.per_channel else ()
        self.scale = nn.Parameter(torch.full(shape, float(c.init)))

    def forward(self, x, ctx=None):
        return (x.float() * self.scale).to(x.dtype)


@register("scale")
def _scale(c, b):
    return Scale(c, b.width if isinstance(b.width, int) else b.d_model)


class Dropout(nn.Module):
    def __init__(self, rate: float):
        super().__init__()
        self.rate = rate

    def forward(self, x, ctx=None):
        if ctx is not None and ctx.training and self.rate > 0:
            return nn.functional.dropout(x, self.rate)
        return x


@register("dropout")
def _dropout(c, b):
    return Dropout(c.rate)
