"""Mixture of experts (``moe``): fp32 router, top-k, balance loss, sorted experts on
grouped GEMMs, optional shared experts; expert parallelism is delegated to
`bux_b200.parallel.experts` when the mesh has an ``expert`` axis.

Reference: ``architecture/experts/moe.py:69-1071``. Expert weights there are stacked
``(E, d, f, 2)`` (up, gate) and ``(E, f, d)``; here ``experts_gate_up`` is ``[E, 2f, d]``
(gate rows first) and ``experts_down`` is ``[E, d, f]``: the K-major operands of the
grouped tcgen05 GEMM. The checkpoint layer converts.
"""

from __future__ import annotations


import torch
from torch import nn

from ... import ops
from ...config import layers as L
from ...ops import reference as ref
from .. import placement
from ..registry import BuildContext, Context, register
from .basic import MLP, Linear, Norm, init_weight


def balance_loss(scores: torch.Tensor, picks: torch.Tensor, k: int, per_sequence: bool) -> torch.Tensor:
    """E · Σ_e f_e P_e (Switch / DeepSeek-V3): 1 when picks and scores are uniform."""
    over = (1,) if per_sequence else (0, 1)
    f = picks.float().mean(over) / k
    p = (scores / scores.sum(-1, keepdim=True)).mean(over)
    return scores.shape[-1] * (f * p).sum(-1).mean()


def budget_loss(scores: torch.Tensor, picks: torch.Tensor, c: L.MoEConfig, per_sequence: bool) -> torch.Tensor:
    """LongCat-Flash's balance loss with zero experts (reference:
    ``architecture/experts/moe.py:512-546``): Σ_j f_j P_j over the FFN experts and the zero
    experts as one more; 1 when the FFN experts take their budget of a token's picks evenly."""
    over = (1,) if per_sequence else (0, 1)
    n, budget = c.num_experts, c.ffn_budget
    count = picks.float().mean(over)
    p = (scores / scores.sum(-1, keepdim=True)).mean(over)
    f = n / budget * count[..., :n]
    f_zero = count[..., n:].sum(-1) / (c.top_k - budget)
    return ((f * p[..., :n]).sum(-1) + f_zero * p[..., n:].sum(-1)).mean()


def budget_move(load: torch.Tensor, c: L.MoEConfig) -> torch.Tensor:
    """The router-bias move with zero experts: each FFN expert by rate · (1 − load / target),
    target = its even share of the FFN budget; the zero experts' bias stays 0
    (``architecture/experts/moe.py:427-449`` there)."""
    n = c.num_experts
    target = c.ffn_budget * load.sum(-1, keepdim=True) / (c.top_k * n)
    picked = target > 0
    shortfall = torch.where(picked, 1 - load[..., :n] / torch.where(picked, target, torch.ones_like(target)),
                            torch.zeros_like(load[..., :n]))
    return torch.cat([c.bias_update_rate * shortfall, torch.zeros_like(load[..., n:])], -1)


def limit_groups(choice: torch.Tensor, groups: int, keep: int) -> torch.Tensor:
    b, t, n = choice.shape
    grouped = choice.view(b, t, groups, n // groups)
    best = grouped.topk(min(2, n // groups), dim=-1).values.sum(-1)
    kept_idx = best.topk(keep, dim=-1).indices
    kept = torch.zeros(b, t, groups, dtype=torch.bool, device=choice.device).scatter_(-1, kept_idx, True)
    return torch.where(kept.unsqueeze(-1), grouped, torch.full_like(grouped, float("-inf"))).view(b, t, n)


class _ScaleGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, share):
        ctx.share = share
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.share, None


class MoE(nn.Module):
    no_weight_decay = ("up_bias", "down_bias")   # stacks, but of vectors

    def __init__(self, c: L.MoEConfig, b: BuildContext):
        super().__init__()
        # plain MLP experts (one projection up, an activation, one down: Nemotron's relu² experts)
        # run the per-expert PyTorch statement of the layer; the kernels' path is the gated one
        self.gated = c.expert.type == "gated_mlp"
        self.c = c
        d = b.width if isinstance(b.width, int) else b.d_model
        e, f = c.num_experts, c.expert.intermediate_size
        scored = e + c.num_zero_experts  # the router scores the zero experts after the routed ones
        inner = c.latent_size or d       # the width the routed experts see (LatentMoE: narrower)
        self.d, self.e, self.f, self.inner = d, e, f, inner
        self.tp_share = 1.0
        self.router = Linear(d, scored + (c.num_shared_experts if c.shared_expert_sink else 0),
                             c.router_bias, b, role="router")
        self.router.weight.data = self.router.weight.data.float()
        if c.latent_size is not None:
            self.to_latent = Linear(d, inner, False, b, role="latent")
            self.from_latent = Linear(inner, d, False, b, role="latent")
        if c.latent_input_norm is not None:
            self.latent_input_norm = Norm(c.latent_input_norm, inner)
        if c.latent_output_norm is not None:
            self.latent_output_norm = Norm(c.latent_output_norm, inner)
        if c.expert_norm is not None:
            self.expert_norm = Norm(c.expert_norm, inner)
        self.experts_gate_up = nn.Parameter(torch.empty(e, (2 if self.gated else 1) * f, inner, dtype=b.dtype))
        self.experts_down = nn.Parameter(torch.empty(e, inner, f, dtype=b.dtype))
        if c.expert.bias:
            # one bias vector per expert and projection: stacks, but of vectors (no weight decay)
            self.up_bias = nn.Parameter(torch.zeros(e, (2 if self.gated else 1) * f, dtype=b.dtype))
            self.down_bias = nn.Parameter(torch.zeros(e, inner, dtype=b.dtype))
        init_weight(self.experts_gate_up, b.init)
        rows = placement.expert_rows(e)   # under expert parallelism: this rank's experts only
        if rows is not None:
            self.experts_gate_up = placement.keep_rows(self.experts_gate_up, rows)
        init_weight(self.experts_down, b.init, "out")
        if rows is not None:
            self.experts_down = placement.keep_rows(self.experts_down, rows)
        if c.load_balancing in ("aux_free", "smebu"):
            self.register_buffer("router_bias", torch.zeros(scored))
            self.register_buffer("router_load", torch.zeros(scored))
            self.register_buffer("bias_velocity", torch.zeros(e))
        if c.num_shared_experts:
            sc = c.shared_expert or c.expert
            sc = sc.model_copy(update={"intermediate_size": sc.intermediate_size * c.num_shared_experts})
            self.shared = MLP(sc, d, b, role="mlp")
            if c.shared_expert_gate:
                self.shared_gate = Linear(d, 1, False, b, role="router")
        self.ep = None  # set by the parallel layer when experts are split over ranks

    # ------------------------------------------------------------------ routing
    def route(self, x: torch.Tensor, ctx: Context):
        c = self.c
        logits = ops.linear_f32(x, self.router.weight, self.router.bias)
        logits = logits * c.router_logit_scale
        if c.random_logits and ctx.training:
            drawn = torch.randn_like(logits)
            logits = drawn + (logits - logits.detach())
        scores = ref.router_scores(logits, c.router)
        n = c.num_experts + c.num_zero_experts
        scores, sinks = scores[..., :n], scores[..., n:]
        choice = scores
        if hasattr(self, "router_bias"):
            choice = scores + self.router_bias
        if c.num_groups > 1:
            choice = limit_groups(choice, c.num_groups, c.top_k_groups)
        if ops.kernels_on(x) and choice.shape[-1] <= 512:
            from ...ops import kernels as K

            idx = K.topk_rows(choice.detach().float(), c.top_k)  # picks carry no gradient: a plain kernel
        else:
            idx = choice.topk(c.top_k, dim=-1).indices
        if ctx.training:
            picks = torch.zeros_like(scores).scatter_add_(-1, idx, torch.ones_like(idx, dtype=scores.dtype))
            w = c.aux_loss_weight
            if w:
                # under tensor parallelism every rank reports the same loss: each gives 1/n of its gradient
                seen = scores if self.tp_share == 1.0 else _ScaleGrad.apply(scores, self.tp_share)
                per_sequence = c.aux_loss_scope == "sequence"
                loss = (budget_loss(seen, picks, c, per_sequence) if c.num_zero_experts
                        else balance_loss(seen, picks, c.top_k, per_sequence))
                ctx.report("balance_loss", loss, w)
            if hasattr(self, "router_load"):
                self.router_load += picks.detach().sum((0, 1))
        if ctx.observing:
            from .. import observe

            observe.router(ctx, logits[..., :n], idx, n, getattr(self, "router_bias", None))
        weights = scores.gather(-1, idx)
        if c.normalize_top_k:
            total = weights.sum(-1, keepdim=True) + sinks.sum(-1, keepdim=True)
            weights, sinks = weights / total, sinks / total
        weights = weights * c.routed_scaling_factor
        return idx, weights, (sinks * c.routed_scaling_factor if sinks.shape[-1] else None)

    @torch.no_grad()
    def step_end_update(self) -> None:
        """Aux-loss-free balancing (DeepSeek-V3): nudge the selection bias of over- and
        under-loaded experts once per step, from the picks counted since the last one."""
        if not hasattr(self, "router_bias"):
            return
        c = self.c
        load = self.router_load
        if load.sum() == 0:
            return
        if c.num_zero_experts:
            self.router_bias.add_(budget_move(load, c))
            load.zero_()
            return
        err = load.mean() - load
        if c.load_balancing == "smebu":
            # each expert's shortfall of the mean load as a fraction of the mean, soft-clamped by
            # tanh(kappa .), times the rate, centred over the experts; the bias moves by the moves'
            # running average (``architecture/experts/moe.py:365-375,407-425`` there)
            mean = load.mean()
            shortfall = err / torch.where(mean > 0, mean, torch.ones_like(mean))
            move = c.bias_update_rate * torch.tanh(c.bias_softclamp * shortfall)
            move = move - move.mean()
            self.bias_velocity.mul_(c.bias_momentum).add_(move, alpha=1 - c.bias_momentum)
            self.router_bias.add_(self.bias_velocity)
        else:
            self.router_bias.add_(torch.sign(err), alpha=c.bias_update_rate)
            if c.center_bias:
                self.router_bias.sub_(self.router_bias.mean())
        load.zero_()

    # ------------------------------------------------------------------ forward
    def forward(self, x, ctx: Context):
        c = self.c
        bsz, t, d = x.shape
        idx, weights, sinks = self.route(x, ctx)
        z = x
        if c.latent_size is not None:
            z = self.to_latent(x, ctx)
        if c.latent_input_norm is not None:
            z = self.latent_input_norm(z, ctx)
        inner = z.shape[-1]
        flat = z.reshape(bsz * t, inner)
        fmt = ctx.precision.of("experts")
        ec = c.expert
        w_ffn, idx_ffn = weights, idx
        if c.num_zero_experts:
            # a zero expert is the token itself times its weight; its picks run no FFN (they
            # are handed to a routed expert with weight 0, which leaves the sum unchanged)
            if self.ep is not None:
                raise NotImplementedError("moe: zero experts under expert parallelism")
            is_zero = idx >= c.num_experts
            w_ffn = torch.where(is_zero, torch.zeros_like(weights), weights)
            idx_ffn = torch.where(is_zero, idx - c.num_experts, idx) % c.num_experts
        if self.ep is not None:
            if c.expert_norm is not None:
                raise NotImplementedError("moe: expert_norm under expert parallelism")
            if not self.gated:
                raise NotImplementedError("moe: plain MLP experts under expert parallelism")
            if ec.up_softcap is not None:
                raise NotImplementedError("moe: experts with up_softcap under expert parallelism")
            if ec.bias:
                raise NotImplementedError("moe: experts with biases under expert parallelism")
            out = self.ep(self, flat, w_ffn.reshape(bsz * t, -1), idx_ffn.reshape(bsz * t, -1), ctx, fmt)
        elif c.expert_norm is not None or not self.gated or ec.up_softcap is not None or ec.bias:
            # each expert's output is normalised before the weighted sum (the rows are needed one
            # by one), the experts are plain MLPs, their up branch is soft-capped or they have
            # biases (the kernels have neither): the per-expert statement of the layer
            norm = (lambda rows: self.expert_norm(rows, ctx)) if c.expert_norm is not None else None
            out = ops.moe_reference(flat, self.experts_gate_up, self.experts_down,
                                          w_ffn.reshape(bsz * t, -1), idx_ffn.reshape(bsz * t, -1),
                                          ec.activation, ec.limit, ec.up_offset, row_fn=norm, gated=self.gated,
                                          up_softcap=ec.up_softcap,
                                          up_bias=getattr(self, "up_bias", None),
                                          down_bias=getattr(self, "down_bias", None))
        else:
            out = ops.moe_experts(flat, self.experts_gate_up, self.experts_down,
                                  w_ffn.reshape(bsz * t, -1), idx_ffn.reshape(bsz * t, -1),
                                  act=ec.activation, limit=ec.limit, up_offset=ec.up_offset, fmt=fmt,
                                  chunks=getattr(ctx.methods, "moe_chunks", 1) if ctx.methods is not None else 1)
        out = out.view(bsz, t, inner)
        if c.num_zero_experts:
            zero = torch.where(is_zero, weights, torch.zeros_like(weights)).sum(-1, keepdim=True)
            out = out + (z.float() * zero).to(out.dtype)
        if c.latent_output_norm is not None:
            out = self.latent_output_norm(out, ctx)
        if c.latent_size is not None:
            out = self.from_latent(out, ctx)
        if c.num_shared_experts:
            if sinks is not None:
                # the router scores the shared experts too: each one's share of the hidden units
                # is weighted by its own score (``architecture/experts/moe.py:390-404`` there)
                f = self.shared.c.intermediate_size // sinks.shape[-1]
                if getattr(self.shared, "f_local", self.shared.c.intermediate_size) != self.shared.c.intermediate_size \
                        and sinks.shape[-1] > 1:
                    raise NotImplementedError("moe(shared_expert_sink=true) with several shared experts under tensor parallelism")
                shared = self.shared(x, ctx, hidden_scale=sinks.float().repeat_interleave(f, dim=-1))
            else:
                shared = self.shared(x, ctx)
            if c.shared_expert_gate:
                shared = (shared.float() * torch.sigmoid(self.shared_gate(x, ctx).float())).to(shared.dtype)
            out = out + shared
        return out


@register("moe")
def _moe(c, b):
    return MoE(c, b)
