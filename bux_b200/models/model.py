"""`Model`: an `ir.Architecture` built into modules, and its forward.

Reference: ``architecture/model.py:18-167`` (`Model`, `num_params`, `active_params`).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..lang import ir
from .graph import GraphBuilder, Repeated
from .registry import Context, Precision


def mark_exemptions(model: nn.Module) -> None:
    """Carry what a module's class says about its parameters onto the parameters themselves,
    where the optimizer reads it: the names in a class's ``no_weight_decay`` are skipped by
    weight decay whatever their rank (stacks of vectors, decay rates, lookup tables), and every
    parameter under a ``no_muon`` class is left to AdamW. Reference: ``train/optim.py:345-349,
    423-428``."""
    for module in model.modules():
        for name in getattr(type(module), "no_weight_decay", ()):
            p = module._parameters.get(name)
            if p is not None:
                p.no_weight_decay = True
        if getattr(type(module), "no_muon", False):
            for p in module.parameters():
                p.no_muon = True


class Model(nn.Module):
    """``Model(arch)(input_ids)`` runs the graph and returns the forward's `Context`:
    ``ctx.heads`` holds every head's `HeadOutput` (hidden states + output matrix, the
    logits are left to the loss), ``ctx.losses`` the auxiliary losses layers reported."""

    def __init__(self, arch: ir.Architecture, dtype: torch.dtype = torch.float32, seed: int = 0,
                 device=None):
        super().__init__()
        self.arch = arch
        self.dtype = dtype
        gen_state = torch.random.get_rng_state()
        torch.manual_seed(seed)
        try:
            with torch.device(device) if device is not None else _null():
                self.graph = GraphBuilder(arch, dtype).build(arch.graph)
        finally:
            torch.random.set_rng_state(gen_state)
        mark_exemptions(self)

    def forward(self, input_ids: torch.Tensor, positions: Optional[torch.Tensor] = None,
                segments: Optional[torch.Tensor] = None, *, training: Optional[bool] = None,
                precision: Optional[Precision] = None, methods=None, parallel=None,
                step: int = 0, observe: Optional[dict] = None, cache=None) -> Context:
        """`cache` (a `bux_b200.models.cache.DecodeCache`): the tokens continue what it holds;
        `segments` then marks padding (0) against real tokens (non-zero), nothing else."""
        ctx = Context(input_ids, positions, segments,
                      training=self.training if training is None else training,
                      precision=precision or Precision(compute=self.dtype), methods=methods,
                      parallel=parallel, step=step)
        if observe is not None:   # an observed step: layers file their statistics in ctx.observed
            ctx.observing = True
            ctx.observe_histograms = bool(observe.get("histograms"))
        if cache is not None:
            real = torch.ones_like(input_ids, dtype=torch.bool) if segments is None else segments != 0
            cache.begin(real)
            ctx.cache = cache
            # padding as a document of its own: recurrences restart and convolutions drop their
            # taps at each row's first real token; attention reads the cache's own marks
            ctx.segments = None if bool(real.all()) else real.to(torch.int32)
        ctx.output = self.graph(input_ids, ctx)
        return ctx

    def logits(self, input_ids, **kw) -> torch.Tensor:
        """Logits of the first head: for tests and small-scale inspection."""
        ctx = self(input_ids, **kw)
        return ctx.heads[0].logits()

    def set_remat(self, on: bool, offload: bool = False, keep_attention=False, kept_to_host: bool = False,
                  first=None) -> None:
        """Checkpoint every pass of every repeated block (keep only its input, rerun it
        in the backward); `offload` keeps those inputs in pinned host memory;
        `keep_attention` also keeps each attention's output and log-sum-exp, so the rerun
        skips the attention forward kernel (the remat preset that keeps ``attention.out``):
        True for every pass, or a number for the last so many passes of each repeat. Kept
        outputs stay on the device unless `kept_to_host` sends them after the inputs. With
        `first`, only the first so many passes of each repeat are checkpointed."""
        for m in self.modules():
            if isinstance(m, Repeated):
                m.remat = on
                m.offload = offload
                m.keep_attention = keep_attention if on else False
                m.kept_to_host = kept_to_host
                m.first = first

    def step_end_update(self) -> None:
        for m in self.modules():
            fn = getattr(m, "step_end_update", None)
            if fn is not None and m is not self:
                fn()

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def active_params(self) -> int:
        """Parameters a token passes through: routed experts count top_k / num_experts."""
        from .layers.moe import MoE

        total = self.num_params()
        for m in self.modules():
            if isinstance(m, MoE):
                routed = m.experts_gate_up.numel() + m.experts_down.numel()
                total -= routed - routed * m.c.top_k // m.c.num_experts
        return total


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
