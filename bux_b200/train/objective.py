"""The training objective: next-token cross-entropy of every head (+ z-loss, weighted
multi-token-prediction heads) plus the auxiliary losses layers report.

Losses are kept as (sum over target tokens, target count) so that microbatches and
ranks add up to the whole batch's mean exactly; the caller divides by the global
count (a device scalar, so nothing synchronises).

Reference: ``train/objective.py:53-477`` (`Heads`, `Objective`, `target_mask`).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..config import training as T


def targets_and_mask(input_ids: torch.Tensor, position_ids: torch.Tensor, loss_mask: torch.Tensor,
                     shift: int = 1):
    """Position t predicts token t+shift where that token is a target and still in t's
    document (positions keep increasing). Returned full-width: the last `shift` columns
    are masked instead of sliced off, so hidden states need no copy."""
    tgt = torch.roll(input_ids, -shift, dims=1)
    nxt_pos = torch.roll(position_ids, -shift, dims=1)
    mask = torch.roll(loss_mask, -shift, dims=1).clone()
    mask &= nxt_pos == position_ids + shift
    mask[:, -shift:] = False
    return tgt, mask


@dataclass
class LossParts:
    total_sum: torch.Tensor            # Σ over targets of everything per-token (differentiable)
    count: torch.Tensor                # number of targets of the first head
    ce_sum: torch.Tensor               # first head's CE alone (for logging)
    per_batch: torch.Tensor            # per-batch terms (aux losses), already weighted
    terms: dict = field(default_factory=dict)


def prefix_weight(c: T.PrefixConfig, share: float) -> float:
    """Prefix-token prediction's weight at `share` of the run's steps: its weight for the
    first `hold` of them, falling linearly to 0 over the next `decay`, then 0
    (``train/objective.py:309-318`` there)."""
    if share <= c.hold:
        return c.weight
    if c.decay == 0:
        return 0.0
    return c.weight * min(1.0, max(0.0, 1 - (share - c.hold) / c.decay))


def compute(ctx, batch, loss_cfg: T.LossConfig, span=None, prefixes=None, progress: float = 0.0) -> LossParts:
    """Loss of one forward `ctx` on `batch` = (input_ids, position_ids, loss_mask). With
    `span` = (start, stop) the forward saw only those positions of the rows (context
    parallelism): targets come from the whole rows, then the span is taken. With
    ``loss(prefix=...)``, `prefixes` (int tensor [vocab]: each id's prefix token, -1 for none)
    adds the first head's cross-entropy of every target's prefix token, weighted by the
    schedule at `progress` (the share of the run's steps done); it is reported unweighted as
    ``prefix_loss``."""
    ids, pos, lmask = batch
    dev = ids.device
    total = torch.zeros((), dtype=torch.float32, device=dev)
    ce0 = None
    count0 = None
    terms: dict = {}
    for k, head in enumerate(ctx.heads):
        shift = k + 1 if k > 0 else 1  # head k>0 is an MTP head looking k+1 ahead
        tgt, mask = targets_and_mask(ids, pos, lmask, shift)
        if span is not None:
            tgt, mask = tgt[:, span[0]:span[1]], mask[:, span[0]:span[1]]
        h = head.hidden.reshape(-1, head.hidden.shape[-1])
        if getattr(head, "pointer", None) is not None:
            if span is not None:
                raise NotImplementedError("a copy pointer with positions split over ranks")
            ce0, count0 = head.pointer.sums(head, tgt, mask, loss_cfg.z)
            total = total + ce0
            continue
        s, n = ops.cross_entropy_head(h, head.weight, tgt.reshape(-1), mask.reshape(-1).float(),
                                      bias=head.bias, z_weight=loss_cfg.z if k == 0 else 0.0,
                                      softcap=head.softcap)
        if k == 0:
            ce0, count0 = s, n
            total = total + s
            if loss_cfg.prefix is not None and prefixes is not None:
                # the same hidden states against each target's prefix token, where it has one;
                # a mean over all the targets, as the cross-entropy itself
                ptgt = prefixes.to(tgt.device)[tgt.reshape(-1).long()]
                pmask = mask.reshape(-1) & (ptgt >= 0)
                ps, _ = ops.cross_entropy_head(h, head.weight, ptgt.clamp_min(0), pmask.float(), bias=head.bias,
                                               softcap=head.softcap)
                terms["prefix_loss"] = (ps / n.clamp_min(1.0)).detach()
                w = prefix_weight(loss_cfg.prefix, progress)
                if w > 0:
                    total = total + w * ps
        else:
            # an MTP head's mean loss, weighted, spread over the first head's tokens
            w = loss_cfg.mtp / max(1, len(ctx.heads) - 1)
            total = total + w * s * (count0 / n.clamp_min(1.0))
            terms[f"mtp{k}_loss"] = (s / n.clamp_min(1.0)).detach()
    per_batch = torch.zeros((), dtype=torch.float32, device=dev)
    for name, value in ctx.losses.items():
        per_batch = per_batch + value.float()
        terms[name] = value.detach()
    if ce0 is None:
        raise ValueError("the model has no head, so there is nothing to train on")
    return LossParts(total, count0, ce0.detach(), per_batch, terms)
