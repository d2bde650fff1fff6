"""The training objective: next-token cross-entropy of every head (+ z-loss, weighted
multi-token-prediction heads) plus the auxiliary losses layers report.

Losses are kept as (sum over target tokens, target count) so that microbatches and
ranks add up to the whole batch's mean exactly; the caller divides by the global
count (a device scalar, so nothing synchronises).

Reference: ``train/objective.py:53-477`` (`Heads`, `Objective`, `target_mask`).
"""

from __future__ import annotations

import math

from dataclasses import dataclass, field

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


# ------------------------------------------------------------------ what an evaluation measures
def per_token_nats(head, targets: torch.Tensor, rows: int = 4096) -> torch.Tensor:
    """The head's cross-entropy of every position, [B, T] fp32, its logits formed a slab of
    positions at a time (an evaluation only: training never holds per-token losses)."""
    hidden = head.hidden.reshape(-1, head.hidden.shape[-1])
    flat = targets.reshape(-1)
    out = torch.empty(flat.shape[0], dtype=torch.float32, device=hidden.device)
    weight = head.weight.to(hidden.dtype)
    for s in range(0, hidden.shape[0], rows):
        logits = torch.nn.functional.linear(hidden[s:s + rows], weight,
                                            None if head.bias is None else head.bias.to(hidden.dtype)).float()
        if head.softcap:
            logits = head.softcap * torch.tanh(logits / head.softcap)
        out[s:s + rows] = torch.nn.functional.cross_entropy(logits, flat[s:s + rows].long(), reduction="none")
    return out.view(targets.shape)


def held_out(ctx, batch, token_bytes=None, positions=()) -> dict:
    """What an evaluation measures of the first head on `batch`, each as (sum, what it is a
    mean of): ``loss`` (nats over targets); with `token_bytes` (int tensor [vocab]: the bytes
    of text each id stands for, 0 for a special token) ``bpb`` (bits over bytes: a target
    that stands for no text is left out); and with `positions`, each of them over the targets
    of each bucket of positions in their documents, named by the bucket's first position
    (``loss_0``, ``loss_2k``, ...). Reference: ``train/objective.py:408-450`` there."""
    ids, pos, lmask = batch
    tgt, mask = targets_and_mask(ids, pos, lmask, 1)
    nats = per_token_nats(ctx.heads[0], tgt)
    weights = {"loss": mask.float()}
    if token_bytes is not None:
        weights["bpb"] = torch.where(mask, token_bytes.to(tgt.device)[tgt.long()].float(), torch.zeros(()).to(nats))
    if positions:
        edges = [0, *positions]
        names = T.buckets(positions)
        for base in list(weights):
            for k, name in enumerate(names):
                inside = pos >= edges[k]
                if k + 1 < len(edges):
                    inside = inside & (pos < edges[k + 1])
                weights[f"{base}_{name}"] = weights[base] * inside.float()
    out = {}
    for name, w in weights.items():
        counted = (w > 0).float()
        total = (nats * counted).sum()
        if name.startswith("bpb"):
            total = total / math.log(2)
        out[name] = (total, w.sum())
    return out
