"""What a training forward observes of the model on the steps ``observe(every=...)`` picks:
the residual stream after every branch that is inside no other (RMS, RMS of what the branch
added, largest magnitude, kurtosis over the features, optionally a log2 histogram), every MoE's
routing (largest and smallest share of an expert, share of dead experts, entropy, z, the
balance bias's spread) and a sample of every attention's logits (their maximum, the entropy
of the probabilities).

A layer observes a value in one line, ``observe.stat(ctx, "router/max_load", value)``; only a
forward whose context has ``observing`` set collects it, so the other steps pay nothing. A
value's name carries the branch it was observed in, numbered among the branches of that name
in the order they run: ``router/max_load/moe.03``.
Reference: ``architecture/observe.py:89-227`` there.
"""

from __future__ import annotations

import torch

LOW, HIGH = -24, 15            # log2 |x| bins of a histogram, one each, the ends open
SAMPLE = 1 << 22               # the most entries a histogram takes: an even sample
NORMS = frozenset({"rmsnorm", "layernorm", "dyt", "scale", "act", "dropout"})


def branch_name(node) -> str:
    """A branch is named for its last layer that is not a norm: ``[norm attn]`` is ``attn``'s type."""
    from ..lang import ir

    names: list = []

    def walk(n):
        if isinstance(n, ir.Layer):
            names.append(n.config.type)
        for field in ("items", "terms", "factors"):
            for child in getattr(n, field, ()) or ():
                walk(child)
        body = getattr(n, "body", None)
        if body is not None:
            walk(body)

    walk(node)
    named = [n for n in names if n not in NORMS]
    return named[-1] if named else (names[-1] if names else "branch")


def stat(ctx, name: str, value) -> None:
    """Record `value` (a scalar tensor) under `name` for the branch that is running."""
    if not getattr(ctx, "observing", False):
        return
    branch = getattr(ctx, "observed_branch", None)
    key = name if branch is None else f"{name}/{branch}"
    ctx.observed[key] = value.detach().float()


def histogram(ctx, name: str, x: torch.Tensor) -> None:
    if not getattr(ctx, "observing", False) or not getattr(ctx, "observe_histograms", False):
        return
    flat = x.detach().reshape(-1)
    if flat.numel() > SAMPLE:
        flat = flat[:: flat.numel() // SAMPLE][:SAMPLE]
    mag = flat.float().abs()
    e = torch.floor(torch.log2(mag.clamp_min(2.0 ** LOW))).clamp(LOW, HIGH).long() - LOW
    branch = getattr(ctx, "observed_branch", None)
    ctx.observed_histograms[name if branch is None else f"{name}/{branch}"] = torch.bincount(e, minlength=HIGH - LOW + 1)


def feature_kurtosis(y: torch.Tensor) -> torch.Tensor:
    """Kurtosis of the features' RMS over the positions: large when a few channels carry the stream."""
    power = y.float().square().mean(dim=tuple(range(y.dim() - 1)))      # per feature
    return power.square().mean() / power.mean().square().clamp_min(1e-30)


def stream(ctx, x: torch.Tensor, y: torch.Tensor) -> None:
    """The residual stream after a branch: `x` went in, `y` came out."""
    if not getattr(ctx, "observing", False) or not isinstance(y, torch.Tensor) or not isinstance(x, torch.Tensor):
        return
    y32 = y.detach().float()
    stat(ctx, "act/rms", y32.square().mean().sqrt())
    if x.shape == y.shape:
        stat(ctx, "act/update_rms", (y32 - x.detach().float()).square().mean().sqrt())
    stat(ctx, "act/max_abs", y32.abs().max())
    stat(ctx, "act/kurtosis", feature_kurtosis(y32))
    histogram(ctx, "act/hist", y32)


def router(ctx, logits: torch.Tensor, picks: torch.Tensor, num_experts: int, bias=None) -> None:
    """An MoE's routing: `logits` [.., E'] before the pick, `picks` [.., k] expert ids."""
    if not getattr(ctx, "observing", False):
        return
    load = torch.bincount(picks.reshape(-1).clamp(0, num_experts - 1), minlength=num_experts).float()
    share = load / load.sum().clamp_min(1.0) * num_experts          # 1 = an even share
    stat(ctx, "router/max_load", share.max())
    stat(ctx, "router/min_load", share.min())
    stat(ctx, "router/dead", (load == 0).float().mean())
    p = torch.softmax(logits.detach().float(), -1)
    stat(ctx, "router/entropy", -(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean())
    stat(ctx, "router/z", torch.logsumexp(logits.detach().float(), -1).square().mean())
    if bias is not None:
        stat(ctx, "router/bias_std", bias.detach().float().std())


def attention_sample(ctx, q: torch.Tensor, k: torch.Tensor, scale, causal: bool = True, queries: int = 64) -> None:
    """Largest logit and mean entropy of the attention of an even sample of `queries` positions
    (all heads): q [b, t, h, d], k [b, s, g, d], rows that see each other causally."""
    if not getattr(ctx, "observing", False):
        return
    b, t, h, d = q.shape
    s, g = k.shape[1], k.shape[2]
    at = torch.arange(0, t, max(t // queries, 1), device=q.device)[:queries]
    qs = q.detach()[:, at].float()
    kk = k.detach().float().repeat_interleave(h // g, dim=2)
    logits = torch.einsum("bthd,bshd->bhts", qs, kk) * (scale if scale is not None else d ** -0.5)
    if causal:
        seen = (at + (s - t)).view(1, 1, -1, 1) >= torch.arange(s, device=q.device).view(1, 1, 1, -1)
        logits = logits.masked_fill(~seen, float("-inf"))
    stat(ctx, "attn/logit_max", logits.max())
    p = torch.softmax(logits, -1)
    stat(ctx, "attn/entropy", -(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean())
