"""Placement while a model is built: which rows of a sharded parameter this rank keeps.

Under expert parallelism a rank owns ``num_experts / n`` experts. With `placing` active, a
layer that creates a stack of experts initialises the whole stack (so that every rank draws
the same values as a one-rank build), keeps its own rows and frees the rest at once: the
rank holds at most one whole stack beside its shards, never the whole model
(Qwen3-30B-A3B: 0.8 GB transient instead of 58 GB of experts on every GPU).
Reference: ``parallel/place.py:70`` (`build`: parameters are created in their sharded
placement).
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Optional

import torch

_experts: Optional[tuple] = None   # (rank, ranks) of the expert axis


@contextmanager
def placing(experts: Optional[tuple] = None):
    global _experts
    before = _experts
    _experts = experts
    try:
        yield
    finally:
        _experts = before


def expert_rows(num_experts: int) -> Optional[slice]:
    """This rank's experts while `placing(experts=...)` is active, else None (keep all)."""
    if _experts is None:
        return None
    rank, ranks = _experts
    if num_experts % ranks:
        raise ValueError(f"{num_experts} experts do not divide over expert={ranks}")
    per = num_experts // ranks
    return slice(rank * per, (rank + 1) * per)


def keep_rows(p: torch.nn.Parameter, rows: slice) -> torch.nn.Parameter:
    """A parameter of `p`'s rows `rows` only (a copy: the whole tensor is freed with `p`)."""
    kept = torch.nn.Parameter(p.data[rows].clone())
    kept.placed_rows = rows
    return kept
