"""Placement while a model is built: which rows of a sharded parameter this rank keeps.

Under sharded parameters (FSDP) with `placing(rows=...)` active, every projection's weight and
the token table are cut the same way as they are created: the whole tensor is initialised (so
that the rank draws the values a one-rank build draws), this rank's rows are kept and the rest
freed at once, so the rank never holds more than one whole parameter beside its shards (a 70B
dense model over eight ranks: 2 GB transient instead of 141 GB). The sharding layer adopts
these shards as they are (`FSDP` reads ``placed_whole``).

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
_rows: Optional[tuple] = None      # (rank, ranks) of the axes dense parameters are sharded over


@contextmanager
def placing(experts: Optional[tuple] = None, rows: Optional[tuple] = None):
    global _experts, _rows
    before = (_experts, _rows)
    _experts, _rows = experts, rows
    try:
        yield
    finally:
        _experts, _rows = before


@contextmanager
def whole_parameters():
    """Inside, dense parameters are built whole (a layer that edits its weights by row right
    after creating them); the sharding layer cuts them afterwards, as it does without placement."""
    global _rows
    before, _rows = _rows, None
    try:
        yield
    finally:
        _rows = before


def dense_rows(n_rows: int) -> Optional[slice]:
    """This rank's rows of a dense parameter of `n_rows` rows while `placing(rows=...)` is
    active and the rows divide over the ranks (the sharding layer's own rule), else None."""
    if _rows is None:
        return None
    rank, ranks = _rows
    if n_rows % ranks or n_rows < ranks:
        return None
    per = n_rows // ranks
    return slice(rank * per, (rank + 1) * per)


def place_dense(p: torch.nn.Parameter) -> torch.nn.Parameter:
    """`p` cut to this rank's rows when dense placement is active (marked with the whole
    parameter's rows for the sharding layer), else `p` itself."""
    rows = dense_rows(p.shape[0]) if p.dim() > 0 else None
    if rows is None:
        return p
    kept = keep_rows(p, rows)
    kept.placed_whole = p.shape[0]
    return kept


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
