"""Parallelism: mesh, layout, and the per-rank engines (FSDP, TP, EP, PP, CP)."""
from . import mesh  # noqa: F401
