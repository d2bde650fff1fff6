"""The device mesh: six named axes in the fixed order (stage, data, fsdp, context,
expert, tensor), one rank per GPU, nodes filled from ``tensor`` outward so that the
innermost (most talkative) axes stay inside a node's NVLink domain.

Reference: ``parallel/mesh.py:27-182`` (`AXES`, `sizes`, `grid`, `split`).
"""

from __future__ import annotations

from typing import Optional

AXES = ("stage", "data", "fsdp", "context", "expert", "tensor")


def sizes(mesh, world: Optional[int] = None) -> dict:
    """Size of every axis; ``data=None`` takes the devices the other axes leave."""
    out = {a: getattr(mesh, a) for a in AXES}
    fixed = 1
    for a in AXES:
        if a != "data":
            fixed *= out[a]
    if out["data"] is None:
        if world is None:
            out["data"] = 1
        else:
            if world % fixed:
                raise ValueError(f"the mesh's axes need a multiple of {fixed} devices, not {world}")
            out["data"] = world // fixed
    return out


def size(mesh, world: Optional[int] = None) -> int:
    n = 1
    for v in sizes(mesh, world).values():
        n *= v
    return n


def coordinates(rank: int, shape: dict) -> dict:
    """Rank → coordinate on every axis (row-major over AXES, tensor fastest)."""
    out = {}
    for a in reversed(AXES):
        out[a] = rank % shape[a]
        rank //= shape[a]
    return out


def rank_of(coords: dict, shape: dict) -> int:
    r = 0
    for a in AXES:
        r = r * shape[a] + coords[a]
    return r


def group_ranks(rank: int, shape: dict, axes: tuple) -> list:
    """Ranks that share `rank`'s coordinates on every axis but `axes` (in rank order)."""
    mine = coordinates(rank, shape)
    out = []

    def walk(i: int, cur: dict):
        if i == len(axes):
            out.append(rank_of(cur, shape))
            return
        for v in range(shape[axes[i]]):
            walk(i + 1, {**cur, axes[i]: v})

    walk(0, dict(mine))
    return sorted(out)


def _axes_of(spec) -> tuple:
    if spec is None:
        return ()
    return (spec,) if isinstance(spec, str) else tuple(spec)


def param_shards(mesh, layout, world: Optional[int] = None) -> int:
    """Over how many devices a (large) parameter's storage is split: the layout's fsdp
    axes (under zero=3), times tensor and stage."""
    s = sizes(mesh, world)
    n = s["stage"] * s["tensor"]
    if layout.zero == 3:
        for a in _axes_of(layout.fsdp):
            n *= s[a]
    return n
