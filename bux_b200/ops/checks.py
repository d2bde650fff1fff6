"""Kernel checks without a sanitizer: guard regions around every buffer a kernel writes,
and run-twice determinism.

``BUX_KERNEL_CHECKS=1`` (or `enable()`) makes the wrappers in `bux_b200.ops.kernels`
allocate each output inside a larger byte buffer whose head and tail are filled with a
pattern. `verify()` (call it after a synchronise; the GPU tests do after every test)
reads the guards back and raises naming the op whose kernel wrote outside its output.
A kernel that overruns therefore corrupts a guard of its own buffer instead of a
neighbour's data, and is named, which is what an address sanitizer would give, for the
writes that matter here (contiguous outputs of hand-written kernels).

`same_twice(fn)` runs a function twice from the same inputs and reports the outputs that
are not bitwise equal: the kernels here use no atomics on their outputs except where the
docstring says so (dq's reduce-add, the RMSNorm weight gradient, the router-scale
gradient), so anything else that differs between two runs is a race.

The reference has neither (it has no native code); its closest tool is XLA's
deterministic-ops flag (``docs/parallelism/attention.md:322-323`` there).
"""

from __future__ import annotations

import os
from typing import Callable, Optional

import torch

GUARD_BYTES = 4096
PATTERN = 0xA5
_on = os.environ.get("BUX_KERNEL_CHECKS", "") not in ("", "0", "off")
_live: list = []      # (op name, whole byte buffer, payload bytes)


def enabled() -> bool:
    return _on


def enable(on: bool = True) -> None:
    global _on
    _on = on
    if not on:
        _live.clear()


def guarded_empty(shape, dtype, device, op: str, fill: Optional[float] = None) -> torch.Tensor:
    """An uninitialised (or `fill`-ed) tensor for a kernel's output. With checks on it sits
    between two guard regions of `GUARD_BYTES` bytes each."""
    if not _on or torch.device(device).type != "cuda":
        if fill is None:
            return torch.empty(shape, dtype=dtype, device=device)
        return torch.full(shape, fill, dtype=dtype, device=device)
    numel = 1
    for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)):
        numel *= int(s)
    item = torch.empty((), dtype=dtype).element_size()
    payload = numel * item
    padded = -(-payload // 256) * 256          # keeps the 16-byte (and TMA's 128-byte) alignment of the payload
    whole = torch.empty(GUARD_BYTES + padded + GUARD_BYTES, dtype=torch.uint8, device=device)
    whole[:GUARD_BYTES].fill_(PATTERN)
    whole[GUARD_BYTES + payload:].fill_(PATTERN)
    out = whole[GUARD_BYTES:GUARD_BYTES + payload].view(dtype).view(shape)
    if fill is not None:
        out.fill_(fill)
    _live.append((op, whole, payload))
    return out


def verify(clear: bool = True) -> None:
    """Raise if any guard region written since the last call no longer holds the pattern.
    Synchronises the devices involved."""
    bad = []
    for op, whole, payload in _live:
        head = whole[:GUARD_BYTES]
        tail = whole[GUARD_BYTES + payload:]
        for name, region in (("before", head), ("after", tail)):
            wrong = (region != PATTERN).nonzero()
            if wrong.numel():
                first = int(wrong[0])
                bad.append(f"{op}: {wrong.numel()} bytes {name} its output were overwritten "
                           f"(first at offset {first if name == 'after' else first - GUARD_BYTES})")
    if clear:
        _live.clear()
    if bad:
        raise AssertionError("a kernel wrote outside its output: " + "; ".join(bad))


def same_twice(fn: Callable[[], object]) -> list:
    """Run `fn` twice; returns the paths of tensors in its results that differ bitwise."""
    def flat(prefix, obj, out):
        if isinstance(obj, torch.Tensor):
            out[prefix] = obj.detach().clone()
        elif isinstance(obj, dict):
            for k, v in obj.items():
                flat(f"{prefix}.{k}", v, out)
        elif isinstance(obj, (tuple, list)):
            for i, v in enumerate(obj):
                flat(f"{prefix}[{i}]", v, out)
        return out

    first = flat("out", fn(), {})
    second = flat("out", fn(), {})
    differing = []
    for name, a in first.items():
        b = second.get(name)
        if b is None or a.shape != b.shape or not torch.equal(a.view(torch.uint8) if a.dtype.itemsize == 1 else a, b.view(torch.uint8) if b.dtype.itemsize == 1 else b):
            differing.append(name)
    return differing
