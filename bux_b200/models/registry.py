"""Layer registry and the per-forward context every layer receives.

`register("gqa")` maps a settings ``type`` to a builder ``(config, BuildContext) ->
nn.Module``; `build_layer` looks it up. A layer's ``forward(x, ctx)`` gets the
`Context` of the running forward: positions, document segments, the tap stacks,
ports, the losses layers report, and the matmul format of each role.

Reference counterparts: ``architecture/registry.py:58-270`` (`Taps`, `Context`,
`register`, `build_layer`).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

BUILDERS: dict = {}


def register(*types: str) -> Callable:
    def wrap(fn):
        for t in types:
            BUILDERS[t] = fn
        return fn

    return wrap


@dataclass
class BuildContext:
    """What a builder knows: the model's width, vocabulary, residual algebra, init."""
    d_model: int
    vocab_size: Optional[int]
    residual: object = None
    init: object = None
    width: object = None  # the layer's inferred input width
    ports: tuple = ()
    embedding: object = None  # the first embedding module, for tied heads / nextn
    dtype: torch.dtype = torch.float32
    layer_index: int = 0
    num_layers: int = 1


def build_layer(config, bctx: BuildContext):
    try:
        builder = BUILDERS[config.type]
    except KeyError:
        raise NotImplementedError(
            f"layer '{config.type}' has no builder: add one under "
            f"@bux_b200.models.register({config.type!r})") from None
    return builder(config, bctx)


@dataclass
class Precision:
    """Matmul format by role, resolved from ``precision(...)`` for this forward.

    `first` / `last`: so many residual branches (the ``[...]`` that are inside no other, counted
    up to the first head: `branches` of them) at the model's start and end multiply in the
    compute dtype; `branch` is the one that is running (set by the graph). `passes`: which of a
    projection's GEMMs (fprop, dgrad, wgrad) multiply in the format.
    Reference: ``architecture/precision/matmuls.py``, ``docs/training/precision.md`` there."""
    compute: torch.dtype = torch.float32
    matmuls: str = "compute"
    roles: dict = field(default_factory=dict)
    enabled: bool = True
    first: int = 0
    last: int = 0
    branches: int = 0
    passes: tuple = ("fprop", "dgrad", "wgrad")
    branch: int = -1

    def at_an_edge(self) -> bool:
        if self.branch < 0 or not (self.first or self.last):
            return False
        return self.branch < self.first or self.branch >= self.branches - self.last

    def of(self, role: str) -> str:
        if not self.enabled or not self.passes or self.at_an_edge():
            return "bf16"
        fmt = self.roles.get(role) or self.matmuls
        return "bf16" if fmt in ("compute", None) else fmt


class Context:
    """State of one forward pass, shared by every layer."""

    def __init__(self, input_ids: torch.Tensor, positions: Optional[torch.Tensor] = None,
                 segments: Optional[torch.Tensor] = None, training: bool = False,
                 precision: Optional[Precision] = None, methods=None, parallel=None,
                 step: int = 0):
        self.input_ids = input_ids
        b, t = input_ids.shape[:2]
        if positions is None:
            positions = torch.arange(t, device=input_ids.device).unsqueeze(0).expand(b, t)
        self.positions = positions
        self.segments = segments
        self.training = training
        self.precision = precision or Precision()
        self.methods = methods
        self.parallel = parallel
        self.step = step
        self.taps: dict = {}
        self.ports: dict = {}
        self.losses: dict = {}
        self.metrics: dict = {}
        self.heads: list = []
        self._rope: dict = {}
        self.branch_index = 0
        self.top_branch = 0     # residual branches that are inside no other, run so far
        self.branch_depth = 0
        # observe(every=...): set for the forward of an observed step (`bux_b200.models.observe`)
        self.observing = False
        self.observe_histograms = False
        self.observed: dict = {}
        self.observed_histograms: dict = {}
        self.observed_branch = None
        self.branch_names: dict = {}   # how many branches of each name ran so far
        self.pending_read = None  # single-pass hyper-connections: the read the last branch computed
        self.cache = None         # a `DecodeCache` when the tokens continue what it holds (incremental decoding)

    # taps are named stacks
    def push(self, name: str, value) -> None:
        self.taps.setdefault(name, []).append(value)

    def read(self, name: str, pop: bool = False):
        stack = self.taps[name]
        return stack.pop() if pop else stack[-1]

    def report(self, name: str, value: torch.Tensor, weight: float = 1.0) -> None:
        """A layer's auxiliary loss (balance_loss, indexer_loss, ...), summed per name."""
        prev = self.losses.get(name)
        item = value * weight
        self.losses[name] = item if prev is None else prev + item

    def metric(self, name: str, value) -> None:
        self.metrics.setdefault(name, []).append(value)

    def rope_tables(self, key, make: Callable):
        if key not in self._rope:
            self._rope[key] = make()
        return self._rope[key]
