"""The architecture IR the compiler emits and every backend consumes.

A graph is a tree of eleven node kinds, each a function of the incoming stream x
(JSON field names are the on-disk ``run.json`` / ``config.json`` contract shared
with the reference, ``src/bux/lang/ir.py:84-176``):

    layer     config(x)            seq       items applied left to right
    residual  x + body(x)          sum/prod  branches summed / multiplied
    neg       -body(x)             const     a scalar inside sum/prod
    identity  x                    repeat    body applied `times` times, fresh weights
    tap       push x to a named stack, pass it on
    ref       top of a named stack (optionally popping it), ignoring x

`Run.id` hashes what a run computes (not how it is watched or split over GPUs).
"""

from __future__ import annotations

import hashlib
import json
from typing import Annotated, Any, Iterator, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field

from ..config import layers as L
from ..config import training as T

Width = Union[int, Literal["tokens", "logits", "streams"]]

_FROZEN = ConfigDict(frozen=True, extra="forbid")


class _Node(BaseModel):
    model_config = _FROZEN
    label: Optional[str] = None
    share: Optional[str] = None


class Port(BaseModel):
    """A layer's internal tensor routed through a tap: ``gqa(v=@v1)`` writes,
    ``gqa(v=$v1)`` reads, ``$v1!`` reads and pops."""

    model_config = _FROZEN
    name: str
    tap: str
    mode: Literal["write", "read", "pop"]


class Layer(_Node):
    kind: Literal["layer"] = "layer"
    config: L.LayerConfig
    width: Optional[Width] = None
    ports: tuple[Port, ...] = ()


class Seq(_Node):
    kind: Literal["seq"] = "seq"
    items: tuple["Node", ...]


class Residual(_Node):
    kind: Literal["residual"] = "residual"
    body: "Node"


class Sum(_Node):
    kind: Literal["sum"] = "sum"
    terms: tuple["Node", ...]


class Prod(_Node):
    kind: Literal["prod"] = "prod"
    factors: tuple["Node", ...]


class Neg(_Node):
    kind: Literal["neg"] = "neg"
    body: "Node"


class Const(_Node):
    kind: Literal["const"] = "const"
    value: float


class Identity(_Node):
    kind: Literal["identity"] = "identity"


class Repeat(_Node):
    kind: Literal["repeat"] = "repeat"
    body: "Node"
    times: int


class Tap(_Node):
    kind: Literal["tap"] = "tap"
    name: str


class Ref(_Node):
    kind: Literal["ref"] = "ref"
    name: str
    pop: bool = False


Node = Annotated[
    Union[Layer, Seq, Residual, Sum, Prod, Neg, Const, Identity, Repeat, Tap, Ref],
    Field(discriminator="kind"),
]
NODE_TYPES = (Layer, Seq, Residual, Sum, Prod, Neg, Const, Identity, Repeat, Tap, Ref)
for _cls in NODE_TYPES:
    _cls.model_rebuild()

_CHILD_FIELD = {Seq: "items", Sum: "terms", Prod: "factors",
                Residual: "body", Neg: "body", Repeat: "body"}


class Architecture(BaseModel):
    """A compiled model: top-level settings plus the graph."""

    model_config = _FROZEN
    d_model: int
    vocab_size: Optional[int] = None
    residual: Optional[L.ResidualConfig] = None
    init: Optional[L.Init] = None
    graph: Node

    def layers(self) -> Iterator[Layer]:
        return unrolled_layers(self.graph)


def children(node) -> tuple:
    name = _CHILD_FIELD.get(type(node))
    if name is None:
        return ()
    kids = getattr(node, name)
    return kids if isinstance(kids, tuple) else (kids,)


def with_children(node, kids: tuple):
    name = _CHILD_FIELD.get(type(node))
    if name is None:
        return node
    return node.model_copy(update={name: kids if name != "body" else kids[0]})


# the reference's name for the same operation
replace_children = with_children


def walk(node) -> Iterator:
    """Pre-order over the tree as written (a repeat's body once)."""
    stack = [node]
    while stack:
        n = stack.pop()
        yield n
        stack.extend(reversed(children(n)))


def unrolled_layers(node) -> Iterator[Layer]:
    """Every layer in execution order, repeats expanded."""
    if isinstance(node, Layer):
        yield node
    elif isinstance(node, Repeat):
        for _ in range(node.times):
            yield from unrolled_layers(node.body)
    else:
        for kid in children(node):
            yield from unrolled_layers(kid)


def strip(node, *, labels: bool = True, widths: bool = True):
    """Drop labels and/or inferred widths so that structure can be compared. Without
    labels, an unshared seq/sum/prod nested directly in the same kind is inlined."""
    kids = tuple(strip(k, labels=labels, widths=widths) for k in children(node))
    if labels and isinstance(node, (Seq, Sum, Prod)):
        flat = []
        for k in kids:
            if type(k) is type(node) and k.share is None:
                flat.extend(children(k))
            else:
                flat.append(k)
        kids = tuple(flat)
    node = with_children(node, kids)
    update: dict = {}
    if labels:
        update["label"] = None
    if widths and isinstance(node, Layer):
        update["width"] = None
    return node.model_copy(update=update) if update else node


def full_attention_rope(arch: Architecture, **fields) -> Architecture:
    """`arch` with `fields` set on the RoPE of every full-attention layer (no sliding
    window), as a curriculum phase changes them."""
    if not fields:
        return arch

    def remade(node):
        if isinstance(node, Layer):
            c = node.config
            rope = getattr(c, "rope", None)
            if (isinstance(c, L.QuadraticAttentionConfig) and not c.sliding_window_size
                    and rope is not None):
                c = c.model_copy(update={"rope": rope.model_copy(update=fields)})
                return node.model_copy(update={"config": c})
            return node
        return with_children(node, tuple(remade(k) for k in children(node)))

    return arch.model_copy(update={"graph": remade(arch.graph)})


# ------------------------------------------------------------------ run identity
# Settings that change how a run is watched, split or searched -- not what it computes.
UNCOMPUTED = frozenset({"log", "eval", "checkpoint", "observe", "profile", "mesh", "layout",
                        "methods", "compiler", "objective", "search"})
# Settings / fields added after ids existed: at these values they compute what older
# runs computed, so they are left out of the hash and old ids (and checkpoints) stay
# valid. Tables follow the reference's back-compat rules (src/bux/lang/ir.py:321-402).
_OLD_SETTING = {"precision": T.PrecisionConfig(compute="float32")}
_OLD_VALUE = {"batch_ramp": None, "curriculum": [], "ema": None}
_OLD_FIELDS = {
    "precision": {
        "matmuls": "compute", "reduce": "compute",
        **T.PrecisionConfig().model_dump(
            mode="json", include={"roles", "first", "last", "passes", "switch"}),
        "moments": "float32", "dispatch": "compute",
    },
    "optimizer": {"ns_coefficients": "jordan", "ns_dtype": "float32",
                  "ns_algorithm": "standard", "ns_restarts": None,
                  "cautious_weight_decay": False},
    "schedule": {"horizon": 1.0},
    "loss": {"prefix": None},
}
_OLD_PHASE_FIELDS = {"rope_scaling": None, "rope_base": None}
_WATCH_ONLY_FIELDS = {"precision": ("eval",)}
_HYGA = {"gate_input_rank": None, "gate_output_rank": None, "gate_cross_head": False}
_OLD_LAYER_FIELDS = {
    "mlp": {"up_offset": 0.0},
    "gated_mlp": {"up_offset": 0.0},
    "moe": {"router_bias": False, "center_bias": False, "bias_softclamp": 2.0,
            "bias_momentum": 0.5, "num_zero_experts": 0, "ffn_experts_per_token": None},
    "mamba2": {"num_heads": None},
    "head": {"pointer": None},
    "gqa": {"gate_head_bias": False, "power_scale": None, "power_scale_length": 2048,
            "qk_norm_all_heads": False, "exclusive": False, "differential": False,
            "paired": False, **_HYGA, "value_embed_gate": 6, "k_eq_v": False,
            "mimetic_vo": None, "mimetic_noise": 0.01},
    "mla": {"gate_head_bias": False, **_HYGA},
    "csa": {"gate_head_bias": False, **_HYGA},
    "indexer": {"pool": "mean", "per_group": False, "relu": True, "loss_over": "own"},
    "layernorm": {"gain_init": 1.0},
    "rmsnorm": {"gain_init": 1.0},
    "normal": {"embed": None, "head": None, "out": None},
    "hc": {"pre_bias": 1.0, "post_bias": 1.0, "res_bias": -8.0},
    "mhc": {"res_bias": -8.0},
}
_INIT_BEFORE = L.FanInitConfig(
    type="fan_in", embed=L.FanInitConfig(type="fan_in", distribution="gaussian"))


def _drop_old_fields(train: dict) -> dict:
    for setting, fields in _OLD_FIELDS.items():
        given = train.get(setting) or {}
        for part in (given, given.get("adam") or {}):
            for name, before in fields.items():
                if name in part and part[name] == before:
                    del part[name]
    for phase in train.get("curriculum") or ():
        for name, before in _OLD_PHASE_FIELDS.items():
            if name in phase and phase[name] == before:
                del phase[name]
    for setting, names in _WATCH_ONLY_FIELDS.items():
        for name in names:
            (train.get(setting) or {}).pop(name, None)
    return train


def _drop_old_layer_fields(node: Any) -> Any:
    if isinstance(node, list):
        return [_drop_old_layer_fields(n) for n in node]
    if not isinstance(node, dict):
        return node
    before = _OLD_LAYER_FIELDS.get(node.get("type"), {})
    return {k: _drop_old_layer_fields(v) for k, v in node.items()
            if not (k in before and v == before[k])}


class Run(BaseModel):
    """One training run: an architecture and every training setting resolved."""

    model_config = _FROZEN
    name: str
    arch: Architecture
    train: T.TrainConfig
    choices: tuple[str, ...] = ()
    axes: tuple[str, ...] = ()

    def arch_at(self, step: int) -> Architecture:
        from ..train import curriculum

        return full_attention_rope(self.arch, **curriculum.rope_at(self.train, step))

    @property
    def id(self) -> str:
        """sha256[:10] of canonical JSON of (arch, train) minus the watch/split
        settings and minus newer fields left at their old-behaviour defaults."""
        arch = self.arch.model_copy(update={"graph": strip(self.arch.graph)})
        train = self.train.model_dump(mode="json", exclude=set(UNCOMPUTED))
        has_moe = any(layer.config.type == "moe" for layer in self.arch.layers())
        if has_moe:
            train["precision"]["roles"]["experts"] = self.train.precision.experts()
        train = _drop_old_fields(train)
        for setting, before in _OLD_SETTING.items():
            old = _drop_old_fields({setting: before.model_dump(mode="json")})
            if train[setting] == old[setting]:
                del train[setting]
        for setting, value in _OLD_VALUE.items():
            if train[setting] == value:
                del train[setting]
        dumped = _drop_old_layer_fields(arch.model_dump(mode="json"))
        if self.arch.init == _INIT_BEFORE and not has_moe:
            del dumped["init"]
        blob = json.dumps({"arch": dumped, "train": train}, sort_keys=True,
                          separators=(",", ":"))
        return hashlib.sha256(blob.encode()).hexdigest()[:10]
