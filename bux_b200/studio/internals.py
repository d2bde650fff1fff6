"""What is inside a layer, as a small diagram in the page's own node format: feed-forwards,
mixtures of experts, attention (`gqa`, `mla`), the delta-rule mixers and Mamba-2 open into the
projections, norms and products they are made of. `inside(config, width)` returns a tree the
diagram draws like any other (boxes are ``layer`` nodes without a span, so they select
nothing in the source). Reference: ``studio/internals.py``."""

from __future__ import annotations

from typing import Optional

_count = 0


def _box(title: str, *chips, type: str = "linear") -> dict:
    global _count
    _count += 1
    return {"id": -_count, "kind": "layer", "span": None, "type": type, "title": title,
            "chips": [str(c) for c in chips if c not in (None, "", False)], "source": "", "ports": [], "opens": False}


def _seq(*items, name: Optional[str] = None) -> dict:
    global _count
    _count += 1
    out = {"id": -_count, "kind": "seq", "span": None, "items": [i for i in items if i is not None]}
    if name:
        out["name"] = name
    return out


def _par(kind: str, *arms) -> dict:
    global _count
    _count += 1
    key = "terms" if kind == "sum" else "factors"
    return {"id": -_count, "kind": kind, "span": None, key: list(arms)}


def _mlp(c, width: int) -> dict:
    f = c.intermediate_size
    down = _box("Down projection", f"{f} → {width}")
    if c.type == "gated_mlp":
        gate = _seq(_box("Gate projection", f"{width} → {f}"), _box(c.activation, type="act"))
        up = _box("Up projection", f"{width} → {f}", f"+{c.up_offset:g}" if c.up_offset else None,
                  f"clip ±{c.limit:g}" if c.limit else None)
        return _seq(_par("prod", gate, up), down)
    return _seq(_box("Up projection", f"{width} → {f}"), _box(c.activation, type="act"), down)


def _moe(c, width: int) -> dict:
    inner = c.latent_size or width
    router = _seq(_box("Router", f"{width} → {c.num_experts + c.num_zero_experts}", c.router, type="rmsnorm"),
                  _box(f"Top {c.top_k}", "normalised" if c.normalize_top_k else None,
                       f"×{c.routed_scaling_factor:g}" if c.routed_scaling_factor != 1 else None,
                       f"{c.top_k_groups} of {c.num_groups} groups" if c.num_groups > 1 else None, type="rmsnorm"))
    experts = _seq(_mlp(c.expert, inner), name=f"{c.num_experts} experts, {c.top_k} per token")
    routed = _seq(_box("To latent", f"{width} → {inner}") if c.latent_size else None, _par("prod", router, experts),
                  _box("From latent", f"{inner} → {width}") if c.latent_size else None)
    if not c.num_shared_experts:
        return routed
    s = c.shared_expert or c.expert
    shared = _seq(_mlp(s.model_copy(update={"intermediate_size": s.intermediate_size * c.num_shared_experts}), width),
                  _box("Gate", "sigmoid", type="act") if c.shared_expert_gate else None,
                  name=f"{c.num_shared_experts} shared")
    return _par("sum", routed, shared)


def _norm_rope(c, what: str) -> Optional[dict]:
    chips = []
    if getattr(c, "qk_norm", None) is not None:
        chips.append(c.qk_norm.type)
    if getattr(c, "rope", None) is not None:
        chips.append(f"RoPE {c.rope.base:g}" + (f" × {c.rope.fraction:g}" if c.rope.fraction != 1 else ""))
    return _box(f"{what}: norm, rotate", *chips, type="rmsnorm") if chips else None


def _gqa(c, width: int) -> dict:
    d = c.head_dim or width // c.num_heads
    dv = c.v_head_dim or d
    q = _seq(_box("Query projection", f"{width} → {c.num_heads} × {d}"), _norm_rope(c, "q"))
    k = _seq(_box("Key projection", f"{width} → {c.num_kv_heads} × {d}"), _norm_rope(c, "k"))
    v = None if c.k_eq_v else _box("Value projection", f"{width} → {c.num_kv_heads} × {dv}")
    attend = _box("Softmax attention", "causal", f"window {c.sliding_window_size}" if c.sliding_window_size else None,
                  "sinks" if c.sinks else None, f"softcap {c.softcap:g}" if c.softcap else None,
                  f"sparse top {c.indexer.top_k}" if c.indexer is not None else None, type="gqa")
    tail = [attend, _box("Output norm", c.output_norm.type, type="rmsnorm") if c.output_norm is not None else None,
            _box("Output gate", c.gate_activation, "per head" if c.gate_per_head else None, type="act") if c.gated else None,
            _box("Output projection", f"{c.num_heads} × {dv} → {width}")]
    return _seq(_par("prod", *(x for x in (q, k, v) if x is not None)), *tail)


def _mla(c, width: int) -> dict:
    qk = c.qk_nope_head_dim + c.qk_rope_head_dim
    q = _seq(_box("Query latent", f"{width} → {c.q_lora_rank}") if c.q_lora_rank else None,
             _box("Query projection", f"→ {c.num_heads} × {qk}"))
    kv = _seq(_box("Key/value latent", f"{width} → {c.kv_lora_rank} + {c.qk_rope_head_dim}"),
              _box("Expand", f"→ {c.num_heads} × ({c.qk_nope_head_dim} + {c.v_head_dim})"))
    return _seq(_par("prod", q, kv), _box("Softmax attention", "causal", type="gqa"),
                _box("Output projection", f"{c.num_heads} × {c.v_head_dim} → {width}"))


def _delta(c, width: int) -> dict:
    hv, dv = c.num_v_heads or c.num_heads, c.v_head_dim or c.head_dim
    conv = _box("Short convolution", f"{c.conv_size} taps", "silu", type="conv") if c.conv_size else None
    qkv = _seq(_box("q, k, v projections", f"{c.num_heads} × {c.head_dim}", f"{hv} × {dv} values"), conv)
    gates = _box("Decay and write gates", {"gdn": "scalar decay per head", "kda": "decay per channel",
                                           "gdn2": "decay per channel", "deltanet": "no decay"}.get(c.type, ""), type="act")
    state = _box("Delta-rule state", f"{c.head_dim} × {dv} per head", "chunks of 64", type="gdn")
    return _seq(_par("prod", qkv, gates), state, _box("Output norm", type="rmsnorm"),
                _box("Output gate", c.output_gate, type="act") if c.output_gate else None,
                _box("Output projection", f"{hv} × {dv} → {width}"))


def _mamba2(c, width: int) -> dict:
    inner = c.num_heads * c.head_dim if c.num_heads else c.expand * width
    return _seq(_box("Input projection", f"{width} → z, x, B, C, dt"), _box("Short convolution", f"{c.conv_size} taps", "silu", type="conv"),
                _box("State-space scan", f"{inner // c.head_dim} heads", f"state {c.state_size}", type="mamba2"),
                _box("Gate and norm", "silu(z)", type="act"), _box("Output projection", f"{inner} → {width}"))


BUILDERS = {"mlp": _mlp, "gated_mlp": _mlp, "moe": _moe, "gqa": _gqa, "mla": _mla, "deltanet": _delta, "gdn": _delta,
            "kda": _delta, "gdn2": _delta, "mamba2": _mamba2}


def inside(config, width: int) -> Optional[dict]:
    """The diagram of what is inside a layer of `config` on a stream `width` wide, or None."""
    make = BUILDERS.get(config.type)
    return make(config, width) if make is not None else None
