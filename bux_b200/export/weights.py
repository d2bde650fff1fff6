"""Tensor naming of an exported checkpoint.

Training keeps fused matrices (``qkv``, ``gate_up``, ``experts_gate_up``); the export
names every projection on its own, as the reference's export does
(``export/weights.py:37``), so a serving stack can shard them by heads or hidden units:

    ...qkv.weight            → ...q.weight, ...k.weight, ...v.weight   (rows q | k | v)
    ...gate_up.weight        → ...gate.weight, ...up.weight            (rows gate | up)
    ...experts_gate_up [E,2f,d] → ...experts.gate [E,f,d], ...experts.up [E,f,d]
    ...experts_down   [E,d,f]   → ...experts.down [E,d,f]

`tensors` goes from a model to the exported names, `fused` back.
"""

from __future__ import annotations

import torch


def _splits(model) -> dict:
    """{fused parameter path: [(exported path, rows)]} from the model's modules."""
    from ..models.layers.attention import GQA
    from ..models.layers.basic import MLP
    from ..models.layers.moe import MoE

    out = {}
    for path, m in model.named_modules():
        pre = f"{path}." if path else ""
        if isinstance(m, GQA):
            for leaf in ("weight", "bias"):
                if getattr(m.qkv, leaf, None) is not None:
                    parts = [(f"{pre}q.{leaf}", m.q_rows), (f"{pre}k.{leaf}", m.k_rows), (f"{pre}v.{leaf}", m.v_rows)]
                    out[f"{pre}qkv.{leaf}"] = [p for p in parts if p[1]]  # k_eq_v: no v projection
        elif isinstance(m, MLP) and m.gated:
            f = m.gate_up.weight.shape[0] // 2
            for leaf in ("weight", "bias"):
                if getattr(m.gate_up, leaf, None) is not None:
                    out[f"{pre}gate_up.{leaf}"] = [(f"{pre}gate.{leaf}", f), (f"{pre}up.{leaf}", f)]
        elif isinstance(m, MoE):
            if m.gated:
                out[f"{pre}experts_gate_up"] = [(f"{pre}experts.gate", m.f), (f"{pre}experts.up", m.f)]
            else:  # plain MLP experts: the up projection alone
                out[f"{pre}experts_gate_up"] = [(f"{pre}experts.up", None)]
            out[f"{pre}experts_down"] = [(f"{pre}experts.down", None)]
    return out


def tensors(model, state: dict = None, dtype=None) -> dict:
    """Exported name → tensor, from the model's parameters and persistent buffers (or `state`)."""
    state = state if state is not None else {k: v for k, v in model.state_dict().items()}
    splits = _splits(model)
    out = {}
    for name, t in state.items():
        t = t.detach()
        if dtype is not None and t.is_floating_point():
            t = t.to(dtype)
        if name in splits:
            parts = splits[name]
            if parts[0][1] is None:
                out[parts[0][0]] = t.contiguous()
                continue
            dim = 1 if t.dim() == 3 else 0
            for (new, _), piece in zip(parts, t.split([r for _, r in parts], dim=dim)):
                out[new] = piece.contiguous()
        else:
            out[name] = t.contiguous()
    return out


def fused(model, exported: dict) -> dict:
    """The inverse: a state dict the model loads."""
    splits = _splits(model)
    taken, out = set(), {}
    for name, parts in splits.items():
        names = [p[0] for p in parts]
        if all(n in exported for n in names):
            pieces = [exported[n] for n in names]
            out[name] = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=1 if pieces[0].dim() == 3 else 0)
            taken.update(names)
    for name, t in exported.items():
        if name not in taken:
            out[name] = t
    return out
