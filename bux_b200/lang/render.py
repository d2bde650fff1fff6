"""`bux render`: a model's graph as a text diagram, one layer per line along the stream.

::

    tokens
      │ embed                                   → 64
      ╭─ ×2 ──────────────────────────────
      │ ├─[ rmsnorm → gqa(4/2 heads) ]─⊕
      │ ├─[ rmsnorm → gated_mlp(256) ]─⊕
      ╰────────────────────────────────────
      │ rmsnorm
      │ head (tied)                             → logits

Reference: ``lang/render.py``.
"""

from __future__ import annotations

from . import ir


def _label(layer: ir.Layer) -> str:
    c = layer.config
    t = c.type
    if t == "gqa":
        return f"gqa({c.num_heads}/{c.num_kv_heads} heads" + (f", window {c.sliding_window_size}" if c.sliding_window_size else "") + ")"
    if t in ("mlp", "gated_mlp"):
        return f"{t}({c.intermediate_size}, {c.activation})"
    if t == "moe":
        return f"moe({c.num_experts} experts, top {c.top_k}, {c.expert.intermediate_size})"
    if t == "head":
        return "head (tied)" if c.tied else "head"
    if hasattr(c, "num_heads") and hasattr(c, "head_dim"):
        return f"{t}({c.num_heads} heads × {c.head_dim})"
    return t


def _inline(node) -> str:
    if isinstance(node, ir.Layer):
        s = _label(node)
        ports = "".join(f" {p.name}{'→@' if p.mode == 'write' else '←$'}{p.tap}" for p in node.ports)
        return s + ports
    if isinstance(node, ir.Seq):
        return " → ".join(_inline(n) for n in node.items)
    if isinstance(node, ir.Residual):
        return f"[ {_inline(node.body)} ]⊕"
    if isinstance(node, ir.Sum):
        return "(" + " + ".join(_inline(n) for n in node.terms) + ")"
    if isinstance(node, ir.Prod):
        return "(" + " * ".join(_inline(n) for n in node.factors) + ")"
    if isinstance(node, ir.Neg):
        return f"-{_inline(node.body)}"
    if isinstance(node, ir.Const):
        return f"{node.value:g}"
    if isinstance(node, ir.Identity):
        return "·"
    if isinstance(node, ir.Repeat):
        return f"({_inline(node.body)})^{node.times}"
    if isinstance(node, ir.Tap):
        return f"@{node.name}"
    if isinstance(node, ir.Ref):
        return f"${node.name}{'!' if node.pop else ''}"
    return str(node)


def _lines(node, indent: str, out: list) -> None:
    if isinstance(node, ir.Seq):
        for n in node.items:
            _lines(n, indent, out)
    elif isinstance(node, ir.Repeat):
        share = " (shared weights)" if node.body.share is not None else ""
        out.append(f"{indent}╭─ ×{node.times}{share} " + "─" * 30)
        _lines(node.body, indent + "│ ", out)
        out.append(f"{indent}╰" + "─" * 36)
    elif isinstance(node, ir.Residual):
        out.append(f"{indent}├─[ {_inline(node.body)} ]─⊕")
    elif isinstance(node, ir.Layer):
        width = node.width if node.width is not None else ""
        tail = f"← {width}" if node.config.type in ("embed", "head", "linear", "merge") and width != "" else ""
        out.append(f"{indent}│ {_inline(node):<44}{tail}".rstrip())
    else:
        out.append(f"{indent}│ {_inline(node)}")


def render(arch: ir.Architecture) -> str:
    out = ["tokens"]
    _lines(arch.graph, "  ", out)
    head = f"d_model {arch.d_model}, vocab {arch.vocab_size}"
    if arch.residual is not None:
        head += f", residual {arch.residual.type}"
    return head + "\n" + "\n".join(out)
