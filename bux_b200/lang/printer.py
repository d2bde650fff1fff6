"""IR → canonical ``.bux`` source: what ``run.bux`` holds and ``bux fmt`` prints.

Settings print with only the fields that differ from their defaults; graph nodes that
carry a label print as definitions (first use wins; a label reused for a different
block gets a numeric suffix), so the text compiles back to the same run id.

Reference: ``lang/printer.py:30-353`` (`run_to_source`, `config_to_source`).
"""

from __future__ import annotations

import re

from pydantic import BaseModel

from ..config import training as T
from . import ir

_NAME = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")
_PREC = {"sum": 1, "prod": 2, "seq": 3, "neg": 4, "repeat": 5}


def value_to_source(v) -> str:
    if v is None:
        return "none"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, float):
        if v == int(v) and abs(v) < 1e15:
            return repr(float(v))
        return repr(v)
    if isinstance(v, str):
        return v if _NAME.match(v) and v not in ("true", "false", "none") else f'"{v}"'
    if isinstance(v, (list, tuple)):
        inner = ", ".join(value_to_source(x) for x in v)
        return f"[{inner}{',' if len(v) == 1 else ''}]"
    if isinstance(v, T.MixtureConfig):
        return " + ".join(f"{value_to_source(w.weight)} * {value_to_source(w.source)}" for w in v.sources)
    if isinstance(v, T.ObjectiveConfig):
        parts = [f"{value_to_source(t.weight)} * {t.metric}" for t in v.terms]
        if v.constant:
            parts.append(value_to_source(v.constant))
        return " + ".join(parts)
    if isinstance(v, BaseModel):
        return config_to_source(v)
    return repr(v)


def config_to_source(c: BaseModel, extra: tuple = ()) -> str:
    tag = getattr(c, "type", type(c).__name__)
    fields = []
    for name, f in type(c).model_fields.items():
        if name == "type":
            continue
        value = getattr(c, name)
        if not f.is_required() and value == f.default:
            continue
        fields.append(f"{name}={value_to_source(value)}")
    fields += list(extra)
    return f"{tag}({', '.join(fields)})"


def port_to_source(p: ir.Port) -> str:
    mark = "@" if p.mode == "write" else "$"
    return f"{p.name}={mark}{p.tap}{'!' if p.mode == 'pop' else ''}"


class _GraphPrinter:
    def __init__(self):
        self.defs: dict = {}    # name -> (key, source)
        self.order: list = []

    def name_for(self, node) -> str:
        key = ir.strip(node, labels=False, widths=True).model_dump_json()
        base = node.label if _NAME.match(node.label or "") else "block"
        base = re.sub(r"\W+", "_", node.label) if not _NAME.match(node.label or "") else base
        base = base.strip("_") or "block"
        if base[0].isdigit():
            base = "b_" + base
        name, k = base, 1
        while name in self.defs and self.defs[name][0] != key:
            k += 1
            name = f"{base}_{k}"
        if name not in self.defs:
            self.defs[name] = (key, None)
            body = self.body(node)
            shared = "shared " if node.share is not None else ""
            self.defs[name] = (key, f"{shared}{name} = {body}")
            self.order.append(name)
        return name

    def expr(self, node, min_prec: int = 0) -> str:
        if node.label is not None and node.label not in ("model",):
            return self.name_for(node)
        text, prec = self.raw(node)
        return f"({text})" if prec < min_prec else text

    def body(self, node) -> str:
        return self.raw(node)[0]

    def raw(self, node) -> tuple:
        if isinstance(node, ir.Layer):
            c = node.config
            ports = tuple(port_to_source(p) for p in node.ports)
            if c.type == "act":
                return c.fn, 9
            src = config_to_source(c, ports)
            if src.endswith("()"):
                src = src[:-2]
            return src, 9
        if isinstance(node, ir.Seq):
            if not node.items:
                return "_", 9
            return " ".join(self.expr(n, 3 + (not isinstance(n, ir.Seq)) * 0) if not isinstance(n, (ir.Sum, ir.Prod))
                            else f"({self.expr(n)})" for n in node.items), 3
        if isinstance(node, ir.Residual):
            return f"[{self.expr(node.body)}]", 9
        if isinstance(node, ir.Sum):
            out = []
            for i, n in enumerate(node.terms):
                if isinstance(n, ir.Neg) and i > 0:
                    out.append("- " + self.expr(n.body, 2))
                elif isinstance(n, ir.Const) and n.value < 0 and i > 0:
                    out.append("- " + value_to_source(-n.value))
                else:
                    out.append(("+ " if i else "") + self.expr(n, 2))
            return " ".join(out), 1
        if isinstance(node, ir.Prod):
            return " * ".join(self.expr(n, 3) for n in node.factors), 2
        if isinstance(node, ir.Neg):
            return "-" + self.expr(node.body, 4), 4
        if isinstance(node, ir.Const):
            return value_to_source(float(node.value)), 9
        if isinstance(node, ir.Identity):
            return "_", 9
        if isinstance(node, ir.Repeat):
            return f"{self.expr(node.body, 6)}^{node.times}", 5
        if isinstance(node, ir.Tap):
            return f"@{node.name}", 9
        if isinstance(node, ir.Ref):
            return f"${node.name}{'!' if node.pop else ''}", 9
        raise AssertionError(node)


def to_source(arch: ir.Architecture) -> str:
    lines = [f"d_model = {arch.d_model}"]
    if arch.vocab_size is not None:
        lines.append(f"vocab_size = {arch.vocab_size}")
    if arch.residual is not None:
        lines.append(f"residual = {config_to_source(arch.residual)}")
    if arch.init is not None:
        lines.append(f"init = {config_to_source(arch.init)}")
    gp = _GraphPrinter()
    graph = arch.graph
    top = graph.model_copy(update={"label": None})
    model = gp.body(top)
    defs = [gp.defs[n][1] for n in gp.order]
    out = "\n".join(lines) + "\n\n"
    if defs:
        out += "\n".join(defs) + "\n\n"
    return out + f"model = {model}\n"


def run_to_source(run: ir.Run) -> str:
    text = f"# {run.name}, run {run.id}\n" + to_source(run.arch) + "\n"
    t = run.train
    for name, f in type(t).model_fields.items():
        value = getattr(t, name)
        if not f.is_required() and value == f.default:
            continue
        text += f"{name} = {value_to_source(value)}\n"
    return text
