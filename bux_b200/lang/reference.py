"""Reference pages generated from the schemas: every layer type and every training
setting with its fields, types and defaults (``bux reference``). Reference:
``lang/reference.py``."""

from __future__ import annotations

from ..config import layers as L
from ..config import training as T


def _fields(cls) -> list:
    rows = []
    for name, f in cls.model_fields.items():
        if name == "type":
            continue
        default = "required" if f.is_required() else repr(f.default)
        ann = getattr(f.annotation, "__name__", None) or str(f.annotation).replace("typing.", "")
        rows.append((name, ann, default))
    return rows


def _table(rows: list) -> str:
    if not rows:
        return "_no settings_\n"
    w = [max(len(str(r[i])) for r in rows + [("field", "type", "default")]) for i in range(3)]
    line = lambda r: "| " + " | ".join(str(c).ljust(n) for c, n in zip(r, w)) + " |"
    return "\n".join([line(("field", "type", "default")), "|" + "|".join("-" * (n + 2) for n in w) + "|",
                      *(line(r) for r in rows)]) + "\n"


def layers() -> str:
    out = ["# Layers\n"]
    for tag, cls in sorted(L.LAYERS.items()):
        ports = ", ".join(sorted(getattr(cls, "ports", ()))) or "none"
        out.append(f"## `{tag}`\n\nports: {ports}\n\n{_table(_fields(cls))}")
    out.append("# Residual algebras\n")
    for tag, cls in sorted(L.RESIDUALS.items()):
        out.append(f"## `{tag}`\n\n{_table(_fields(cls))}")
    return "\n".join(out)


def settings() -> str:
    out = ["# Training settings\n", _table(_fields(T.TrainConfig))]
    for tag, cls in sorted(T.TRAINING.items()):
        out.append(f"## `{tag}`\n\n{_table(_fields(cls))}")
    return "\n".join(out)


def reference() -> str:
    return layers() + "\n" + settings()
