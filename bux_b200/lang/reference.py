"""What the schemas and the catalogue say about every layer and setting, as Markdown: the
editor's hovers (`bux_b200.lang.lsp`) and the reference pages (``python -m
bux_b200.lang.reference``) are made of the same pieces.

Names, types and defaults come from the pydantic schemas (`bux_b200.config.layers`,
`bux_b200.config.training`); the prose comes from `bux_b200.config.docs`. A type is written
the way its values are written in a ``.bux`` file (``int | none``, ``relu | gelu``,
``rope``), a default the way the printer writes it (``1e-06``, ``none``, ``rope()``).
Reference: ``lang/reference.py:38-195``.
"""

from __future__ import annotations

import types
import typing
from functools import lru_cache

from ..config import docs
from ..config import layers as L
from ..config import training as T
from .printer import value_to_source

TYPES = {**L.LAYERS, **L.SUBCONFIGS, **L.RESIDUALS, **L.INITS, **T.TRAINING, **T.DISTRIBUTIONS}


def members(annotation) -> list:
    """The alternatives of an annotation, with `Annotated` and unions opened."""
    origin = typing.get_origin(annotation)
    if origin is typing.Annotated:
        return members(typing.get_args(annotation)[0])
    if origin in (typing.Union, types.UnionType):
        return [m for a in typing.get_args(annotation) for m in members(a)]
    return [annotation]


def config_classes(annotation) -> list:
    """The config classes a field's annotation takes (through tuples and lists too)."""
    out = []
    for m in members(annotation):
        if isinstance(m, type) and issubclass(m, L.Config):
            out.append(m)
        elif typing.get_origin(m) in (tuple, list):
            out += [c for a in typing.get_args(m) if a is not Ellipsis for c in config_classes(a)]
    return out


def tags(cls) -> tuple:
    """The names a config is called by in a ``.bux`` file."""
    f = cls.model_fields.get("type")
    if f is None:
        return ()
    return tuple(a for m in members(f.annotation) for a in typing.get_args(m))


def literals(annotation) -> list:
    """The literal options an annotation allows (strings written bare in a file)."""
    return [a for m in members(annotation) if typing.get_origin(m) is typing.Literal for a in typing.get_args(m)]


def type_text(annotation) -> str:
    parts = []
    for m in members(annotation):
        origin = typing.get_origin(m)
        if origin is typing.Literal:
            parts += [value_to_source(a) for a in typing.get_args(m)]
        elif m is type(None):
            parts.append("none")
        elif isinstance(m, type) and issubclass(m, L.Config):
            parts += tags(m) or (m.__name__,)
        elif origin in (tuple, list):
            inner = " | ".join(dict.fromkeys(type_text(a) for a in typing.get_args(m) if a is not Ellipsis))
            parts.append(f"list of {inner}")
        else:
            parts.append(getattr(m, "__name__", str(m)))
    return " | ".join(dict.fromkeys(parts))


def default_text(f) -> str:
    return value_to_source(f.get_default(call_default_factory=True))


def field_doc(cls, name: str, tag: typing.Optional[str] = None) -> str:
    """One line on a field: ``"`eps: float = 1e-06` — note"`` or ``"`num_heads: int` (required)"``."""
    f = cls.model_fields[name]
    text = f"`{name}: {type_text(f.annotation)}"
    text += "` (required)" if f.is_required() else f" = {default_text(f)}`"
    note = next((n for t in ((tag,) if tag else ()) + tags(cls) if (n := docs.note(t, name))), "")
    return text + (f" — {note}" if note else "")


def kind_of(name: str) -> str:
    if name in L.LAYERS:
        return "layer"
    if name in L.RESIDUALS:
        return "residual algebra"
    if name in L.INITS:
        return "initialiser"
    if name in T.DISTRIBUTIONS:
        return "search dimension"
    return "setting"


@lru_cache(maxsize=None)
def type_doc(name: str) -> str:
    """The Markdown on the config called `name`: heading, summary, one line a field, ports."""
    cls = TYPES[name]
    parts = [f"**{name}** — {kind_of(name)}"]
    if name in docs.SUMMARY:
        parts.append(docs.SUMMARY[name])
    elif cls.__dict__.get("__doc__"):
        parts.append(cls.__doc__.strip().split("\n\n")[0])
    fields = [f for f in cls.model_fields if f != "type"]
    if fields:
        parts.append("\n".join(f"- {field_doc(cls, f, name)}" for f in fields))
    ports = sorted(getattr(cls, "ports", ()))
    if ports:
        parts.append("Ports: " + ", ".join(f"`{p}`" for p in ports))
    return "\n\n".join(parts)


def activation_doc(name: str) -> str:
    return (f"**{name}** — activation\n\nA layer that applies it elementwise (`linear(features=h) {name}`), "
            f"or a value of settings such as `activation={name}`.")


def setting_doc(name: str) -> str:
    """The Markdown on a top-level setting of a file (`steps`, `optimizer`, `d_model`, ...)."""
    if name in docs.MODEL_SETTINGS:
        return f"**{name}** — model setting\n\n{docs.MODEL_SETTINGS[name]}"
    f = T.TrainConfig.model_fields[name]
    head = f"`{name}: {type_text(f.annotation)}" + ("` (required)" if f.is_required() else f" = {default_text(f)}`")
    note = docs.TRAIN_FIELDS.get(name, "")
    return f"**{name}** — training setting\n\n{head}" + (f" — {note}" if note else "")


# ------------------------------------------------------------------------------ pages
def _section(title: str, names) -> str:
    return "\n\n".join([f"# {title}", *(("## `%s`\n\n" % n) + type_doc(n).split("\n\n", 1)[-1] for n in names)])


def layers() -> str:
    acts = "\n".join(f"- `{a}`" for a in L.ACTIVATIONS)
    return "\n\n".join([
        _section("Layers", sorted(L.LAYERS)),
        "# Activations\n\nEach is a layer and a value of `activation=` settings.\n\n" + acts,
        _section("Layer parts", sorted(set(L.SUBCONFIGS) - set(L.RESIDUALS) - set(L.INITS))),
        _section("Residual algebras", sorted(L.RESIDUALS)),
        _section("Initialisers", sorted(L.INITS)),
    ])


def settings() -> str:
    top = "\n".join(f"- {setting_doc(n).split(chr(10) + chr(10), 1)[1]}"
                    for n in (*docs.MODEL_SETTINGS, *T.TrainConfig.model_fields))
    return "\n\n".join(["# Settings of a file\n\n" + top,
                        _section("Training settings", sorted(set(T.TRAINING) - set(T.DISTRIBUTIONS))),
                        _section("Search dimensions", sorted(T.DISTRIBUTIONS))])


def reference() -> str:
    return layers() + "\n\n" + settings() + "\n"


def undocumented() -> list:
    """``tag`` and ``tag.field`` names the catalogue says nothing about (a to-do list)."""
    out = [t for t in TYPES if t not in docs.SUMMARY]
    for t, cls in TYPES.items():
        out += [f"{t}.{f}" for f in cls.model_fields if f != "type" and not docs.note(t, f)]
    return sorted(out)


if __name__ == "__main__":
    print(reference(), end="")
