"""The inspector: the settings of what is selected, field by field.

`inspect(source, start, end)` answers, for the layer written at that span, every field of
its config with its type as the page should edit it (``bool``, ``int``, ``float``,
``choice`` with its options, ``config`` with the types it takes, ``text``), its value now,
its default, whether the file sets it, a note, and, when the field cannot be set where the
layer is written, why. Reference: ``studio/forms.py``.
"""

from __future__ import annotations

import typing
from typing import Optional

from ..config import layers as L
from ..lang import ir, reference
from ..lang import syntax as S
from ..lang.lsp import features
from ..lang.printer import value_to_source
from . import edits


def field_kind(annotation) -> dict:
    members = reference.members(annotation)
    options = [o for o in reference.literals(annotation) if isinstance(o, (str, int))]
    classes = reference.config_classes(annotation)
    optional = type(None) in members
    if classes:
        return {"kind": "config", "types": sorted({t for c in classes for t in reference.tags(c)}), "optional": optional}
    if options and all(typing.get_origin(m) is typing.Literal or m is type(None) or m is bool for m in members):
        return {"kind": "choice", "options": [value_to_source(o) for o in options] + (["true", "false"] if bool in members else []),
                "optional": optional}
    if bool in members and len([m for m in members if m is not type(None)]) == 1:
        return {"kind": "bool", "optional": optional}
    if int in members and float not in members:
        return {"kind": "int", "optional": optional}
    if float in members or int in members:
        return {"kind": "float", "optional": optional}
    return {"kind": "text", "optional": optional}


def _config_at(ix: features.Index, e):
    """(config class, config value or None, name shown) of the expression."""
    if isinstance(e, S.Call) and e.name not in ix.names:
        cls = ix.cls_of(e.name)
        return cls, None, e.name
    name = getattr(e, "name", None)
    if name is None:
        return None, None, None
    cls = ix.cls_of(name)
    value = ix.value_of(name)
    cfg = value.config if isinstance(value, ir.Layer) else value
    return cls, cfg if isinstance(cfg, L.Config) else None, name


def inspect(source: str, start: int, end: int, path: Optional[str] = None) -> dict:
    ix = features.Index(source, path)
    e, st = edits.node_at(ix, start, end)
    if e is None:
        return {"fields": [], "why": "nothing is written at that place"}
    params = {p.name for p in (st.params or ())}
    if getattr(e, "name", None) in params:
        return {"fields": [], "name": e.name,
                "why": f"'{e.name}' is a parameter of the macro '{st.name}': each call passes its own layer"}
    cls, cfg, name = _config_at(ix, e)
    if cls is None:
        return {"fields": [], "name": name, "why": "a block: select one of its layers to see settings"}
    why = None
    written: dict = {}
    call = e if isinstance(e, S.Call) and e.name not in ix.names else None
    where = ix.path
    if call is None and name in ix.names:
        try:
            call, _, where = edits._call_of(ix, name)
        except edits.EditError as err:
            why = str(err)
    for a in (call.args if call is not None else ()):
        if a.key:
            written[".".join(a.key)] = " ".join(ix.text[a.value.span.start:a.value.span.end].split())
    tag = ix.leads_to(name) if name in ix.names else name
    fields = []
    for fname, f in cls.model_fields.items():
        if fname == "type":
            continue
        now = getattr(cfg, fname) if cfg is not None else (None if f.is_required() else f.get_default(call_default_factory=True))
        fields.append({"name": fname, **field_kind(f.annotation), "required": f.is_required(),
                       "default": None if f.is_required() else reference.default_text(f),
                       "value": written.get(fname, value_to_source(now) if now is not None or not f.is_required() else ""),
                       "written": fname in written, "note": reference.docs.note(tag, fname) if tag else ""})
    return {"name": name, "type": tag, "doc": reference.docs.SUMMARY.get(tag, ""), "fields": fields, "why": why,
            "module": None if where == ix.path else where, "ports": sorted(getattr(cls, "ports", ()))}
