"""Structural edits of a ``.bux`` source, each one a splice of the text.

An edit lands where the file writes what it changes, and the rest of the file (comments,
macros, patterns, alignment) stays as it was. Every function returns the new source; the
caller compiles it again before it draws it. Offsets are into the buffer.

* `set_field`: one setting of a call (``gqa(num_heads=4)``): replaced where it is written,
  added to the call when it is not, removed when set back to nothing. A name that is a
  definition is changed at its definition; one defined in a module, by an amendment in this
  file (``attn.num_heads = 12``).
* `set_setting`: a top-level statement (``steps = 200``), replaced or appended;
  `set_setting_field`: one field of a setting written as a call (``schedule = wsd(warmup=20)``).
* `insert`, `delete`, `wrap`, `unwrap`, `set_repeat`: the graph's shape, at a node's span.
* `alt_replace`, `alt_add`, `alt_remove`: one alternative of a sweep axis.

`EditError` says why an edit cannot be made where it is asked (a macro's parameter, one
letter of a pattern, ...). Reference: ``studio/edits.py``.
"""

from __future__ import annotations

import re
from typing import Optional

from ..lang import syntax as S
from ..lang.lsp import features


class EditError(ValueError):
    """An edit that has no place in the file's text; the message says why."""


def splice(source: str, start: int, end: int, text: str) -> str:
    return source[:start] + text + source[end:]


# ------------------------------------------------------------------------------ finding things
def _walk(e):
    yield e
    for name in ("items", "options"):
        for k in getattr(e, name, ()) or ():
            yield from _walk(k)
    for name in ("body", "operand", "left", "right", "base"):
        k = getattr(e, name, None)
        if isinstance(k, S.Expr):
            yield from _walk(k)
    for a in getattr(e, "args", ()) or ():
        yield from _walk(a.value)


def node_at(ix: features.Index, start: int, end: int):
    """The smallest expression of the buffer whose span is exactly [start, end), with its statement."""
    for st in ix.own:
        if st.body is None:
            continue
        for e in _walk(st.body):
            if e.span.start - ix.base == start and e.span.end - ix.base == end:
                return e, st
    return None, None


def _call_of(ix: features.Index, name: str, seen=()):
    """The call that writes the settings of the definition `name` (following ``a = b``),
    with the statement and file it is in; (None, statement, file) when it is a bare builtin."""
    hit = ix.names.get(name)
    if hit is None or name in seen:
        return None, None, None
    st, file = hit
    body = st.body
    if isinstance(body, S.Alt):
        raise EditError(f"'{name}' is a sweep's alternatives: edit the alternative itself")
    if isinstance(body, S.Call):
        return body, st, file
    if isinstance(body, S.Name):
        if body.name in ix.names:
            return _call_of(ix, body.name, (*seen, name))
        return None, st, file          # ``norm = rmsnorm``: a bare builtin, no call yet
    raise EditError(f"'{name}' is not written as a call: its settings cannot be set here")


# ------------------------------------------------------------------------------ settings of a call
def set_field(source: str, start: int, end: int, key: str, value: Optional[str], path: Optional[str] = None) -> str:
    """Set `key` (dotted for a nested setting: ``rope.base``) of what is written at [start, end)
    to the source text `value`; None removes it (back to its default)."""
    ix = features.Index(source, path)
    e, st = node_at(ix, start, end)
    if e is None:
        raise EditError("nothing is written at that place any more: the drawing is behind the text")
    keys = tuple(key.split("."))
    params = {p.name for p in (st.params or ())}
    if isinstance(e, S.Name) and e.name in params:
        raise EditError(f"'{e.name}' is a parameter of the macro '{st.name}': its settings are those of what each call passes")
    if isinstance(e, S.Lit) or (isinstance(e, S.Name) and len(e.name) == 1 and source[start - 1:start] == '"'):
        raise EditError("one letter of a pattern cannot be changed alone: change the definition it names, or the whole pattern")
    if isinstance(e, S.Call) and e.name not in ix.names:
        return _in_call(source, e, ix.base, keys, value)            # ``gqa(...)`` written in place
    name = e.name if isinstance(e, (S.Name, S.Call)) else None
    if name is None:
        raise EditError("this is a block, not a layer: select one of its layers")
    if name not in ix.names:                                          # a bare builtin: ``rmsnorm`` -> ``rmsnorm(eps=1e-5)``
        if value is None:
            return source
        return splice(source, end, end, f"({key}={value})")
    call, dst, file = _call_of(ix, name)
    if file != ix.path:
        return _amend(source, name, key, value)                       # defined in a module: amend it here
    if call is None:                                                  # ``norm = rmsnorm``
        at = dst.body.span.end - ix.base
        return source if value is None else splice(source, at, at, f"({key}={value})")
    return _in_call(source, call, ix.base, keys, value)


def _in_call(source: str, call: S.Call, base: int, keys: tuple, value: Optional[str]) -> str:
    for a in call.args:
        if a.key == keys:
            s, e = a.span.start - base, a.span.end - base
            if value is None:                                         # drop the argument and one comma
                rest = source[e:]
                m = re.match(r"\s*,\s*", rest)
                if m:
                    return splice(source, s, e + m.end(), "")
                before = re.search(r",\s*$", source[:s])
                return splice(source, before.start() if before else s, e, "")
            vs, ve = a.value.span.start - base, a.value.span.end - base
            return splice(source, vs, ve, value)
        if a.key and a.key == keys[:1] and len(keys) > 1 and isinstance(a.value, S.Call):
            return _in_call(source, a.value, base, keys[1:], value)   # ``rope=rope(...)``: inside it
    if value is None:
        return source
    close = call.span.end - base - 1
    if source[close] != ")":                                          # a call without parentheses cannot be here
        raise EditError("this call's settings are not written between parentheses")
    inner = source[call.name_span.end - base:close]
    empty = inner.strip() in ("(", "")
    return splice(source, close, close, ("" if empty else ", ") + f"{'.'.join(keys)}={value}")


def _amend(source: str, name: str, key: str, value: Optional[str]) -> str:
    pat = re.compile(rf"^{re.escape(name)}\.{re.escape(key)}\s*=.*$", re.M)
    m = pat.search(source)
    if value is None:
        return source if m is None else splice(source, m.start(), min(len(source), m.end() + 1), "")
    line = f"{name}.{key} = {value}"
    if m is not None:
        return splice(source, m.start(), m.end(), line)
    # after the last `use`, so the amendment follows the module it amends
    uses = list(re.finditer(r"^use\s+.*$", source, re.M))
    at = uses[-1].end() if uses else 0
    return splice(source, at, at, ("\n" if uses else "") + line + ("" if uses else "\n"))


def set_setting(source: str, name: str, value: Optional[str]) -> str:
    """The statement ``name = value`` replaced where the file writes it (continuation lines
    included), appended when it does not, removed for None."""
    nl = "\r\n" if "\r\n" in source else "\n"
    lines = source.split(nl)
    pat = re.compile(rf"^{re.escape(name)}\s*=")
    for i, line in enumerate(lines):
        if pat.match(line):
            j = i + 1
            while j < len(lines) and lines[j][:1] in (" ", "\t") and lines[j].strip():
                j += 1
            new = [] if value is None else [f"{name} = {value}"]
            return nl.join([*lines[:i], *new, *lines[j:]])
    if value is None:
        return source
    return source.rstrip("\r\n") + f"{nl}{name} = {value}{nl}"


def set_setting_field(source: str, name: str, key: str, value: Optional[str], kind: Optional[str] = None,
                      path: Optional[str] = None) -> str:
    """One field of a top-level setting written as a call (``schedule = wsd(warmup=20)``): the
    field replaced, added or removed inside the call and the rest of it kept. A setting the
    file does not write is appended as ``name = kind(key=value)``."""
    ix = features.Index(source, path)
    st = next((s for s in ix.own if s.name == name and not s.amends and s.body is not None), None)
    if st is None:
        if value is None:
            return source
        if kind is None:
            raise EditError(f"the file does not set '{name}': say which type to write")
        return set_setting(source, name, f"{kind}({key}={value})")
    body = st.body
    if isinstance(body, S.Call):
        return _in_call(source, body, ix.base, tuple(key.split(".")), value)
    if isinstance(body, S.Name):
        at = body.span.end - ix.base
        return source if value is None else splice(source, at, at, f"({key}={value})")
    raise EditError(f"'{name}' is not written as one call (a sweep's alternatives, say): edit it in the source")


# ------------------------------------------------------------------------------ the graph's shape
def _checked(source: str, start: int, end: int, path) -> None:
    ix = features.Index(source, path)
    e, _ = node_at(ix, start, end)
    if e is None:
        raise EditError("nothing is written at that place any more: the drawing is behind the text")
    if source[max(0, start - 1):start] == '"' or source[end:end + 1] == '"' or isinstance(e, S.Lit):
        raise EditError("a pattern's letters stand for definitions: change the definition, or write the pattern out")


def insert(source: str, start: int, end: int, text: str, after: bool = True, path: Optional[str] = None) -> str:
    """`text` composed after (or before) what is written at [start, end)."""
    _checked(source, start, end, path)
    return splice(source, end, end, " " + text) if after else splice(source, start, start, text + " ")


def delete(source: str, start: int, end: int, path: Optional[str] = None) -> str:
    _checked(source, start, end, path)
    s, e = start, end
    if source[e:e + 1] == " ":
        e += 1
    elif source[s - 1:s] == " ":
        s -= 1
    out = splice(source, s, e, "")
    if re.search(r"\[\s*\]|\(\s*\)(?!\s*=)", out[max(0, s - 2):s + 2]):
        raise EditError("that would leave an empty branch: delete the branch instead")
    return out


def wrap(source: str, start: int, end: int, path: Optional[str] = None) -> str:
    """``f`` -> ``[f]``: a residual branch around what is written there."""
    _checked(source, start, end, path)
    return splice(source, start, end, "[" + source[start:end] + "]")


def unwrap(source: str, start: int, end: int, path: Optional[str] = None) -> str:
    _checked(source, start, end, path)
    text = source[start:end]
    if not (text.startswith("[") and text.endswith("]")):
        raise EditError("that is not a residual branch")
    inner = text[1:-1].strip()
    needs = bool(re.search(r"[+|]|(?<![\w)\]])-", inner)) and " " in inner
    return splice(source, start, end, f"({inner})" if needs else inner)


def set_repeat(source: str, start: int, end: int, times: int, path: Optional[str] = None) -> str:
    """``f^n`` with a new count (at the repeat's own span), or ``f`` -> ``f^n``."""
    if times < 1:
        raise EditError("a repeat runs at least once")
    text = source[start:end]
    m = re.search(r"\^\s*(\d+)\s*$", text)
    if m:
        return splice(source, start + m.start(1), start + m.end(1), str(times))
    m = re.search(r"\^\s*([A-Za-z_]\w*)\s*$", text)
    if m:
        return set_setting(source, m.group(1), str(times))           # ``block^depth``: the count is a definition
    needs = " " in text.strip() and not (text.startswith(("(", "[")) and text.endswith((")", "]")))
    return splice(source, start, end, (f"({text})" if needs else text) + f"^{times}")


# ------------------------------------------------------------------------------ sweeps
def alt_replace(source: str, start: int, end: int, text: str) -> str:
    return splice(source, start, end, text)


def alt_add(source: str, last_start: int, last_end: int, text: str, label: Optional[str] = None) -> str:
    """A new alternative after the one written at [last_start, last_end), laid out as that one is
    (on a line of its own when the alternatives are written a line each)."""
    line_start = source.rfind("\n", 0, last_start) + 1
    lead = source[line_start:last_start]
    item = (f"{label}: " if label else "") + text
    m = re.match(r"(\s*)\|\s*(?:[A-Za-z_]\w*\s*:\s*)?$", lead)
    if m is not None:                                                  # ``    | name: value`` lines
        return splice(source, last_end, last_end, "\n" + m.group(1) + "| " + item)
    return splice(source, last_end, last_end, " | " + item)


def alt_remove(source: str, start: int, end: int) -> str:
    """Remove one alternative with its ``|`` (and its label), leaving the others' lines alone."""
    s = start
    label = re.search(r"[A-Za-z_]\w*\s*:\s*$", source[:s])
    if label:
        s = label.start()
    before = re.search(r"[ \t]*\|\s*$", source[:s])
    if before is not None:
        s = before.start()
        # a line that held only this alternative goes too
        line_start = source.rfind("\n", 0, s) + 1
        if not source[line_start:s].strip() and line_start > 0:
            s = line_start - 1
        return splice(source, s, end, "")
    after = re.match(r"\s*\|\s*", source[end:])
    if after is None:
        raise EditError("the last alternative cannot be removed: write the value instead of the sweep")
    return splice(source, s, end + after.end(), "")


OPERATIONS = {"set_field": set_field, "set_setting": set_setting, "set_setting_field": set_setting_field, "insert": insert, "delete": delete, "wrap": wrap,
              "unwrap": unwrap, "set_repeat": set_repeat, "alt_replace": alt_replace, "alt_add": alt_add,
              "alt_remove": alt_remove}


def apply(source: str, edit: dict, path: Optional[str] = None) -> str:
    """Run one edit given as ``{"op": name, ...arguments}``."""
    op = edit.get("op")
    if op not in OPERATIONS:
        raise EditError(f"no edit called {op!r}")
    args = {k: v for k, v in edit.items() if k != "op"}
    if op in ("set_field", "set_setting_field", "insert", "delete", "wrap", "unwrap", "set_repeat"):
        args["path"] = path
    return OPERATIONS[op](source, **args)
