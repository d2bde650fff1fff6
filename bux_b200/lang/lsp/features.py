"""Language features over a `.bux` source text: diagnostics, hover, completion,
go-to-definition. Pure functions (positions are 0-based line / character), so the
server and the tests share them. Reference: ``lang/lsp/features.py``."""

from __future__ import annotations

import re
from typing import Optional

from ...config import layers as L
from ...config import training as T
from .. import compiler, syntax

WORD = re.compile(r"[A-Za-z_][A-Za-z0-9_]*")


def _line_col(source: str, offset: int) -> tuple:
    before = source[:offset]
    line = before.count("\n")
    return line, offset - (before.rfind("\n") + 1)


def _offset(source: str, line: int, character: int) -> int:
    lines = source.split("\n")
    return sum(len(x) + 1 for x in lines[:line]) + min(character, len(lines[line]) if line < len(lines) else 0)


def diagnostics(source: str, filename: str = "<buffer>") -> list:
    """[{range, message, hint}] for every mistake `check` finds (not only the first)."""
    try:
        report = compiler.check(source, filename=filename)
        errors = report.errors
    except syntax.BuxError as err:
        errors = [err]
    out = []
    for e in errors:
        span = getattr(e, "span", None)
        start = _line_col(source, span.start) if span is not None else (0, 0)
        end = _line_col(source, span.end) if span is not None else (0, 1)
        out.append({"range": {"start": {"line": start[0], "character": start[1]},
                              "end": {"line": end[0], "character": end[1]}},
                    "severity": 1, "source": "bux",
                    "message": e.message + (f"\nhint: {e.hint}" if getattr(e, "hint", None) else "")})
    return out


def word_at(source: str, line: int, character: int) -> Optional[tuple]:
    """(word, start offset, end offset) under the position."""
    at = _offset(source, line, character)
    for m in WORD.finditer(source):
        if m.start() <= at <= m.end():
            return m.group(0), m.start(), m.end()
    return None


def _schema(name: str):
    return L.LAYERS.get(name) or L.SUBCONFIGS.get(name) or L.RESIDUALS.get(name) or L.INITS.get(name) \
        or T.TRAINING.get(name) or T.DISTRIBUTIONS.get(name)


def _describe(cls) -> str:
    rows = []
    for n, f in cls.model_fields.items():
        if n == "type":
            continue
        rows.append(f"  {n}" + ("" if f.is_required() else f" = {f.default!r}"))
    doc = (cls.__doc__ or "").strip().split("\n\n")[0]
    return (doc + "\n" if doc else "") + "\n".join(rows)


def definitions(source: str) -> dict:
    """name → (line, character) of its definition ``name = ...`` / ``name(args) = ...``."""
    out = {}
    for m in re.finditer(r"^([A-Za-z_][A-Za-z0-9_]*)\s*(\([^)]*\))?\s*=", source, re.M):
        out.setdefault(m.group(1), _line_col(source, m.start(1)))
    return out


def hover(source: str, line: int, character: int) -> Optional[str]:
    hit = word_at(source, line, character)
    if hit is None:
        return None
    word = hit[0]
    cls = _schema(word)
    if cls is not None:
        return f"{word}(...)\n{_describe(cls)}"
    if word in T.TrainConfig.model_fields:
        f = T.TrainConfig.model_fields[word]
        return f"setting `{word}`" + ("" if f.is_required() else f" (default {f.default!r})")
    where = definitions(source).get(word)
    if where is not None:
        text = source.split("\n")[where[0]].strip()
        return f"defined on line {where[0] + 1}: {text}"
    return None


def completion(source: str, line: int, character: int) -> list:
    """Names that fit at the position: fields inside a call's parentheses, else layers,
    settings and the file's own definitions."""
    at = _offset(source, line, character)
    before = source[:at]
    prefix = re.search(r"[A-Za-z_0-9]*$", before).group(0)
    depth, i = 0, len(before) - 1
    callee = None
    while i >= 0:
        ch = before[i]
        if ch == ")":
            depth += 1
        elif ch == "(":
            if depth == 0:
                m = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", before[:i])
                callee = m.group(1) if m else None
                break
            depth -= 1
        elif ch == "\n" and depth == 0 and (i + 1 >= len(before) or not before[i + 1].isspace()):
            break
        i -= 1
    items = []
    cls = _schema(callee) if callee else None
    if cls is not None:
        items = [{"label": n, "kind": 5, "insertText": f"{n}="} for n in cls.model_fields if n != "type"]
        items += [{"label": p, "kind": 5, "insertText": f"{p}="} for p in sorted(getattr(cls, "ports", ()))]
    else:
        items = [{"label": n, "kind": 3} for n in sorted({*L.LAYERS, *L.RESIDUALS, *T.TRAINING, *T.DISTRIBUTIONS})]
        items += [{"label": n, "kind": 10} for n in T.TrainConfig.model_fields]
        items += [{"label": n, "kind": 6} for n in definitions(source)]
    return [it for it in items if it["label"].startswith(prefix)]


def definition(source: str, line: int, character: int) -> Optional[dict]:
    hit = word_at(source, line, character)
    if hit is None:
        return None
    where = definitions(source).get(hit[0])
    if where is None:
        return None
    return {"start": {"line": where[0], "character": where[1]},
            "end": {"line": where[0], "character": where[1] + len(hit[0])}}
