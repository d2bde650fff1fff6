"""Language features over a ``.bux`` source text: diagnostics, hover, completion and
go-to-definition, as plain functions of (text, offset) so that the stdio server and the
tests share them.

The features read the parsed statements (`bux_b200.lang.syntax`), with the modules the
file uses loaded as the compiler loads them, so a name defined in a module hovers and
completes like one of the file's own. What a name *is* comes from following definitions
down to a builtin (``local = attn(...)``, ``attn = gqa(...)`` makes ``local(`` offer
gqa's settings); what a definition *evaluates to* comes from the compiler's evaluator.
Prose comes from `bux_b200.lang.reference`. Reference: ``lang/lsp/features.py:71-759``.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Iterator, Optional

from ...config import layers as L
from ...config import training as T
from .. import compiler, ir, reference
from .. import syntax as S
from ..printer import config_to_source, value_to_source


@dataclass(frozen=True)
class Diagnostic:
    start: int
    end: int
    message: str


@dataclass(frozen=True)
class Completion:
    label: str
    kind: str = "text"      # field, value, layer, setting, definition, parameter, tap, keyword
    detail: str = ""
    doc: str = ""
    insert: Optional[str] = None
    sort: str = "5"


@dataclass(frozen=True)
class Hover:
    start: int
    end: int
    text: str


# ------------------------------------------------------------------------------ diagnostics
def diagnostics(source: str, path: Optional[str] = None) -> list:
    """Every mistake `check` finds. A mistake inside a module shows at the ``use`` that
    brought the module in, prefixed with the module's file and line."""
    name = path or "<buffer>"
    try:
        errors = compiler.check(source, filename=name).errors
    except S.BuxError as err:
        errors = [err]
    uses = {m.group(1): m.span(1) for m in re.finditer(r"^use\s+([A-Za-z_][\w.]*)", source, re.M)}
    out = []
    for e in errors:
        text = e.message + (f"\nhint: {e.hint}" if getattr(e, "hint", None) else "")
        foreign = getattr(e, "filename", None) not in (None, name)
        if foreign:
            where = e.location()
            stem = re.sub(r"\.bux$", "", str(e.filename).replace("\\", "/").rsplit("/", 1)[-1])
            at = next((span for mod, span in uses.items() if mod.split(".")[-1] == stem),
                      next(iter(uses.values()), (0, 1)))
            out.append(Diagnostic(at[0], at[1], f"{e.filename}:{where[0] if where else '?'}: {text}"))
        elif e.span is not None:
            out.append(Diagnostic(e.span.start, max(e.span.end, e.span.start + 1), text))
        else:
            out.append(Diagnostic(0, 1, text))
    return out


# ------------------------------------------------------------------------------ the index
_ALL_TYPES = reference.TYPES
_TOP = (*compiler.SETTINGS, *compiler.TRAIN_SETTINGS, "model")


class Index:
    """A file's statements and the modules', and what their names lead to."""

    def __init__(self, source: str, path: Optional[str] = None):
        self.source, self.path = source, path or "<buffer>"
        self.base = 0                      # where the buffer starts inside the program's text
        self.program = None
        try:
            self.program = compiler._load(source, self.path, (), None, recover=True)
        except S.BuxError:
            pass
        self.own: list = []               # the buffer's statements (spans in the program's text)
        self.names: dict = {}             # name -> (statement, file name), the last definition
        if self.program is not None:
            main = next((f for f in self.program.files if f.filename == self.path), None)
            self.base = main.start if main else 0
            for layer in self.program.layers:
                for st in layer:
                    f = self.program.file_of(st.span.start)
                    if not st.amends:
                        self.names[st.name] = (st, f.filename)
                    if main is not None and main.start <= st.span.start <= main.stop:
                        self.own.append(st)
            self.text = self.program.source
            self.ev = compiler.Evaluator(self.program, report=lambda err: None)
        else:                              # the file does not even load: its own statements only
            errors: list = []
            try:
                self.own = list(S.parse(source, errors)[0])
            except S.BuxError:
                self.own = []
            self.names = {st.name: (st, self.path) for st in self.own if not st.amends and st.use is None}
            self.text, self.ev = source, None

    # -- names
    def statement(self, name: str):
        hit = self.names.get(name)
        return hit[0] if hit else None

    def leads_to(self, name: str, seen: tuple = ()) -> Optional[str]:
        """The builtin type a name is, through the definitions it is written with."""
        if name in seen:
            return None
        st = self.statement(name)
        if st is None or st.params is not None:
            return name if name in _ALL_TYPES else None
        body = st.body
        while isinstance(body, S.Alt) and body.options:
            body = body.options[0]
        if isinstance(body, S.Call):
            return self.leads_to(body.name, (*seen, name)) if body.name != name else (name if name in _ALL_TYPES else None)
        if isinstance(body, S.Name):
            return self.leads_to(body.name, (*seen, name))
        return None

    def cls_of(self, name: str):
        tag = self.leads_to(name)
        return _ALL_TYPES.get(tag) if tag else None

    def value_of(self, name: str):
        """What the definition evaluates to, or None when it does not evaluate."""
        if self.ev is None or name not in self.ev.chain:
            return None
        try:
            return compiler.unwrap(self.ev.definition(name))
        except (S.BuxError, RecursionError):
            return None

    def written(self, st) -> str:
        return " ".join(self.text[st.span.start:st.span.end].split())

    def enclosing(self, offset: int):
        """The statement `offset` is in; when that statement did not parse (it is being
        typed), the definition its first line starts, if the file has one of that name."""
        at = offset + self.base
        for st in self.own:
            if st.span.start <= at <= st.span.end:
                return st
        head = self.source[:offset]
        starts = [m for m in re.finditer(r"^(?:shared\s+)?([A-Za-z_]\w*)[^\n=]*=", head, re.M)]
        if starts:
            name = starts[-1].group(1)
            return self.statement(name) or S.Statement(name, S.Span(0, 0), None, S.Span(0, 0))
        return None


def field_class(cls, name: str):
    """The config class the field `name` of `cls` takes (``rope`` of gqa -> RoPEConfig)."""
    if cls is None or name not in cls.model_fields:
        return None
    found = reference.config_classes(cls.model_fields[name].annotation)
    return found[0] if found else None


def _descend(cls, keys: tuple):
    for k in keys:
        cls = field_class(cls, k)
    return cls


# ------------------------------------------------------------------------------ occurrences
def occurrences(ix: Index) -> Iterator[tuple]:
    """(span, what) for every place of the buffer a hover can say something about. `what` is
    a tuple whose first item names the kind: ``define``, ``setting``, ``name``, ``call``,
    ``key`` (class, dotted keys), ``tap``, ``param``, ``field`` (an ``a.b`` read)."""
    for st in ix.own:
        if st.use is not None:
            yield st.name_span, ("module", st.use)
            continue
        params = {p.name for p in st.params or ()}
        kind = "setting" if st.name in _TOP and st.params is None else "define"
        yield st.name_span, (kind, st.name)
        for p in st.params or ():
            yield p.span, ("param", p.name, st.name)
            if p.default is not None:
                yield from _walk(p.default, ix, params, st, None)
        if st.body is not None:
            owner = None
            if st.amends:       # ``a.b = v``: the body is a call of `a` with the keys as arguments
                owner = ix.cls_of(st.name)
            elif st.name in T.TrainConfig.model_fields:
                found = reference.config_classes(T.TrainConfig.model_fields[st.name].annotation)
                owner = found[0] if found else None
            yield from _walk(st.body, ix, params, st, owner)


def _walk(e, ix: Index, params: set, st, expected) -> Iterator[tuple]:
    if isinstance(e, S.Name):
        yield e.span, (("param", e.name, st.name) if e.name in params else ("name", e.name, expected))
    elif isinstance(e, S.Call):
        cls = ix.cls_of(e.name) if e.name not in params else None
        if not e.amend:
            yield e.name_span, (("param", e.name, st.name) if e.name in params else ("call", e.name))
        macro = ix.statement(e.name)
        macro_params = {p.name for p in macro.params} if macro is not None and macro.params is not None else set()
        for a in e.args:
            sub = None
            if a.key:
                if a.key[0] in macro_params:
                    yield a.key_spans[0], ("param", a.key[0], e.name)
                else:
                    for i, span in enumerate(a.key_spans):
                        yield span, ("key", _descend(cls, a.key[:i]), a.key[: i + 1], e.name)
                owner = _descend(cls, a.key[:-1])
                sub = (owner, a.key[-1]) if owner is not None else None
            yield from _walk(a.value, ix, params, st, sub)
    elif isinstance(e, S.Attr):
        yield from _walk(e.base, ix, params, st, None)
        yield e.field_span, ("field", e)
    elif isinstance(e, S.Tap):
        yield e.span, ("tap", e.name)
    elif isinstance(e, S.Ref):
        yield e.span, ("tap", e.name)
    elif isinstance(e, (S.Seq, S.ListExpr)):
        for k in e.items:
            yield from _walk(k, ix, params, st, expected)
    elif isinstance(e, S.Residual):
        yield from _walk(e.body, ix, params, st, None)
    elif isinstance(e, S.Neg):
        yield from _walk(e.operand, ix, params, st, None)
    elif isinstance(e, S.BinOp):
        yield from _walk(e.left, ix, params, st, expected)
        yield from _walk(e.right, ix, params, st, expected)
    elif isinstance(e, S.Alt):
        for k in e.options:
            yield from _walk(k, ix, params, st, expected)


# ------------------------------------------------------------------------------ hover
def hover(source: str, offset: int, path: Optional[str] = None) -> Optional[Hover]:
    ix = Index(source, path)
    at = offset + ix.base
    best = None
    for span, what in occurrences(ix):
        if span.start <= at <= span.end and (best is None or span.end - span.start <= best[0].end - best[0].start):
            best = (span, what)
    if best is None:
        return None
    text = _hover_text(ix, best[1])
    if not text:
        return None
    return Hover(best[0].start - ix.base, best[0].end - ix.base, text)


def _line_of(ix: Index, offset: int) -> int:
    f = ix.program.file_of(offset) if ix.program is not None else None
    start = f.start if f else 0
    return ix.text.count("\n", start, offset) + 1


def _definition_doc(ix: Index, name: str) -> str:
    st, file = ix.names[name]
    parts = [f"```bux\n{ix.written(st)}\n```"]
    if st.doc:
        parts.insert(0, st.doc)
    if st.params is not None:
        parts.append("a macro of " + ", ".join(f"`{p.name}`" for p in st.params))
    else:
        value = ix.value_of(name)
        shown = _value_text(value)
        if shown and shown != " ".join(ix.written(st).split("=", 1)[-1].split()):
            parts.append(f"evaluates to `{shown}`")
        tag = ix.leads_to(name)
        if tag and tag != name:
            parts.append(f"a `{tag}`: {reference.docs.SUMMARY.get(tag, '')}".rstrip(": "))
    if file != ix.path:
        parts.append(f"defined in `{file}`, line {_line_of(ix, st.span.start)}")
    elif st.shared:
        parts.append("`shared`: every use is the same layer, with one set of weights")
    return "\n\n".join(parts)


def _value_text(v) -> Optional[str]:
    if v is None:
        return None
    if isinstance(v, ir.Layer):
        return config_to_source(v.config)
    if isinstance(v, ir.NODE_TYPES):
        n = sum(1 for _ in ir.unrolled_layers(v))
        return f"a block of {n} layer{'s' if n != 1 else ''}"
    if isinstance(v, L.Config):
        return config_to_source(v)
    if isinstance(v, (compiler.Builtin, compiler.Macro, compiler.Bare)):
        return None
    try:
        return value_to_source(v)
    except Exception:
        return None


def _taps(ix: Index, name: str) -> str:
    writes, reads, pops, ports = [], [], [], []
    for m in re.finditer(r"([@$])" + re.escape(name) + r"\b(!?)", ix.source):
        line = ix.source.count("\n", 0, m.start()) + 1
        through_port = ix.source[:m.start()].rstrip().endswith("=")
        if m.group(1) == "@":
            (ports if through_port else writes).append(line)
        else:
            (pops if m.group(2) else reads).append(line)

    def lines(xs):
        return ", ".join(f"line {x}" for x in xs)

    parts = [f"tap **{name}**"]
    if writes:
        parts.append(f"written (the stream pushed) on {lines(writes)}")
    if ports:
        parts.append(f"written by a layer's port on {lines(ports)}")
    if reads:
        parts.append(f"read on {lines(reads)}")
    if pops:
        parts.append(f"popped on {lines(pops)}")
    if not writes and not ports:
        parts.append("never written in this file")
    return "\n\n".join(parts)


def _hover_text(ix: Index, what: tuple) -> Optional[str]:
    kind = what[0]
    if kind == "module":
        return f"module `{what[1]}`: its definitions are visible in this file"
    if kind == "setting":
        try:
            doc = reference.setting_doc(what[1])
        except KeyError:
            return None
        value = _value_text(ix.value_of(what[1]))
        return doc + (f"\n\nhere: `{value}`" if value else "")
    if kind == "define":
        return _definition_doc(ix, what[1]) if what[1] in ix.names else None
    if kind == "param":
        return f"parameter `{what[1]}` of the macro `{what[2]}`"
    if kind == "tap":
        return _taps(ix, what[1])
    if kind in ("name", "call"):
        name = what[1]
        if name in ix.names:
            return _definition_doc(ix, name)
        if name in _ALL_TYPES:
            return reference.type_doc(name)
        if name in L.ACTIVATIONS:
            return reference.activation_doc(name)
        if name in ("true", "false", "none"):
            return None
        expected = what[2] if kind == "name" and len(what) > 2 else None
        if expected is not None:
            cls, field = expected
            if cls is not None and field in cls.model_fields:
                options = reference.literals(cls.model_fields[field].annotation)
                if name in options:
                    return f"`{name}`: an option of `{field}` — {reference.field_doc(cls, field)}"
                return f"`{name}` is not defined: here it is the string \"{name}\" — {reference.field_doc(cls, field)}"
        return f"`{name}` is not defined: as a setting's value it is the string \"{name}\""
    if kind == "key":
        cls, keys = what[1], what[2]
        if cls is None:
            return None
        if keys[-1] in cls.model_fields:
            return reference.field_doc(cls, keys[-1])
        if keys[-1] in getattr(cls, "ports", ()):
            return f"port `{keys[-1]}` of `{what[3]}`: `{keys[-1]}=@name` writes it to a tap, `{keys[-1]}=$name` reads it from one"
        return None
    if kind == "field":
        e = what[1]
        base = e.base.name if isinstance(e.base, S.Name) else None
        cls = ix.cls_of(base) if base else None
        if cls is not None and e.field in cls.model_fields:
            value = ix.value_of(base)
            cfg = value.config if isinstance(value, ir.Layer) else value
            now = getattr(cfg, e.field, None) if isinstance(cfg, L.Config) else None
            here = f"\n\nhere: `{value_to_source(now)}`" if cfg is not None and isinstance(cfg, L.Config) else ""
            return reference.field_doc(cls, e.field) + here
    return None


# ------------------------------------------------------------------------------ definition
def definition(source: str, offset: int, path: Optional[str] = None) -> Optional[tuple]:
    """(file, start, end) of the definition of the name at `offset`; offsets are in that file."""
    ix = Index(source, path)
    at = offset + ix.base
    for span, what in occurrences(ix):
        if span.start <= at <= span.end and what[0] in ("name", "call", "define", "setting"):
            hit = ix.names.get(what[1])
            if hit is None:
                return None
            st, file = hit
            f = ix.program.file_of(st.span.start) if ix.program is not None else None
            shift = f.start if f else 0
            return file, st.name_span.start - shift, st.name_span.end - shift
        if span.start <= at <= span.end and what[0] == "tap":
            m = re.search(r"@" + re.escape(what[1]) + r"\b", ix.source)
            return (ix.path, m.start(), m.end()) if m else None
    return None


# ------------------------------------------------------------------------------ completion
_WORD_END = re.compile(r"[A-Za-z_][A-Za-z0-9_]*$")


@dataclass
class _Open:
    """A bracket still open before the cursor: its callee and what has been typed in it."""
    callee: Optional[str]
    keys: list            # keys given so far (first parts of dotted keys)
    current: str          # the text of the argument being typed


def _open_call(before: str) -> Optional[_Open]:
    """The innermost ``name(`` still open at the end of `before` (within the statement)."""
    depth, i, current_start = 0, len(before) - 1, len(before)
    commas: list = []
    in_string = False
    while i >= 0:
        ch = before[i]
        if ch == '"':
            in_string = not in_string
        elif in_string:
            pass
        elif ch in ")]":
            depth += 1
        elif ch in "([":
            if depth == 0:
                if ch == "[":
                    return None
                m = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", before[:i])
                inside = before[i + 1:]
                parts = _split_args(inside)
                keys = [re.match(r"\s*([A-Za-z_]\w*)", p).group(1) for p in parts[:-1]
                        if re.match(r"\s*[A-Za-z_][\w.]*\s*=", p)]
                return _Open(m.group(1) if m else None, keys, parts[-1] if parts else "")
            depth -= 1
        elif ch == "\n" and depth == 0 and i + 1 < len(before) and not before[i + 1].isspace():
            return None
        i -= 1
    return None


def _split_args(text: str) -> list:
    parts, depth, cur, quoted = [], 0, "", False
    for ch in text:
        if ch == '"':
            quoted = not quoted
        if not quoted and ch in "([":
            depth += 1
        elif not quoted and ch in ")]":
            depth -= 1
        if ch == "," and depth == 0 and not quoted:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    parts.append(cur)
    return parts


def _definition_item(ix: Index, name: str, sort: str = "1") -> Completion:
    st, file = ix.names[name]
    tag = ix.leads_to(name)
    detail = ("macro(" + ", ".join(p.name for p in st.params) + ")") if st.params is not None else (tag or "definition")
    return Completion(name, "definition", detail, ix.written(st), sort=sort)


def _value_items(ix: Index, cls, field: str) -> list:
    """What may follow ``field=``: literal options, activations, configs by tag and the
    file's definitions that lead to one of those tags, booleans, none."""
    if cls is None or field not in cls.model_fields:
        return []
    ann = cls.model_fields[field].annotation
    items = [Completion(str(o), "value", f"option of {field}", sort="0") for o in reference.literals(ann)
             if isinstance(o, str)]
    wanted = {t for c in reference.config_classes(ann) for t in reference.tags(c)}
    for t in sorted(wanted):
        items.append(Completion(t, "layer", reference.kind_of(t), reference.docs.SUMMARY.get(t, ""), sort="2"))
    for name in ix.names:
        if ix.leads_to(name) in wanted and name not in wanted:
            items.append(_definition_item(ix, name, "1"))
    members = reference.members(ann)
    if bool in members:
        items += [Completion("true", "value", sort="0"), Completion("false", "value", sort="0")]
    if type(None) in members:
        items.append(Completion("none", "value", sort="3"))
    return items


def _field_items(ix: Index, cls, given=(), tag: Optional[str] = None, values=None, assign: bool = True) -> list:
    out = []
    for name, f in cls.model_fields.items():
        if name == "type" or name in given:
            continue
        detail = reference.type_text(f.annotation)
        if values is not None:
            detail = f"= {value_to_source(getattr(values, name))}"
        out.append(Completion(name, "field", detail, reference.field_doc(cls, name, tag),
                              insert=f"{name}=" if assign else name, sort="0" if f.is_required() else "1"))
    for p in sorted(getattr(cls, "ports", ())):
        if p not in given and assign:
            out.append(Completion(p, "field", "port", f"`{p}=@name` writes it to a tap, `{p}=$name` reads it",
                                  insert=f"{p}=", sort="2"))
    return out


def complete(source: str, offset: int, path: Optional[str] = None) -> list:
    """What fits at `offset`, best first within each kind (`Completion.sort`)."""
    before = source[:offset]
    word = _WORD_END.search(before)
    prefix = word.group(0) if word else ""
    head = before[: len(before) - len(prefix)]
    ix = Index(source, path)
    items: list = []

    # inside a string: a pattern's letters are the one-letter definitions
    line = before.rsplit("\n", 1)[-1]
    if line.count('"') % 2 == 1:
        items = [_definition_item(ix, n) for n in ix.names if len(n) == 1]
        return _unique(items)
    if head.endswith(("@", "$")):
        seen = sorted(set(re.findall(r"[@$]([A-Za-z_]\w*)", source[:offset - len(prefix) - 1] + source[offset:])))
        return _unique([Completion(n, "tap", "tap") for n in seen if n.startswith(prefix)])
    if head.endswith("."):
        chain = re.search(r"((?:[A-Za-z_]\w*\.)+)$", head)
        names = chain.group(1).rstrip(".").split(".") if chain else []
        if names:
            cls = ix.cls_of(names[0])
            value = ix.value_of(names[0])
            cfg = value.config if isinstance(value, ir.Layer) else value
            if cls is None:
                # ``rope.`` as a dotted key inside a call: the field's class
                opened = _open_call(head[: -len(chain.group(1))])
                owner = ix.cls_of(opened.callee) if opened and opened.callee else None
                cls, cfg = _descend(owner, tuple(names)) if owner is not None else None, None
            else:
                for n in names[1:]:
                    cls = field_class(cls, n)
                    cfg = getattr(cfg, n, None) if isinstance(cfg, L.Config) else None
            if cls is not None:
                items = _field_items(ix, cls, values=cfg if isinstance(cfg, L.Config) else None, assign=False)
        return _unique([i for i in items if i.label.startswith(prefix)])

    opened = _open_call(head)
    if opened is not None and opened.callee:
        macro = ix.statement(opened.callee)
        arg = opened.current
        if "=" in arg:                                        # a value position
            key = arg.split("=", 1)[0].strip()
            cls = ix.cls_of(opened.callee)
            keys = tuple(key.split("."))
            items = _value_items(ix, _descend(cls, keys[:-1]), keys[-1])
            items += _expression_items(ix, offset, sort="4") if not items else []
        elif macro is not None and macro.params is not None:   # a macro call: its parameters
            items = [Completion(p.name, "parameter", f"parameter of {opened.callee}", insert=f"{p.name}=", sort="0")
                     for p in macro.params if p.name not in opened.keys]
            items += _expression_items(ix, offset, sort="3")
        else:
            cls = ix.cls_of(opened.callee)
            if cls is not None:
                items = _field_items(ix, cls, opened.keys, ix.leads_to(opened.callee))
            else:
                items = _expression_items(ix, offset)
        return _unique([i for i in items if i.label.startswith(prefix)])

    at_line_start = line.strip() == prefix
    if at_line_start:
        items = [Completion(n, "setting", "setting", _safe(reference.setting_doc, n), sort="2") for n in _TOP]
        items += [Completion("use", "keyword", "use MODULE", sort="3"), Completion("shared", "keyword", sort="3")]
        items += [_definition_item(ix, n, "1") for n in ix.names]   # to amend: ``attn.num_heads = 8``
    else:
        m = re.match(r"\s*([A-Za-z_]\w*)\s*=\s*[^=]*$", line)
        if m and m.group(1) in T.TrainConfig.model_fields and "(" not in line.split("=", 1)[1]:
            items = _value_items(ix, T.TrainConfig, m.group(1))
        items += _expression_items(ix, offset)
    return _unique([i for i in items if i.label.startswith(prefix)])


def _safe(fn, *a) -> str:
    try:
        return fn(*a)
    except KeyError:
        return ""


def _expression_items(ix: Index, offset: int, sort: str = "2") -> list:
    items = []
    st = ix.enclosing(offset)
    for p in (st.params or ()) if st is not None else ():
        items.append(Completion(p.name, "parameter", f"parameter of {st.name}", sort="0"))
    items += [_definition_item(ix, n, "1") for n in ix.names if n not in _TOP]
    # a training setting's statement is written with the training types, anything else
    # (a block, the model, a layer's definition) with layers and their parts
    training = st is not None and st.name in T.TrainConfig.model_fields
    pool = {**T.TRAINING, **T.DISTRIBUTIONS} if training else {**L.LAYERS, **L.SUBCONFIGS, **L.RESIDUALS, **L.INITS}
    items += [Completion(n, "layer", reference.kind_of(n), reference.docs.SUMMARY.get(n, ""), sort=sort)
              for n in sorted(pool)]
    if not training:
        items += [Completion(a, "layer", "activation", sort=sort) for a in L.ACTIVATIONS]
    return items


def _unique(items: list) -> list:
    seen, out = set(), []
    for it in sorted(items, key=lambda i: (i.sort, i.label)):
        if it.label not in seen:
            seen.add(it.label)
            out.append(it)
    return out


# ------------------------------------------------------------------------------ positions
def offset_of(source: str, line: int, character: int) -> int:
    lines = source.split("\n")
    line = min(line, len(lines) - 1)
    return sum(len(x) + 1 for x in lines[:line]) + min(character, len(lines[line]))


def position_of(source: str, offset: int) -> tuple:
    before = source[:offset]
    return before.count("\n"), offset - (before.rfind("\n") + 1)
