"""Lexer, syntax tree and parser of the ``.bux`` language.

Grammar (loosest binding first; reference: ``docs/language/grammar.md:79-108`` and
``src/bux/lang/syntax.py``)::

    program    := [item] { (NEWLINE | ";") [item] }
    item       := "use" (NAME|STRING) | ["shared"] NAME "=" expr
                | NAME "(" params ")" "=" expr | NAME "." NAME {"." NAME} "=" expr
    expr       := option { "|" option }            option := [NAME ":"] sum
    sum        := prod { ("+"|"-") prod }
    prod       := chain { ("*"|"/"|"//") chain }
    chain      := unary { ["->"|"→"] unary }       juxtaposition composes
    unary      := "-" unary | power                power := atom ["^" unary]
    atom       := NAME [call] {"." NAME} | NUMBER | STRING | "_" | true|false|none
                | "@" NAME | "$" NAME ["!"] | "(" expr ")" | "[" expr "]" | list

A statement ends at a line break unless a bracket is open or the next non-blank
line is indented. ``f(x)`` (no blank) is a call, ``f (x)`` a composition.

The parser is a small hand-written precedence climber over a token cursor; every
tree node keeps the source `Span` it came from so that later compiler errors can
point at the text.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from decimal import Decimal
from typing import Optional, Union


@dataclass(frozen=True)
class Span:
    start: int
    end: int

    def to(self, other: "Span") -> "Span":
        return Span(self.start, other.end)


class BuxError(Exception):
    """A mistake in ``.bux`` source, printed rustc-style once attached to its file::

        error: unknown layer or block 'nrom'
         --> tiny.bux:2:15
          |
        2 | model = embed nrom head
          |               ^^^^
          = hint: did you mean 'norm'?
    """

    def __init__(self, message: str, span: Optional[Span] = None, hint: Optional[str] = None):
        super().__init__(message)
        self.message, self.span, self.hint = message, span, hint
        self.source: Optional[str] = None
        self.filename = "<string>"

    def attach(self, source: str, filename: str) -> "BuxError":
        if self.source is None:
            self.source, self.filename = source, filename
        return self

    def location(self) -> Optional[tuple]:
        """(line, column), both 1-based, or None without a span and source."""
        if self.source is None or self.span is None:
            return None
        start = min(self.span.start, len(self.source))
        line = self.source.count("\n", 0, start) + 1
        return line, start - (self.source.rfind("\n", 0, start) + 1) + 1

    def __str__(self) -> str:
        out = [f"error: {self.message}"]
        where = self.location()
        if where is None:
            if self.hint:
                out.append(f"hint: {self.hint}")
            return "\n".join(out)
        line, col = where
        src = self.source or ""
        begin = src.rfind("\n", 0, min(self.span.start, len(src))) + 1
        stop = src.find("\n", begin)
        stop = len(src) if stop < 0 else stop
        width = max(1, min(self.span.end, stop) - (begin + col - 1))
        gutter = " " * len(str(line))
        out += [
            f"{gutter}--> {self.filename}:{line}:{col}",
            f"{gutter} |",
            f"{line} | {src[begin:stop]}",
            f"{gutter} | {' ' * (col - 1)}{'^' * width}",
        ]
        if self.hint:
            out.append(f"{gutter} = hint: {self.hint}")
        return "\n".join(out)


# ------------------------------------------------------------------ tokens
@dataclass(frozen=True)
class Token:
    kind: str  # NAME NUMBER STRING OP NEWLINE EOF
    text: str
    span: Span
    spaced: bool  # blanks or a line break before it
    value: Union[int, float, str, None] = None


_NUM = re.compile(r"\d(?:_?\d)*(\.\d(?:_?\d)*)?([eE][+-]?\d+)?(?:([kKMBT])(?![A-Za-z0-9_]))?")
_IDENT = re.compile(r"[A-Za-z_][A-Za-z0-9_]*")
_POWERS = {"k": 3, "K": 3, "M": 6, "B": 9, "T": 12}
_SYMBOLS = ("->", "//", "→", "|", ":", "+", "-", "*", "/", "^", "=", ",", "(", ")", "[", "]",
            "@", "$", "!", ".", ";")
KEYWORDS = frozenset({"true", "false", "none", "shared", "_"})


def _next_line_indented(src: str, pos: int, stop: int) -> bool:
    """Whether the next line holding anything but blanks/comments starts indented."""
    while pos < stop:
        j = pos
        while j < stop and src[j] in " \t\r":
            j += 1
        if j < stop and src[j] not in "\n#":
            return j > pos
        nl = src.find("\n", j, stop)
        if nl < 0:
            return False
        pos = nl + 1
    return False


def _read_number(m: re.Match, spaced: bool) -> Token:
    text = m.group()
    digits = text.replace("_", "")
    if m.group(3):
        exact = Decimal(digits[:-1]).scaleb(_POWERS[m.group(3)])
        value = int(exact) if exact == exact.to_integral() else float(exact)
    elif m.group(1) or m.group(2):
        value = float(digits)
    else:
        value = int(digits)
    return Token("NUMBER", text, Span(m.start(), m.end()), spaced, value)


def tokenize(src: str, start: int = 0, stop: Optional[int] = None,
             errors: Optional[list] = None) -> list:
    """Split source into tokens. With an `errors` list, mistakes are collected and
    lexing goes on (what an editor needs); without, the first one raises."""

    def fail(err: BuxError) -> None:
        if errors is None:
            raise err
        errors.append(err)

    stop = len(src) if stop is None else stop
    out: list = []
    pos, depth, spaced = start, 0, True
    while pos < stop:
        ch = src[pos]
        if ch == "\n":
            if (depth == 0 and out and out[-1].kind != "NEWLINE"
                    and not _next_line_indented(src, pos + 1, stop)):
                out.append(Token("NEWLINE", "\n", Span(pos, pos + 1), spaced))
            pos, spaced = pos + 1, True
            continue
        if ch in " \t\r":
            pos, spaced = pos + 1, True
            continue
        if ch == "#":
            nl = src.find("\n", pos, stop)
            pos, spaced = (stop if nl < 0 else nl), True
            continue
        tok = None
        m = _NUM.match(src, pos, stop)
        if m:
            if src.startswith("_", m.end()):
                fail(BuxError("a number's '_' goes between two digits: 1_000",
                              Span(m.end(), m.end() + 1)))
            tok = _read_number(m, spaced)
        elif (m := _IDENT.match(src, pos, stop)):
            tok = Token("NAME", m.group(), Span(pos, m.end()), spaced)
        elif ch in "\"'":
            close = src.find(ch, pos + 1, stop)
            if close < 0 or "\n" in src[pos:close]:
                fail(BuxError("unterminated string", Span(pos, pos + 1)))
                close = src.find("\n", pos, stop)
                close = stop if close < 0 else close
                tok = Token("STRING", src[pos:close], Span(pos, close), spaced, src[pos + 1:close])
            else:
                tok = Token("STRING", src[pos:close + 1], Span(pos, close + 1), spaced,
                            src[pos + 1:close])
        else:
            sym = next((s for s in _SYMBOLS if src.startswith(s, pos)), None)
            if sym is not None:
                tok = Token("OP", sym, Span(pos, pos + len(sym)), spaced)
        if tok is None:
            fail(BuxError(f"unexpected character {ch!r}", Span(pos, pos + 1)))
            pos, spaced = pos + 1, False
            continue
        if tok.kind == "OP" and tok.text in "([":
            depth += 1
        elif tok.kind == "OP" and tok.text in ")]":
            depth = max(0, depth - 1)
        out.append(tok)
        pos, spaced = tok.span.end, False
    tail = next((t.span.end for t in reversed(out) if t.kind != "NEWLINE"), stop)
    out.append(Token("EOF", "", Span(tail, tail), spaced))
    return out


# ------------------------------------------------------------------ tree
@dataclass(frozen=True)
class Expr:
    span: Span


@dataclass(frozen=True)
class Lit(Expr):
    value: object = None


@dataclass(frozen=True)
class Name(Expr):
    name: str = ""


@dataclass(frozen=True)
class Identity(Expr):
    pass


@dataclass(frozen=True)
class Tap(Expr):
    name: str = ""


@dataclass(frozen=True)
class Ref(Expr):
    name: str = ""
    pop: bool = False


@dataclass(frozen=True)
class ListExpr(Expr):
    items: tuple = ()


@dataclass(frozen=True)
class Residual(Expr):
    body: Expr = None  # type: ignore[assignment]


@dataclass(frozen=True)
class Seq(Expr):
    items: tuple = ()


@dataclass(frozen=True)
class Neg(Expr):
    operand: Expr = None  # type: ignore[assignment]


@dataclass(frozen=True)
class BinOp(Expr):
    op: str = ""
    left: Expr = None  # type: ignore[assignment]
    right: Expr = None  # type: ignore[assignment]


@dataclass(frozen=True)
class Arg:
    span: Span
    key: Optional[tuple]  # dotted key parts, or None for a positional argument
    value: Expr
    key_spans: tuple = ()


@dataclass(frozen=True)
class Call(Expr):
    name: str = ""
    name_span: Span = None  # type: ignore[assignment]
    args: tuple = ()
    amend: bool = False  # made by an amendment statement ``a.b = v``
    where: Optional[str] = None  # "definition.setting" a dimension is written at


@dataclass(frozen=True)
class Attr(Expr):
    base: Expr = None  # type: ignore[assignment]
    field: str = ""
    field_span: Span = None  # type: ignore[assignment]


@dataclass(frozen=True)
class Alt(Expr):
    options: tuple = ()
    labels: tuple = ()  # one per option, or empty
    where: str = ""  # the definition (and setting) its first alternative is written at


@dataclass(frozen=True)
class Param:
    name: str
    span: Span
    default: Optional[Expr] = None


@dataclass(frozen=True)
class Statement:
    name: str
    name_span: Span
    body: Optional[Expr]
    span: Span
    params: Optional[tuple] = None  # a macro's parameters
    shared: bool = False
    amends: bool = False
    use: Optional[str] = None  # ``use module``: the module's name
    doc: str = ""


# ------------------------------------------------------------------ parser
_STARTS_ATOM_OPS = {"(", "[", "@", "$", "-"}


class _Cursor:
    def __init__(self, tokens: list, src: str):
        self.toks, self.i, self.src = tokens, 0, src

    @property
    def tok(self) -> Token:
        return self.toks[self.i]

    def peek(self, k: int = 1) -> Token:
        return self.toks[min(self.i + k, len(self.toks) - 1)]

    def advance(self) -> Token:
        t = self.toks[self.i]
        if t.kind != "EOF":
            self.i += 1
        return t

    def at(self, text: str) -> bool:
        return self.tok.kind == "OP" and self.tok.text == text

    def take(self, text: str) -> Optional[Token]:
        return self.advance() if self.at(text) else None

    def expect(self, text: str, what: Optional[str] = None) -> Token:
        if not self.at(text):
            raise BuxError(f"expected {what or repr(text)}, found {describe(self.tok)}",
                           self.tok.span)
        return self.advance()


def describe(tok: Token) -> str:
    if tok.kind == "EOF":
        return "end of input"
    if tok.kind == "NEWLINE":
        return "end of line"
    return f"'{tok.text}'"


class Parser:
    """Recursive-descent parser; `where` tracks the definition being parsed so
    sweep axes and search dimensions know the setting they were written at."""

    def __init__(self, src: str, tokens: list):
        self.c = _Cursor(tokens, src)
        self.src = src
        self.context: list = []  # name path: definition, then call keys

    # ---- statements
    def program(self, errors: Optional[list] = None) -> tuple:
        """Return (statements, names of definitions that failed to parse)."""
        items, broken = [], []
        c = self.c
        while c.tok.kind != "EOF":
            if c.tok.kind == "NEWLINE" or c.at(";"):
                c.advance()
                continue
            mark = c.i
            try:
                items.append(self.statement())
                if c.tok.kind not in ("NEWLINE", "EOF") and not c.at(";"):
                    raise BuxError(f"unexpected {describe(c.tok)}", c.tok.span,
                                   self._juxtaposition_hint())
            except BuxError as err:
                if errors is None:
                    raise
                errors.append(err)
                first = c.toks[mark]
                if first.kind == "NAME":
                    name = c.toks[mark + 1].text if first.text == "shared" else first.text
                    broken.append(name)
                while c.tok.kind not in ("NEWLINE", "EOF"):
                    c.advance()
        return items, broken

    def _juxtaposition_hint(self) -> Optional[str]:
        return None

    def statement(self) -> Statement:
        c = self.c
        first = c.tok
        if first.kind != "NAME":
            raise BuxError(f"expected a definition, found {describe(first)}", first.span,
                           "a statement is name = expression")
        if first.text == "use" and c.peek().kind in ("NAME", "STRING") and not (
                c.peek(2).kind == "OP" and c.peek(2).text == "="):
            c.advance()
            mod = c.advance()
            name = mod.value if mod.kind == "STRING" else mod.text
            return Statement(name=str(name), name_span=mod.span, body=None,
                             span=first.span.to(mod.span), use=str(name))
        shared = False
        if first.text == "shared" and c.peek().kind == "NAME":
            c.advance()
            shared = True
        name_tok = c.advance()
        if name_tok.kind != "NAME" or name_tok.text in KEYWORDS:
            raise BuxError(f"expected a name to define, found {describe(name_tok)}",
                           name_tok.span)
        name = name_tok.text
        params = None
        # a macro: name(params) = ...   (no blank before the parenthesis)
        if c.at("(") and not c.tok.spaced and self._is_macro_head():
            params = self._params()
        if c.at("."):
            return self._amendment(name_tok, shared)
        if not c.at("="):
            raise BuxError(f"expected '=' after '{name}', found {describe(c.tok)}", c.tok.span,
                           "a statement is name = expression")
        c.advance()
        self.context = [name]
        body = self.expr()
        return Statement(name=name, name_span=name_tok.span, body=body,
                         span=name_tok.span.to(body.span), params=params, shared=shared)

    def _is_macro_head(self) -> bool:
        """Look ahead for ``( ... ) =`` at depth 0."""
        depth, k = 0, 0
        while True:
            t = self.c.peek(k)
            if t.kind in ("EOF", "NEWLINE"):
                return False
            if t.kind == "OP" and t.text in "([":
                depth += 1
            elif t.kind == "OP" and t.text in ")]":
                depth -= 1
                if depth == 0:
                    nxt = self.c.peek(k + 1)
                    return nxt.kind == "OP" and nxt.text == "="
            k += 1

    def _params(self) -> tuple:
        c = self.c
        c.expect("(")
        params = []
        while not c.at(")"):
            t = c.advance()
            if t.kind != "NAME" or t.text in KEYWORDS:
                raise BuxError(f"expected a parameter name, found {describe(t)}", t.span)
            default = None
            if c.take("="):
                default = self.expr()
            params.append(Param(t.text, t.span, default))
            if not c.take(","):
                break
        c.expect(")")
        names = [p.name for p in params]
        for p in params:
            if names.count(p.name) > 1:
                raise BuxError(f"parameter '{p.name}' is given twice", p.span)
        return tuple(params)

    def _amendment(self, name_tok: Token, shared: bool) -> Statement:
        """``a.b.c = v`` means ``a = a(b.c=v)``, keeping what ``a`` was."""
        c = self.c
        keys, spans = [], []
        while c.take("."):
            t = c.advance()
            if t.kind != "NAME":
                raise BuxError(f"expected a setting's name, found {describe(t)}", t.span)
            keys.append(t.text)
            spans.append(t.span)
        c.expect("=")
        self.context = [name_tok.text, ".".join(keys)]
        value = self.expr()
        whole = name_tok.span.to(value.span)
        arg = Arg(spans[0].to(value.span), tuple(keys), value, tuple(spans))
        body = Call(whole, name_tok.text, name_tok.span, (arg,), amend=True)
        return Statement(name=name_tok.text, name_span=name_tok.span, body=body, span=whole,
                         shared=shared, amends=True)

    # ---- expressions
    def expr(self) -> Expr:
        c = self.c
        options, labels = [], []
        while True:
            label = None
            if c.tok.kind == "NAME" and c.peek().kind == "OP" and c.peek().text == ":":
                label = c.advance().text
                c.advance()
            options.append(self.sum())
            labels.append(label)
            if not c.take("|"):
                break
        if len(options) == 1 and labels[0] is None:
            return options[0]
        if len(options) == 1:
            raise BuxError("a label names one of several alternatives: a: x | b: y",
                           options[0].span)
        if any(labels) and not all(labels):
            raise BuxError("label every alternative or none of them", options[0].span.to(options[-1].span),
                           "name: a | other: b")
        if all(labels) and len(set(labels)) < len(labels):
            raise BuxError("two alternatives have the same label",
                           options[0].span.to(options[-1].span))
        return Alt(options[0].span.to(options[-1].span), tuple(options),
                   tuple(labels) if all(labels) else (), ".".join(self.context))

    def sum(self) -> Expr:
        left = self.prod()
        while self.c.at("+") or self.c.at("-"):
            op = self.c.advance().text
            right = self.prod()
            left = BinOp(left.span.to(right.span), op, left, right)
        return left

    def prod(self) -> Expr:
        left = self.chain()
        while self.c.at("*") or self.c.at("/") or self.c.at("//"):
            op = self.c.advance().text
            right = self.chain()
            left = BinOp(left.span.to(right.span), op, left, right)
        return left

    def _starts_unary(self) -> bool:
        t = self.c.tok
        if t.kind in ("NAME", "NUMBER", "STRING"):
            # `name:` starts the next labeled alternative only after a `|`
            return True
        return t.kind == "OP" and t.text in ("(", "[", "@", "$")

    def chain(self) -> Expr:
        items = [self.unary()]
        while True:
            if self.c.at("->") or self.c.at("→"):
                self.c.advance()
                items.append(self.unary())
            elif self._starts_unary():
                items.append(self.unary())
            else:
                break
        if len(items) == 1:
            return items[0]
        return Seq(items[0].span.to(items[-1].span), tuple(items))

    def unary(self) -> Expr:
        if self.c.at("-"):
            minus = self.c.advance()
            operand = self.unary()
            return Neg(minus.span.to(operand.span), operand)
        return self.power()

    def power(self) -> Expr:
        base = self.atom()
        if self.c.at("^"):
            self.c.advance()
            exponent = self.unary()
            return BinOp(base.span.to(exponent.span), "^", base, exponent)
        return base

    def atom(self) -> Expr:
        c = self.c
        t = c.tok
        if t.kind == "NUMBER":
            c.advance()
            return Lit(t.span, t.value)
        if t.kind == "STRING":
            c.advance()
            return Lit(t.span, t.value)
        if t.kind == "NAME":
            c.advance()
            if t.text == "_":
                return Identity(t.span)
            if t.text in ("true", "false"):
                return Lit(t.span, t.text == "true")
            if t.text == "none":
                return Lit(t.span, None)
            if t.text == "shared":
                raise BuxError("'shared' starts a definition: shared name = ...", t.span)
            node: Expr = Name(t.span, t.text)
            if c.at("(") and not c.tok.spaced:
                node = self._call(t)
            while c.at(".") and not c.tok.spaced and c.peek().kind == "NAME":
                c.advance()
                f = c.advance()
                node = Attr(node.span.to(f.span), node, f.text, f.span)
            return node
        if t.kind == "OP":
            if t.text == "(":
                c.advance()
                inner = self.expr()
                close = c.expect(")", "')'")
                return inner
            if t.text == "[":
                return self._bracket()
            if t.text == "@":
                c.advance()
                n = c.advance()
                if n.kind != "NAME" or n.spaced:
                    raise BuxError("'@' names a tap: @name", t.span.to(n.span))
                return Tap(t.span.to(n.span), n.text)
            if t.text == "$":
                c.advance()
                n = c.advance()
                if n.kind != "NAME" or n.spaced:
                    raise BuxError("'$' reads a tap: $name", t.span.to(n.span))
                end = n.span
                pop = False
                if c.at("!") and not c.tok.spaced:
                    end = c.advance().span
                    pop = True
                return Ref(t.span.to(end), n.text, pop)
        raise BuxError(f"expected a layer, a block or a value, found {describe(t)}", t.span)

    def _bracket(self) -> Expr:
        """``[f]`` is a residual branch; ``[a, b]``, ``[a,]`` and ``[]`` are lists."""
        c = self.c
        open_ = c.expect("[")
        if c.at("]"):
            return ListExpr(open_.span.to(c.advance().span), ())
        first = self.expr()
        if c.at("]"):
            return Residual(open_.span.to(c.advance().span), first)
        items = [first]
        while c.take(","):
            if c.at("]"):
                break
            items.append(self.expr())
        close = c.expect("]", "']'")
        return ListExpr(open_.span.to(close.span), tuple(items))

    def _call(self, name_tok: Token) -> Call:
        c = self.c
        c.expect("(")
        args = []
        saved = list(self.context)
        while not c.at(")"):
            start = c.tok
            key, key_spans = None, ()
            if start.kind == "NAME" and self._keyed():
                parts, spans = [c.advance()], []
                while c.take("."):
                    parts.append(c.advance())
                key = tuple(p.text for p in parts)
                key_spans = tuple(p.span for p in parts)
                c.expect("=")
                self.context = saved + [".".join(key)] if len(saved) <= 1 else \
                    saved[:-1] + [saved[-1] + "." + ".".join(key)]
            value = self.expr()
            self.context = saved
            args.append(Arg(start.span.to(value.span), key, value, key_spans))
            if not c.take(","):
                break
        close = c.expect(")", "')' or ','")
        where = ".".join(saved) if saved else None
        return Call(name_tok.span.to(close.span), name_tok.text, name_tok.span, tuple(args),
                    where=where)

    def _keyed(self) -> bool:
        """Whether the tokens ahead read ``name{.name} =``."""
        k = 1
        while True:
            t = self.c.peek(k)
            if t.kind == "OP" and t.text == "." and self.c.peek(k + 1).kind == "NAME":
                k += 2
                continue
            return t.kind == "OP" and t.text == "="


def parse(src: str, errors: Optional[list] = None) -> tuple:
    """Parse source into (statements, broken definition names)."""
    tokens = tokenize(src, errors=errors)
    return Parser(src, tokens).program(errors)


def parse_statement(src: str) -> Statement:
    """Parse exactly one statement, as a command-line override gives it."""
    items, _ = parse(src)
    if len(items) != 1:
        raise BuxError("an override is one statement: name=value", Span(0, len(src)))
    return items[0]
