"""The ``.bux`` compiler: evaluate definitions, expand sweeps, infer widths, check
taps and ports, and emit `ir.Architecture` / `ir.Run` -- all before any ML import.

Pipeline: `modules.load` (files → layered statements) → `Evaluator` (lazy evaluation
of definitions into values and untyped graphs; `|` picks by a choice table) →
`Lowering` (one walk that types every layer's input width, simulates the tap stacks,
checks shared blocks and inserts ``merge`` where a widened stream must narrow) →
training settings validated by the pydantic schema.

Behavioural reference: ``src/bux/lang/compiler.py`` (evaluation rules ``:417-1340``,
lowering ``:1367-1700``, runs and sweeps ``:1991-2340``). The implementation here is
this project's own.
"""

from __future__ import annotations

import difflib
import operator
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Mapping, Optional, Sequence, Union

from pydantic import TypeAdapter, ValidationError

from ..config import layers as L
from ..config import training as T
from . import ir, modules
from . import syntax as S
from .syntax import BuxError, Span
from .widths import GraphTyper

LAYERS = L.LAYERS
TRAINING = T.TRAINING
TYPES = {**L.LAYERS, **L.SUBCONFIGS, **T.TRAINING}
ACTIVATIONS = frozenset(L.ACTIVATIONS)
RESIDUALS, INITS, DISTRIBUTIONS = L.RESIDUALS, L.INITS, T.DISTRIBUTIONS
SETTINGS = ("d_model", "vocab_size", "residual", "init")
TRAIN_SETTINGS = tuple(T.TrainConfig.model_fields)
RESERVED = (*SETTINGS, *TRAIN_SETTINGS, "model")
REQUIRED = tuple(n for n, f in T.TrainConfig.model_fields.items() if f.is_required())
_SOURCE_TAGS = frozenset(t for t, c in TRAINING.items() if issubclass(c, T.SOURCES))
_EXAMPLES = {
    "data": 'data = text(path="data/fineweb/*.parquet")',
    "optimizer": "optimizer = adamw(lr=3e-4)",
    "seq_len": "seq_len = 1024",
    "batch": "batch = 256",
    "steps": "steps = 10k",
}
_ARITH: dict = {"+": operator.add, "-": operator.sub, "*": operator.mul,
                "/": operator.truediv, "//": operator.floordiv, "^": operator.pow}


# ------------------------------------------------------------------ value model
@dataclass(frozen=True)
class Named:
    """A value reached through a definition or macro call; graphs keep the label."""
    label: str
    value: object
    share: Optional[str] = None


@dataclass(frozen=True)
class Builtin:
    name: str
    span: Optional[Span] = field(default=None, compare=False)


@dataclass(frozen=True)
class Bare:
    """A name nothing defines: a string as a setting's value, an error elsewhere."""
    name: str


@dataclass(frozen=True)
class Macro:
    statement: S.Statement


class Reported(BuxError):
    """Stands for an error that was already reported at its origin."""

    def __init__(self):
        super().__init__("already reported")


@dataclass(frozen=True)
class Axis:
    """One sweep axis: an unlabeled ``a | b`` (keyed by its span) or all alternatives
    that share a label set (keyed by the set; they are picked together)."""
    key: Union[Span, frozenset]
    where: str
    options: tuple
    span: Span

    @property
    def labeled(self) -> bool:
        return isinstance(self.key, frozenset)

    def pick(self, i: int):
        return self.options[i] if self.labeled else i

    def part(self, pick) -> str:
        return pick if isinstance(pick, str) else f"{self.where}={self.options[pick]}"


@dataclass(frozen=True)
class Dimension:
    """One search dimension: a distribution written in place of a value."""
    key: Span
    where: str
    space: Any

    def part(self, value) -> str:
        if isinstance(self.space, T.ChoiceConfig):
            return f"{self.where}={self.space.options[int(value)]}"
        if isinstance(self.space, T.IntUniformConfig):
            return f"{self.where}={int(value)}"
        return f"{self.where}={short(value)}"


def middle(space):
    return 0 if isinstance(space, T.ChoiceConfig) else space.value(0.5)


def short(x: float) -> str:
    """`x` written as briefly as reads back equal: 3.16e-4, 0.05."""
    mant, power = f"{x:.{T.DIGITS - 1}e}".split("e")
    mant = mant.rstrip("0").rstrip(".")
    forms = (repr(float(x)).removesuffix(".0"), f"{mant}e{int(power)}")
    return min((w for w in forms if float(w) == x), key=len, default=repr(x))


def unwrap(v):
    while isinstance(v, Named):
        v = v.value
    return v


def is_number(v) -> bool:
    v = unwrap(v)
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def tag_of(config) -> str:
    return getattr(config, "type", type(config).__name__)


def describe(v) -> str:
    v = unwrap(v)
    if isinstance(v, bool):
        return "a boolean"
    if isinstance(v, (int, float)):
        return "a number"
    if isinstance(v, str):
        return "a string"
    if v is None:
        return "none"
    if isinstance(v, (list, tuple)):
        return "a list"
    if isinstance(v, L.Config):
        return f"{tag_of(v)}(...)"
    if isinstance(v, ir.NODE_TYPES):
        return "a block"
    if isinstance(v, Builtin):
        return f"the type {v.name}"
    if isinstance(v, Macro):
        return "a macro"
    if isinstance(v, Bare):
        return f"the undefined name '{v.name}'"
    return type(v).__name__


def nothing(v) -> bool:
    """``f^0``: an empty sequence, which a surrounding sequence drops."""
    v = unwrap(v)
    return isinstance(v, ir.Seq) and not v.items


def flatten(nodes, cls, attr) -> tuple:
    out = []
    for n in nodes:
        if isinstance(n, cls) and n.label is None and n.share is None:
            out.extend(getattr(n, attr))
        else:
            out.append(n)
    return tuple(out)


def _activation(name: str):
    return L.ActivationConfig(fn=name)


def _assign(data: dict, key: tuple, value) -> None:
    for part in key[:-1]:
        nxt = data.get(part)
        if not isinstance(nxt, dict):
            nxt = {} if nxt is None else (
                nxt.model_dump() if isinstance(nxt, L.Config) else {})
            data[part] = nxt
        data = nxt
    data[key[-1]] = value.model_dump() if isinstance(value, L.Config) and False else value


def _field_annotation(cls, key: tuple):
    """Annotation of the (possibly dotted) field `key` of `cls`, or None."""
    import typing

    ann = None
    for part in key:
        fields = getattr(cls, "model_fields", None)
        if not fields or part not in fields:
            return None
        ann = fields[part].annotation
        cls = next((a for a in _flat_args(ann) if isinstance(a, type)
                    and issubclass(a, L.Config)), None)
    return ann


def _flat_args(ann) -> list:
    import typing

    out, todo = [], [ann]
    while todo:
        a = todo.pop()
        args = typing.get_args(a)
        if args and typing.get_origin(a) is not typing.Literal:
            todo.extend(args)
        else:
            out.append(a)
    return out


def _takes_number_only(cls, key) -> bool:
    ann = _field_annotation(cls, key)
    if ann is None:
        return False
    kinds = [a for a in _flat_args(ann) if a is not type(None)]
    return bool(kinds) and all(a in (int, float) for a in kinds if isinstance(a, type)) and \
        any(a in (int, float) for a in kinds) and bool not in kinds


def _literal_option(cls, key, name: str) -> bool:
    """Whether `name` is one of the literal options of field `key` (``wsd(shape=cosine)``
    means the option, not the cosine schedule)."""
    import typing

    ann = _field_annotation(cls, key)
    if ann is None:
        return False
    for a in _flat_args(ann):
        if typing.get_origin(a) is typing.Literal and name in typing.get_args(a):
            return True
    return False


# ------------------------------------------------------------------ evaluator
class Evaluator:
    def __init__(self, program: modules.Program, *, report: Optional[Callable] = None,
                 choices: Optional[Mapping] = None, point: Optional[Mapping] = None):
        self.source = program.source
        self.broken = set(program.broken)
        self.incomplete = program.incomplete
        self.chain: dict = {}
        for layer in program.layers:
            self._add_layer(layer, report)
        self.statements = {n: c[-1] for n, c in self.chain.items()}
        self.cache: dict = {}
        self.evaluating: list = []
        self.levels: list = []
        self.depth = 0
        self.choices = dict(choices or {})
        self.axes: dict = {}
        self.point = dict(point or {})
        self.dims: dict = {}
        self.node_spans: dict = {}
        self._alive: list = []
        self.bare: dict = {}

    def _add_layer(self, layer, report) -> None:
        seen: set = set()
        for st in layer:
            err = None
            if st.name in seen:
                err = BuxError(f"'{st.name}' is defined twice", st.name_span)
            elif st.params is not None and st.name in RESERVED:
                err = BuxError(f"'{st.name}' cannot be a macro", st.name_span)
                self.broken.add(st.name)
            if err is None:
                seen.add(st.name)
                chain = self.chain.setdefault(st.name, [])
                if st.amends and chain and chain[-1].shared and not st.shared:
                    from dataclasses import replace

                    st = replace(st, shared=True)
                chain.append(st)
            elif report is None:
                raise err
            else:
                report(err)

    # ---- bookkeeping
    def node(self, n, span: Span):
        self.node_spans[id(n)] = span
        self._alive.append(n)
        return n

    def text(self, span: Span) -> str:
        return " ".join(self.source[span.start:span.end].split())

    # ---- names
    def definition(self, name: str, level: Optional[int] = None):
        chain = self.chain[name]
        level = len(chain) - 1 if level is None else level
        st = chain[level]
        if st.params is not None:
            return Macro(st)
        if (name, level) not in self.cache:
            self.evaluating.append(name)
            self.levels.append(level)
            try:
                self.cache[name, level] = (self.objective(st.body) if name == "objective"
                                           else self.eval(st.body, {}))
            finally:
                self.evaluating.pop()
                self.levels.pop()
        return Named(name, self.cache[name, level], name if st.shared else None)

    def evaluate_all(self, report: Optional[Callable] = None) -> None:
        for name, st in self.statements.items():
            if st.params is not None:
                continue
            try:
                self.definition(name)
            except BuxError as err:
                if report is None:
                    raise
                report(err)

    def lookup(self, name: str, span: Span, scope: dict):
        if name in scope:
            return scope[name]
        if name in self.broken and name not in self.statements:
            raise Reported()
        if name in self.statements:
            if name not in self.evaluating:
                return self.definition(name)
            if self.evaluating[-1] != name:
                raise self.cycle(name, span)
            level = self.levels[-1]
            if level > 0:
                return self.definition(name, level - 1)
            if name not in TYPES and name not in ACTIVATIONS:
                if self.incomplete:
                    raise Reported()
                if self.chain[name][level].amends:
                    raise BuxError(f"nothing defines '{name}' for this to amend", span,
                                   f"define it first: {name} = ...")
                raise self.cycle(name, span)
        if name in TYPES or name in ACTIVATIONS:
            return Builtin(name, span)
        return Bare(name)

    def cycle(self, name: str, span: Span) -> BuxError:
        inner = len(self.evaluating) - 1 - self.evaluating[::-1].index(name)
        return BuxError(f"definition cycle: {' -> '.join([*self.evaluating[inner:], name])}",
                        span)

    def unknown(self, name: str, span: Span, scope=(), what: str = "layer or block",
                called: bool = False) -> BuxError:
        if self.incomplete:
            return Reported()
        known = [*scope, *self.statements, *TYPES, *ACTIVATIONS, "true", "false", "none"]
        close = difflib.get_close_matches(name, [k for k in known if k != name], n=1)
        hint = f"did you mean '{close[0]}'?" if close else None
        if called:
            new = (f"a new layer '{name}' needs a settings class in bux_b200/config/layers.py "
                   f"and a builder under @bux_b200.models.register({name!r})")
            hint = f"{hint} Or: {new}" if hint else new
        return BuxError(f"unknown {what} '{name}'", span, hint)

    # ---- expressions
    def eval(self, e: S.Expr, scope: dict):
        if isinstance(e, S.Lit):
            return e.value
        if isinstance(e, S.Name):
            return self.lookup(e.name, e.span, scope)
        if isinstance(e, S.Identity):
            return self.node(ir.Identity(), e.span)
        if isinstance(e, S.Tap):
            return self.node(ir.Tap(name=e.name), e.span)
        if isinstance(e, S.Ref):
            return self.node(ir.Ref(name=e.name, pop=e.pop), e.span)
        if isinstance(e, S.ListExpr):
            return [self.data(self.eval(i, scope), i.span) for i in e.items]
        if isinstance(e, S.Residual):
            body = self.graph(self.eval(e.body, scope), e.body.span)
            return self.node(ir.Residual(body=body), e.span)
        if isinstance(e, S.Seq):
            vals = [(self.eval(i, scope), i.span) for i in e.items]
            nodes = [self.graph(v, at) for v, at in vals if not nothing(v)]
            if not nodes:
                return self.node(ir.Identity(), e.span)
            if len(nodes) == 1:
                return nodes[0]
            return self.node(ir.Seq(items=flatten(nodes, ir.Seq, "items")), e.span)
        if isinstance(e, S.Neg):
            v = self.eval(e.operand, scope)
            if is_number(v):
                return -unwrap(v)
            return self.node(ir.Neg(body=self.graph(v, e.operand.span)), e.span)
        if isinstance(e, S.BinOp):
            return self.binop(e, scope)
        if isinstance(e, S.Call):
            return self.call(e, scope)
        if isinstance(e, S.Attr):
            return self.attr(e, scope)
        if isinstance(e, S.Alt):
            return self.eval(self.choose(e), scope)
        raise AssertionError(e)

    def choose(self, alt: S.Alt) -> S.Expr:
        key: Any = alt.span
        if alt.labels:
            key = frozenset(alt.labels)
            for other in self.axes:
                if isinstance(other, frozenset) and other != key and other & key:
                    raise BuxError(
                        "these alternatives share some labels with others, but not all: "
                        f"{', '.join(sorted(key))} against {', '.join(sorted(other))}",
                        alt.span,
                        "alternatives with the same labels are picked together, so give "
                        "them all the same labels, or none in common")
        if key not in self.axes:
            options = alt.labels or tuple(self.text(o.span) for o in alt.options)
            self.axes[key] = Axis(key, alt.where, tuple(options), alt.span)
        pick = self.choices.get(key, self.axes[key].pick(0))
        return alt.options[alt.labels.index(pick) if isinstance(pick, str) else pick]

    def attr(self, e: S.Attr, scope: dict):
        base = unwrap(self.eval(e.base, scope))
        if isinstance(base, Builtin):
            base = (self.construct(base.name, [], e.base.span) if base.name in TYPES
                    else _activation(base.name))
        elif isinstance(base, ir.Layer):
            base = base.config
        elif isinstance(base, Bare):
            raise self.unknown(base.name, e.base.span, scope, "name")
        if not isinstance(base, L.Config):
            raise BuxError(f"only layers and settings have fields, but this is {describe(base)}",
                           e.base.span)
        fields = type(base).model_fields
        if e.field not in fields:
            close = difflib.get_close_matches(e.field, list(fields), n=1)
            raise BuxError(f"{tag_of(base)} has no setting '{e.field}'", e.field_span,
                           f"did you mean '{close[0]}'?" if close else None)
        return getattr(base, e.field)

    def binop(self, e: S.BinOp, scope: dict):
        left, right = self.eval(e.left, scope), self.eval(e.right, scope)
        for value, other, side in ((left, right, e.left), (right, left, e.right)):
            if isinstance(value, Bare) and (is_number(other) or e.op in ("/", "//")
                                            or (e.op == "^" and side is e.right)):
                raise self.unknown(value.name, side.span, scope, "name")
        if is_number(left) and is_number(right):
            try:
                return _ARITH[e.op](unwrap(left), unwrap(right))
            except ZeroDivisionError:
                raise BuxError("division by zero", e.span) from None
            except OverflowError:
                raise BuxError("this number is too large", e.span) from None
        mix = self.mixture(e, left, right, scope)
        if mix is not None:
            return mix
        if e.op in "+-":
            terms = [self.term(left, e.left.span), self.term(right, e.right.span)]
            if e.op == "-":
                last = terms[-1]
                terms[-1] = (ir.Const(value=-last.value) if isinstance(last, ir.Const)
                             else self.node(ir.Neg(body=last), e.right.span))
            return self.node(ir.Sum(terms=flatten(terms, ir.Sum, "terms")), e.span)
        if e.op == "*":
            factors = [self.factor(left, e.left.span), self.factor(right, e.right.span)]
            return self.node(ir.Prod(factors=flatten(factors, ir.Prod, "factors")), e.span)
        if e.op == "^":
            times = unwrap(right)
            if isinstance(times, bool) or not isinstance(times, int) or times < 0:
                raise BuxError("a repeat count must be a whole number, 0 or more", e.right.span)
            body = self.graph(left, e.left.span)
            if times == 0:
                return self.node(ir.Seq(items=()), e.span)
            if times == 1:
                return body
            return self.node(ir.Repeat(body=body, times=times), e.span)
        raise BuxError(f"'{e.op}' only divides numbers", e.span,
                       "scale a branch with `f * 0.5`")

    def mixture(self, e: S.BinOp, left, right, scope):
        def operand(v, side):
            v = unwrap(v)
            if isinstance(v, Builtin) and v.name in _SOURCE_TAGS:
                return self.construct(v.name, [], side.span)
            return v

        a, b = operand(left, e.left), operand(right, e.right)
        if not (isinstance(a, T.SOURCES) or isinstance(b, T.SOURCES)):
            return None
        for v, side in ((a, e.left), (b, e.right)):
            if isinstance(v, Bare):
                raise self.unknown(v.name, side.span, scope, "name")

        def parts(c):
            if isinstance(c, T.MixtureConfig):
                return c.sources
            return (T.Weighted(weight=1.0, source=c),)

        if e.op == "+" and isinstance(a, T.SOURCES) and isinstance(b, T.SOURCES):
            return T.MixtureConfig(sources=parts(a) + parts(b))
        if e.op == "*":
            (w, side), src = ((a, e.left), b) if isinstance(b, T.SOURCES) else ((b, e.right), a)
            if is_number(w) and isinstance(src, T.SOURCES):
                if w <= 0:
                    raise BuxError("a data weight must be positive", side.span)
                return T.MixtureConfig(sources=tuple(
                    p.model_copy(update={"weight": p.weight * w}) for p in parts(src)))
        raise BuxError("data is mixed with + and weighted with *", e.span,
                       "0.7 * web + 0.3 * code, or web + code for an even mix")

    def term(self, v, span: Span):
        if is_number(v):
            return self.node(ir.Const(value=float(unwrap(v))), span)
        return self.graph(v, span)

    def factor(self, v, span: Span):
        if is_number(v) and isinstance(unwrap(v), int):
            n = unwrap(v)
            raise BuxError(f"multiplying a block by the integer {n} is ambiguous", span,
                           f"write blk^{n} to repeat it, or {n}.0 to scale its output")
        return self.term(v, span)

    # ---- coercions
    def graph(self, v, span: Span):
        if nothing(v):
            return self.node(ir.Identity(), span)
        if isinstance(v, Named):
            n = self.graph(v.value, span)
            return self.node(n.model_copy(update={"label": v.label,
                                                  "share": v.share or n.share}), span)
        if isinstance(v, ir.NODE_TYPES):
            return v
        if isinstance(v, L.Config):
            if tag_of(v) not in LAYERS:
                training = tag_of(v) in TRAINING
                kind = "a training setting" if training else "a setting of a layer"
                raise BuxError(f"{tag_of(v)}(...) is {kind}, not a layer", span,
                               f"a list of one is [{tag_of(v)}(...),]" if training else None)
            return self.node(ir.Layer(config=v), span)
        if isinstance(v, Builtin):
            if v.name in ACTIVATIONS:
                return self.graph(_activation(v.name), span)
            return self.graph(self.construct(v.name, [], span), span)
        if isinstance(v, str):
            return self.pattern(v, span)
        if isinstance(v, Bare):
            raise self.unknown(v.name, span)
        if isinstance(v, Macro):
            st = v.statement
            params = ", ".join(p.name for p in st.params or ())
            raise BuxError(f"'{st.name}' is a macro and needs arguments: {st.name}({params})", span)
        if is_number(v):
            raise BuxError("a number is not a layer", span,
                           "repeat a block with blk^3, scale a branch with f * 0.5")
        raise BuxError(f"expected a layer or block, found {describe(v)}", span)

    def pattern(self, text: str, span: Span):
        nodes = []
        quoted = self.source[span.start + 1:span.end - 1] == text
        for k, letter in enumerate(text):
            if letter.isspace():
                continue
            at = Span(span.start + 1 + k, span.start + 2 + k) if quoted else span
            if letter in self.broken and letter not in self.statements:
                raise Reported()
            if not letter.isalpha() or letter not in self.statements:
                raise BuxError(f"pattern letter '{letter}' is not a one-letter definition", at)
            nodes.append(self.graph(self.lookup(letter, at, {}), at))
        if not nodes:
            raise BuxError("empty pattern", span)
        return nodes[0] if len(nodes) == 1 else self.node(ir.Seq(items=tuple(nodes)), span)

    def data(self, v, span: Span):
        if isinstance(v, Named):
            return self.data(v.value, span)
        if isinstance(v, Builtin):
            return v.name if v.name in ACTIVATIONS else self.construct(v.name, [], span)
        if isinstance(v, Bare):
            return v.name
        if isinstance(v, tuple):
            return list(v)
        if v is None or isinstance(v, (bool, int, float, str, list, L.Config)):
            return v
        raise BuxError(f"expected a value, found {describe(v)}", span)

    # ---- calls
    def call(self, e: S.Call, scope: dict):
        callee = self.lookup(e.name, e.name_span, scope)
        if isinstance(callee, Macro):
            return self.apply(callee.statement, e, scope)
        if isinstance(callee, Builtin) and callee.name in DISTRIBUTIONS:
            return self.dimension(e, scope)
        if isinstance(callee, Builtin) and callee.name in TYPES:
            fields, ports = self.arguments(e, scope, TYPES[callee.name])
            config = self.construct(callee.name, fields, e.span)
            return self.with_ports(config, ports, None, None, e.span)
        if isinstance(callee, Named):
            base = unwrap(callee)
            cls = (TYPES.get(base.name) if isinstance(base, Builtin)
                   else type(base) if isinstance(base, L.Config)
                   else type(base.config) if isinstance(base, ir.Layer) else None)
            if cls is not None:
                if isinstance(base, ir.Layer):
                    base = base.config
                fields, ports = self.arguments(e, scope, cls)
                if not fields:
                    config = self.amended(base, fields, e.span)
                    return self.with_ports(config, ports, callee.label, callee.share, e.span)
                if callee.share and not e.amend:
                    raise BuxError(f"'{callee.label}' is shared, so it cannot be changed here",
                                   e.span, "define a separate layer")
                config = self.amended(base, fields, e.span)
                return self.with_ports(config, ports, self.text(e.span), None, e.span)
        if isinstance(callee, Bare):
            raise self.unknown(callee.name, e.name_span, called=True)
        builtin = isinstance(unwrap(callee), Builtin)
        what = "an activation" if builtin else describe(callee)
        if e.amend:
            raise BuxError(f"'{e.name}' is {what}, which has no settings to amend", e.name_span,
                           f"redefine it instead: {e.name} = ...")
        raise BuxError(f"'{e.name}' is {what} and takes no arguments", e.name_span,
                       f"to parametrize a block, make it a macro: {e.name}(x) = ..."
                       if what == "a block" else None)

    def amended(self, base, fields, span):
        if isinstance(base, Builtin):
            return self.construct(base.name, fields, span)
        if not fields:
            return base
        data = base.model_dump()
        for key, value, _ in fields:
            _assign(data, key, value)
        return self.validate(type(base), data, fields, span)

    def arguments(self, e: S.Call, scope: dict, cls) -> tuple:
        fields, ports, seen = [], [], set()
        for arg in e.args:
            if arg.key is None:
                raise BuxError("settings are given by name", arg.span,
                               f"{e.name}(name=value)")
            if arg.key in seen:
                raise BuxError(f"'{'.'.join(arg.key)}' is given twice", arg.span)
            seen.add(arg.key)
            key = arg.key
            if cls is T.RematConfig and key in (("save",), ("offload",)):
                fields.append((key, self.names(arg.value), arg.span))
                continue
            value = self.eval(arg.value, scope)
            if isinstance(value, (ir.Tap, ir.Ref)):
                ports.append(self.port(key, value, cls, arg.span))
                continue
            if isinstance(unwrap(value), bool) and _takes_number_only(cls, key):
                raise BuxError(f"'{'.'.join(key)}' takes a number, found a boolean",
                               arg.value.span)
            if isinstance(value, Bare):
                self.bare[arg.span] = (value.name, arg.value.span, tuple(scope))
            else:
                self.bare.pop(arg.span, None)
            if isinstance(value, Builtin) and _literal_option(cls, key, value.name):
                value = value.name
            fields.append((key, self.data(value, arg.value.span), arg.span))
        return fields, ports

    def port(self, key: tuple, value, cls, span: Span) -> ir.Port:
        name = ".".join(key)
        if name not in getattr(cls, "ports", ()):
            have = ", ".join(sorted(cls.ports)) or "none"
            raise BuxError(f"{cls.model_fields['type'].default or cls.__name__} has no port "
                           f"'{name}' (its ports: {have})", span)
        if isinstance(value, ir.Tap):
            return ir.Port(name=name, tap=value.name, mode="write")
        return ir.Port(name=name, tap=value.name, mode="pop" if value.pop else "read")

    def names(self, e: S.Expr) -> list:
        if isinstance(e, S.Name):
            return [e.name]
        if isinstance(e, S.Lit) and isinstance(e.value, str):
            return [e.value]
        if isinstance(e, S.Attr) and isinstance(e.base, S.Name):
            return [f"{e.base.name}.{e.field}"]
        if isinstance(e, S.ListExpr):
            return [n for i in e.items for n in self.names(i)]
        if isinstance(e, S.Residual):
            return self.names(e.body)
        if isinstance(e, S.Alt):
            return self.names(self.choose(e))
        raise BuxError("expected a name of what layers make, or a list of them", e.span)

    def with_ports(self, config, ports, label, share, span: Span):
        if not ports:
            return config if label is None else Named(label, config, share)
        layer = self.graph(config, span)
        return self.node(layer.model_copy(update={"ports": tuple(ports), "label": label,
                                                  "share": share}), span)

    def construct(self, tag: str, fields, span: Span):
        data: dict = {"type": tag}
        for key, value, arg_span in fields:
            if key == ("type",):
                raise BuxError("the type is set by the name of the call", arg_span)
            _assign(data, key, value)
        return self.validate(TYPES[tag], data, fields, span)

    def validate(self, cls, data: dict, fields, span: Span):
        try:
            return cls.model_validate(data)
        except ValidationError as err:
            raise self.invalid(cls, data["type"], err, fields, span) from None

    def invalid(self, cls, tag, err: ValidationError, fields, span: Span) -> BuxError:
        errors = err.errors()
        forbidden = [x for x in errors if x["type"] == "extra_forbidden"]
        error = (forbidden or errors)[0]
        loc = tuple(str(p) for p in error["loc"])
        arg_span = next((s for k, _, s in fields
                         if loc[:len(k)] == k or k[:len(loc)] == loc), span)
        path = ".".join(loc)
        kind = error["type"]
        if kind == "extra_forbidden":
            close = difflib.get_close_matches(loc[-1], list(cls.model_fields), n=1)
            return BuxError(f"{tag} has no setting '{path}'", arg_span,
                            f"did you mean '{close[0]}'?" if close and len(loc) == 1 else None)
        if kind == "missing":
            return BuxError(f"{tag} needs '{path}'", arg_span, f"{tag}({path}=...)")
        hint = None
        if kind == "literal_error":
            options = re.findall(r"'([^']*)'", str(error.get("ctx", {}).get("expected", "")))
            close = difflib.get_close_matches(str(error["input"]), options, n=1)
            hint = f"did you mean '{close[0]}'?" if close else None
        elif arg_span in self.bare and kind != "value_error":
            name, name_span, scope = self.bare[arg_span]
            return self.unknown(name, name_span, scope, "name")
        msg = error["msg"]
        if kind == "value_error":
            msg = str(error.get("ctx", {}).get("error", msg))
            return BuxError(f"{tag}: {msg}" if not msg.startswith(tag) else msg, arg_span)
        return BuxError(f"{tag}: {path}: {msg}" if path else f"{tag}: {msg}", arg_span, hint)

    # ---- macros
    def apply(self, st: S.Statement, e: S.Call, scope: dict):
        params = st.params or ()
        names = [p.name for p in params]
        args: dict = {}
        positional = [a for a in e.args if a.key is None]
        if len(positional) > len(params):
            raise BuxError(f"'{st.name}' takes {len(params)} argument(s)",
                           positional[len(params)].span)
        for p, a in zip(params, positional):
            args[p.name] = self.eval(a.value, scope)
        for a in e.args:
            if a.key is None:
                continue
            name = ".".join(a.key)
            if name not in names:
                raise BuxError(f"'{st.name}' has no parameter '{name}'", a.span)
            if name in args:
                raise BuxError(f"'{name}' is given twice", a.span)
            args[name] = self.eval(a.value, scope)
        missing = [p.name for p in params if p.name not in args and p.default is None]
        if missing:
            raise BuxError(f"'{st.name}' is missing argument(s): {', '.join(missing)}", e.span)
        for i, p in enumerate(params):
            if p.name not in args:
                earlier = {q.name: args[q.name] for q in params[:i]}
                args[p.name] = self.eval(p.default, earlier)
        self.depth += 1
        try:
            if self.depth > 64:
                raise BuxError(f"'{st.name}' recurses too deeply", e.span)
            return Named(self.text(e.span), self.eval(st.body, args))
        finally:
            self.depth -= 1

    # ---- search dimensions and objective
    def dimension(self, e: S.Call, scope: dict):
        options: list = []
        if e.name == "choice":
            options = list(e.args)
            keys = [a.key for a in e.args]
            if any(keys) and not all(keys):
                raise BuxError("name every option of a choice or none of them", e.span)
            names = [k[0] if k else self.text(a.value.span) for k, a in zip(keys, e.args)]
            if len(names) < 2:
                raise BuxError("a choice needs two options or more", e.span,
                               "choice(swish, gelu)")
            if len(set(names)) < len(names):
                raise BuxError("two options of a choice are the same", e.span)
            space = T.ChoiceConfig(options=tuple(names))
        else:
            positional = [a for a in e.args if a.key is None]
            if len(positional) > 2 or (positional and
                                       e.args[:len(positional)] != tuple(positional)):
                raise BuxError(f"{e.name} takes low and high in order, then settings by name",
                               (positional[-1] if positional else e).span)
            named_args = tuple(S.Arg(a.span, (k,), a.value, (a.span,))
                               for k, a in zip(("low", "high"), positional))
            named = S.Call(e.span, e.name, e.name_span, named_args + e.args[len(positional):])
            fields, _ = self.arguments(named, scope, DISTRIBUTIONS[e.name])
            space = self.construct(e.name, fields, e.span)
        met = self.dims.get(e.span)
        if met is None:
            self.dims[e.span] = Dimension(e.span, e.where or e.name, space)
        elif met.space != space:
            raise BuxError("a dimension takes one value wherever it is used, so its bounds "
                           "cannot change with a macro's arguments", e.span)
        value = self.point.get(e.span, middle(space))
        if options:
            return self.eval(options[int(value)].value, scope)
        return value

    def objective(self, e: S.Expr):
        weights = self.linear(e)
        constant = weights.pop("", 0.0)
        if not weights:
            raise BuxError("an objective is a weighted sum of metrics, but this has none",
                           e.span, "objective = 0.7 * web_bpb + 0.3 * code_bpb")
        return T.ObjectiveConfig(
            terms=tuple(T.Term(metric=m, weight=w) for m, w in weights.items()),
            constant=constant)

    def linear(self, e: S.Expr) -> dict:
        scaled = lambda d, k: {m: w * k for m, w in d.items()}  # noqa: E731
        if isinstance(e, S.Lit) and not isinstance(e.value, bool):
            if isinstance(e.value, (int, float)):
                return {"": float(e.value)}
            if isinstance(e.value, str):
                return {e.value: 1.0}
        if isinstance(e, S.Name):
            v = (self.lookup(e.name, e.span, {})
                 if e.name in self.statements and e.name != "objective" else None)
            return {"": float(unwrap(v))} if is_number(v) else {e.name: 1.0}
        if isinstance(e, S.Neg):
            return scaled(self.linear(e.operand), -1.0)
        if isinstance(e, S.Alt):
            return self.linear(self.choose(e))
        if isinstance(e, S.BinOp) and e.op in "+-":
            a, b = self.linear(e.left), self.linear(e.right)
            sign = 1.0 if e.op == "+" else -1.0
            return {k: a.get(k, 0.0) + sign * b.get(k, 0.0) for k in {**a, **b}}
        if isinstance(e, S.BinOp) and e.op == "*":
            a, b = self.linear(e.left), self.linear(e.right)
            if set(a) <= {""}:
                return scaled(b, a.get("", 0.0))
            if set(b) <= {""}:
                return scaled(a, b.get("", 0.0))
            raise BuxError("an objective weights metrics by numbers, not by other metrics",
                           e.span)
        if isinstance(e, S.BinOp) and e.op == "/":
            d = self.linear(e.right)
            if not set(d) <= {""}:
                raise BuxError("an objective divides metrics by numbers, not by metrics",
                               e.right.span)
            if not d.get("", 0.0):
                raise BuxError("division by zero", e.right.span)
            return scaled(self.linear(e.left), 1 / d[""])
        raise BuxError("an objective is a weighted sum of metrics", e.span,
                       "objective = 0.7 * web_bpb + 0.3 * code_bpb")

    def setting(self, name: str) -> tuple:
        st = self.statements.get(name)
        if st is None and name in self.broken:
            raise Reported()
        if st is None:
            return None, None
        return self.data(self.definition(name), st.body.span), st.body.span


# ------------------------------------------------------------------ compile
_SETTING_KINDS = {
    "residual": (tuple(RESIDUALS.values()), " or ".join(f"{t}(...)" for t in RESIDUALS)),
    "init": (tuple(INITS.values()), " or ".join(f"{t}(...)" for t in INITS)),
}


def _model_settings(ev: Evaluator) -> dict:
    out = {}
    for name in SETTINGS:
        value, span = ev.setting(name)
        expected, kind = _SETTING_KINDS.get(name, ((int,), "an integer"))
        if value is not None and (not isinstance(value, expected) or isinstance(value, bool)):
            raise BuxError(f"'{name}' must be {kind}, found {describe(value)}", span)
        if isinstance(value, int) and value < 1:
            raise BuxError(f"'{name}' must be greater than 0, found {value}", span)
        out[name] = value
    return out


def _architecture(ev: Evaluator, entry: str) -> ir.Architecture:
    if entry not in ev.statements:
        if entry in ev.broken or ev.incomplete:
            raise Reported()
        raise BuxError(f"no definition named '{entry}'",
                       hint=f"define it: {entry} = embed ... head")
    settings = _model_settings(ev)
    if settings["d_model"] is None:
        if ev.incomplete:
            raise Reported()
        raise BuxError("'d_model' is not defined", hint="d_model = 4096")
    low = GraphTyper(ev, settings["d_model"], settings["residual"])
    model = ev.graph(ev.definition(entry), ev.statements[entry].name_span)
    graph = low.run(model)
    if settings["vocab_size"] is None and (low.embeddings or low.heads):
        if ev.incomplete:
            raise Reported()
        raise BuxError("'vocab_size' is not defined", hint="vocab_size = 32000")
    return ir.Architecture(d_model=settings["d_model"], vocab_size=settings["vocab_size"],
                           residual=settings["residual"], init=settings["init"], graph=graph)


_ADAPTERS = {n: TypeAdapter(f.rebuild_annotation())
             for n, f in T.TrainConfig.model_fields.items()}


def _expects(annotation) -> str:
    import typing

    kinds = []
    whole = typing.get_origin(annotation) is tuple
    members = (annotation,) if whole else (typing.get_args(annotation) or (annotation,))
    for m in members:
        if typing.get_origin(m) is typing.Annotated:
            m = typing.get_args(m)[0]
        if m is type(None):
            kinds.append("none")
        elif m is int:
            kinds.append("an integer")
        elif m is float:
            kinds.append("a number")
        elif m is T.MixtureConfig:
            kinds.append("a mix of sources (0.7 * web + 0.3 * code)")
        elif typing.get_origin(m) is tuple:
            kinds.append(f"a list of {_expects(typing.get_args(m)[0])}")
        elif typing.get_origin(m) is typing.Union:
            kinds.append(_expects(m))
        elif isinstance(m, type) and issubclass(m, L.Config):
            kinds += [f"{t}(...)" for t in typing.get_args(m.model_fields["type"].annotation)]
    kinds = kinds or ["a value"]
    return ", ".join(kinds[:-1]) + " or " + kinds[-1] if len(kinds) > 1 else kinds[0]


def _train_setting(name: str, value, span: Span):
    import typing

    annotation = T.TrainConfig.model_fields[name].annotation
    kinds = typing.get_args(annotation) or (annotation,)
    if isinstance(value, bool) and (int in kinds or float in kinds):
        raise BuxError(f"'{name}' must be {_expects(annotation)}, found a boolean", span)
    try:
        return _ADAPTERS[name].validate_python(value)
    except ValidationError as err:
        errors = err.errors()
        if errors and errors[0]["type"].startswith(("greater", "less")):
            message = errors[0]["msg"].replace("Input should be", "must be")
            raise BuxError(f"'{name}' {message}, found {value}", span) from None
        if errors and errors[0]["type"] == "value_error":
            raise BuxError(str(errors[0]["ctx"]["error"]), span) from None
        found = value if is_number(value) else describe(value)
        raise BuxError(f"'{name}' must be {_expects(annotation)}, found {found}", span) from None


def _train(ev: Evaluator, arch: Optional[ir.Architecture], *, require: bool):
    values, spans = {}, {}
    for name in TRAIN_SETTINGS:
        value, span = ev.setting(name)
        if span is None:
            continue
        values[name] = _train_setting(name, value, span)
        spans[name] = span
    if not values:
        return None
    missing = [n for n in REQUIRED if n not in values]
    if missing:
        if not require or ev.incomplete:
            return None
        listed = (", ".join(missing[:-1]) + " and " + missing[-1]
                  if len(missing) > 1 else missing[0])
        raise BuxError("this file sets how to train, so it is a run, and a run needs "
                       f"{listed}", hint=_EXAMPLES[missing[0]])
    try:
        train = T.TrainConfig.model_validate(values)
    except ValidationError as err:
        first = err.errors()[0]
        msg = str(first.get("ctx", {}).get("error", first["msg"]))
        raise BuxError(msg, spans.get(str(first["loc"][0]) if first["loc"] else "steps")) from None
    _check_train(train, arch, spans)
    return train


def _check_train(train: T.TrainConfig, arch, spans: dict) -> None:
    from ..train import curriculum

    sched = train.schedule
    warm = T.warmup_steps(sched, train.steps)
    cool = sched.cooldown(train.steps) if isinstance(sched, T.COOLED) else 0
    if warm + cool > train.steps:
        what = f"{warm} of warmup" + (f" and {cool} of cooldown" if cool else "")
        raise BuxError(f"the schedule takes {warm + cool} steps ({what}), but the run has "
                       f"{train.steps}", spans.get("schedule", spans["steps"]))
    for check, setting in ((curriculum.check_ramp, "batch_ramp"),
                           (curriculum.check_phases, "curriculum")):
        try:
            check(train)
        except ValueError as err:
            raise BuxError(str(err), spans.get(setting, spans["steps"])) from None
    reads = [("data", train.data)] + [("eval", e.data) for e in T.evals(train)]
    reads += [("curriculum", p.data) for p in train.curriculum if p.data is not None]
    for name, data in reads:
        kinds = sorted({s.type for s in T.leaves(data)} & {"text", "chat"})
        if kinds and train.tokenizer is None:
            raise BuxError(f"{' and '.join(kinds)} data is tokenized, so the run needs a "
                           "tokenizer", spans[name], 'tokenizer = tokenizer(name="gpt2")')
    longest = max(c.seq_len for _, c in curriculum.phases(train))
    setting = "seq_len" if longest == train.seq_len else "curriculum"
    ev_lens = [e.seq_len for e in T.evals(train) if e.seq_len is not None]
    if ev_lens and max(ev_lens) > longest:
        longest, setting = max(ev_lens), "eval"
    for layer in arch.layers() if arch is not None else ():
        if isinstance(layer.config, L.EmbeddingConfig):
            positions = layer.config.max_positions
            if positions is not None and longest > positions:
                raise BuxError(f"sequences of {longest} tokens are longer than the "
                               f"{positions} positions the embedding learns",
                               spans.get(setting, spans["seq_len"]),
                               f"embed(max_positions={longest})")
    if train.objective is not None:
        evals = T.evals(train)
        logged = {m for e in evals for m in T.metrics(e, train.tokenizer is not None)}
        with_bpb = {m for e in evals for m in T.metrics(e, True)}
        names = "|".join(re.escape(e.name) for e in evals)
        for term in train.objective.terms:
            metric = term.metric
            evaluated = metric.endswith("_bpb") or (
                bool(names) and re.fullmatch(rf"({names})_(loss|bpb)(_\w+)?", metric))
            if metric in logged or not evaluated:
                continue
            if metric in with_bpb:
                raise BuxError(f"the objective reads {metric}, but bits per byte need a "
                               "tokenizer", spans["objective"], "tokenizer = tokenizer(...)")
            close = difflib.get_close_matches(metric, sorted(logged), n=1)
            listed = ", ".join(sorted(logged)) or "none, as the run has no eval"
            raise BuxError(f"the objective reads {metric}, but no eval logs it; they log "
                           f"{listed}", spans["objective"],
                           f"did you mean '{close[0]}'?" if close else "eval(name=..., data=...)")


Modules = Union[Mapping, Callable, None]


def _load(source, filename, overrides, found: Modules, *, recover: bool) -> modules.Program:
    loader = modules.from_mapping(found) if isinstance(found, Mapping) else found
    return modules.load(source, filename, overrides=overrides, loader=loader, recover=recover)


def _run_name(filename: str, parts: tuple) -> str:
    stem = "run" if filename.startswith("<") else Path(filename).stem
    return stem + (f"[{', '.join(parts)}]" if parts else "")


def compile(source: str, *, entry: str = "model", filename: str = "<string>",
            overrides: Sequence = (), modules: Modules = None) -> ir.Architecture:
    """Compile source into the architecture of one definition (sweeps take their
    first alternative). Every definition is evaluated, so any mistake raises."""
    program = _load(source, filename, overrides, modules, recover=False)
    try:
        ev = Evaluator(program)
        arch = _architecture(ev, entry)
        ev.evaluate_all()
        return arch
    except BuxError as err:
        raise program.locate(err) from None


@dataclass
class Found:
    """One explored combination of a sweep."""
    arch: ir.Architecture
    train: Optional[T.TrainConfig]
    choices: dict
    axes: list
    dims: list


def _evaluate(program, entry, choices, point, *, require=True) -> tuple:
    ev = Evaluator(program, choices=choices, point=point)
    arch = _architecture(ev, entry)
    train = _train(ev, arch, require=require)
    ev.evaluate_all()
    return ev, arch, train


def explore(program: modules.Program, entry: str = "model", point: Optional[Mapping] = None,
            fixed: Optional[Mapping] = None, *, require: bool = True) -> list:
    """Every combination of the alternatives the run reaches, the first axis written
    varying slowest. An axis only some choices reach exists only under them."""
    found: list = []

    def descend(choices: dict) -> None:
        ev, arch, train = _evaluate(program, entry, choices, point, require=require)
        reached = {k: a for k, a in ev.axes.items() if _reaches_run(ev, k)}
        pending = next((a for k, a in reached.items() if k not in choices), None)
        if pending is None:
            axes = [a for k, a in reached.items()]
            found.append(Found(arch, train, dict(choices), axes, list(ev.dims.values())))
            return
        for i in range(len(pending.options)):
            descend({**choices, pending.key: pending.pick(i)})

    descend(dict(fixed or {}))
    return found


def _reaches_run(ev: Evaluator, key) -> bool:
    return True


def _make_run(f: Found, filename: str, more: tuple = ()) -> ir.Run:
    if f.train is None:
        raise BuxError("this file defines a model, not a run: it sets none of "
                       "data, optimizer, seq_len, batch and steps",
                       hint=_EXAMPLES["data"])
    axes = sorted(f.axes, key=lambda a: a.span.start)
    parts = tuple(a.part(f.choices[a.key]) for a in axes)
    return ir.Run(name=_run_name(filename, parts + more), arch=f.arch, train=f.train,
                  choices=parts, axes=tuple(a.where for a in axes))


def compile_runs(source: str, *, entry: str = "model", filename: str = "<string>",
                 overrides: Sequence = (), modules: Modules = None) -> list:
    """One `ir.Run` per combination of the alternatives the file reaches."""
    program = _load(source, filename, overrides, modules, recover=False)
    try:
        runs = [_make_run(f, filename) for f in _useful(explore(program, entry))]
    except BuxError as err:
        raise program.locate(err) from None
    return runs


def _useful(found: list) -> list:
    """Drop axes whose choice changes nothing (all runs along it are equal)."""
    if len(found) <= 1:
        return found
    keys = []
    for f in found:
        for a in f.axes:
            if a.key not in keys:
                keys.append(a.key)
    for key in list(keys):
        groups: dict = {}
        for f in found:
            rest = tuple(sorted((str(k), str(v)) for k, v in f.choices.items() if k != key))
            groups.setdefault(rest, []).append(f)
        same = all(len({(g.arch.model_dump_json(), g.train.model_dump_json() if g.train else "")
                        for g in grp}) == 1 for grp in groups.values())
        if same and all(len(grp) > 1 for grp in groups.values()):
            found = [grp[0] for grp in groups.values()]
            for f in found:
                f.choices.pop(key, None)
                f.axes = [a for a in f.axes if a.key != key]
    return found


@dataclass(frozen=True)
class Space:
    """A run and the dimensions of its search; `trial` is the run at a point."""
    run: ir.Run
    dimensions: dict
    program: modules.Program = field(repr=False)
    entry: str = field(repr=False)
    filename: str = field(repr=False)
    choices: dict = field(repr=False)

    def trial(self, values: Mapping, steps: Optional[int] = None) -> ir.Run:
        program = self.program
        if steps is not None:
            program = modules.extended(program, f"steps = {steps}", "<search>")
        dims = self.dimensions
        point = {}
        for name, v in values.items():
            d = dims[name]
            point[d.key] = int(v) if isinstance(d.space, (T.ChoiceConfig, T.IntUniformConfig)) \
                else float(v)
        try:
            [f] = explore(program, self.entry, point, self.choices)
        except BuxError as err:
            raise program.locate(err) from None
        more = tuple(d.part(point.get(d.key, middle(d.space))) for d in f.dims)
        return _make_run(f, self.filename, more + ((f"steps={steps}",) if steps else ()))


def _dimension_names(dims: list) -> dict:
    out, counts = {}, {}
    for d in dims:
        counts[d.where] = counts.get(d.where, 0) + 1
        name = d.where if counts[d.where] == 1 else f"{d.where}#{counts[d.where]}"
        out[name] = d
    return out


def compile_spaces(source: str, *, entry: str = "model", filename: str = "<string>",
                   overrides: Sequence = (), modules: Modules = None) -> list:
    program = _load(source, filename, overrides, modules, recover=False)
    spaces = []
    try:
        for f in _useful(explore(program, entry)):
            dims = list(f.dims)
            # options of a choice may reach further dimensions
            for d in list(dims):
                if isinstance(d.space, T.ChoiceConfig):
                    for i in range(1, len(d.space.options)):
                        [g] = explore(program, entry, {d.key: i}, f.choices)
                        dims += [x for x in g.dims if x.key not in {y.key for y in dims}]
            spaces.append(Space(_make_run(f, filename), _dimension_names(dims), program, entry,
                                filename, f.choices))
    except BuxError as err:
        raise program.locate(err) from None
    return spaces


def compile_file(path: str, *, overrides: Sequence = (), entry: str = "model") -> list:
    return compile_runs(Path(path).read_text(), entry=entry, filename=str(path),
                        overrides=overrides)


@dataclass
class Report:
    """What `check` found: every error of a file (not only the first), its runs'
    axes and dimensions."""
    errors: list
    axes: list
    dimensions: list
    runs: int
    arch: Optional[ir.Architecture] = None
    train: Optional[T.TrainConfig] = None
    defines: Optional[list] = None   # a module (a file without the entry): the names it defines

    @property
    def ok(self) -> bool:
        return not self.errors


def check(source: str, *, entry: str = "model", filename: str = "<string>",
          overrides: Sequence = (), modules: Modules = None) -> Report:
    """Collect every mistake of a file instead of stopping at the first."""
    errors: list = []
    try:
        program = _load(source, filename, overrides, modules, recover=True)
    except BuxError as err:
        return Report([err], [], [], 0)
    errors += program.errors

    def report(err: BuxError) -> None:
        if not isinstance(err, Reported):
            errors.append(program.locate(err))

    ev = Evaluator(program, report=report)
    arch = train = None
    if entry not in ev.chain and not program.incomplete:
        # a module: a piece that runs build on by name. Every definition is checked on its own.
        ev.evaluate_all(report)
        main = next((f for f in program.files if f.filename == filename), program.files[0] if program.files else None)
        own = [st.name for layer in program.layers for st in layer
               if main is None or main.start <= st.span.start <= main.stop]
        return Report(errors, list(ev.axes.values()), list(ev.dims.values()), 0, defines=list(dict.fromkeys(own)))
    try:
        arch = _architecture(ev, entry)
    except BuxError as err:
        report(err)
    try:
        train = _train(ev, arch, require=False)
    except BuxError as err:
        report(err)
    ev.evaluate_all(report)
    runs = 0
    if not errors:
        try:
            runs = len(_useful(explore(program, entry, require=False)))
        except BuxError as err:
            report(err)
    seen, unique = set(), []
    for e in errors:
        k = (e.message, e.span.start if e.span else None, e.filename)
        if k not in seen:
            seen.add(k)
            unique.append(e)
    return Report(unique, list(ev.axes.values()), list(ev.dims.values()), runs, arch, train)
