"""The typing pass over a model's graph: what flows into every layer.

A value flowing along the graph is one of four kinds: ``"tokens"`` (ids, before the
embedding), an ``int`` (hidden states of that width), ``"streams"`` (the residual
algebra's widened stream: several copies of the hidden states) or ``"logits"`` (after a
head). `GraphTyper` walks the graph once, stamps every layer with the kind it receives
(`ir.Layer.width`), inserts the ``merge`` that reads a widened stream back into one where a
plain layer meets it, and checks on the way what can only be checked with the kinds known:
branch and repeat bodies keep their width, parallel branches agree, taps are written
before they are read, ports meet ports, shared blocks are used alike.

Taps are stacks (``@h`` pushes, ``$h`` reads the top, ``$h!`` pops). `TapLedger` replays
those stacks over the walk, including every pass of a repeat, and tracks which labelled
block last read a value it also wrote, to catch a later read that would silently get
that block's private value instead of the one written before it.

Behaviour and messages follow the reference (``lang/compiler.py:1367-1700`` there, its
``_Lowering``); the structure here is this project's own.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Callable, Optional

from ..config import layers as L
from . import ir
from .syntax import BuxError

TOKENS, STREAMS, LOGITS = "tokens", "streams", "logits"


class PortValue:
    """What a tap holds after a layer wrote one of its ports to it (not hidden states)."""

    def __init__(self, port: str):
        self.port = port

    def __eq__(self, other):
        return isinstance(other, PortValue) and other.port == self.port

    def __hash__(self):
        return hash(("port", self.port))

    def __repr__(self):
        return f"PortValue({self.port!r})"


def splice(nodes, cls, attr) -> tuple:
    """`nodes` with every anonymous, unshared `cls` among them replaced by its children."""
    out = []
    for n in nodes:
        if isinstance(n, cls) and n.label is None and n.share is None:
            out.extend(getattr(n, attr))
        else:
            out.append(n)
    return tuple(out)


# ---------------------------------------------------------------- taps
class _Scope:
    """A labelled stretch of the walk: a named definition, or one pass of a repeat."""

    __slots__ = ("label", "reads")

    def __init__(self, label: str):
        self.label = label
        self.reads: list = []   # slots whose latest read happened with this scope as the meeting point


class _Slot:
    """One value on a tap's stack."""

    __slots__ = ("value", "written_in", "met_in", "private_to", "gone")

    def __init__(self, value, written_in: tuple):
        self.value = value
        self.written_in = written_in          # the scopes open when it was written, outermost first
        self.met_in: Optional[_Scope] = None  # innermost scope that holds both the write and the latest read
        self.private_to: Optional[str] = None  # label of a closed scope that wrote it, read it and left it
        self.gone = False


class TapLedger:
    """The tap stacks as the forward pass will see them."""

    def __init__(self, fail: Callable[..., BuxError]):
        self.fail = fail
        self.stacks: dict = {}
        self.open: list = []

    @contextmanager
    def scope(self, label: str):
        sc = _Scope(label)
        self.open.append(sc)
        try:
            yield sc
        finally:
            self.open.pop()
            # what this scope wrote, read for itself and did not pop stays on the stack as
            # its private value: a later reader most likely wants the value below it
            for slot in sc.reads:
                if slot.met_in is sc and not slot.gone:
                    slot.private_to = sc.label

    def push(self, tap: str, value) -> None:
        self.stacks.setdefault(tap, []).append(_Slot(value, tuple(self.open)))

    def take(self, tap: str, pop: bool):
        stack = self.stacks.get(tap)
        if stack is None:
            raise self.fail(f"tap '{tap}' is read before anything writes it", f"write it first with @{tap}")
        if not stack:
            raise self.fail(f"tap '{tap}' is empty: everything written to it was already popped")
        top = stack[-1]
        if top.private_to is not None:
            if any(below.private_to is None for below in stack[:-1]):
                who = top.private_to
                raise self.fail(
                    f"tap '{tap}' here reads the value that '{who}' wrote and read for "
                    "itself, not the one written before it",
                    f"pop it in '{who}' with ${tap}! where it is read last, or give one "
                    "of the two taps another name")
        else:
            meeting = None
            for then, now in zip(top.written_in, self.open):
                if then is not now:
                    break
                meeting = then
            if meeting is not None:
                top.met_in = meeting
                meeting.reads.append(top)
        if pop:
            stack.pop()
            top.gone = True
        return top.value


# ---------------------------------------------------------------- the walk
class GraphTyper:
    """One walk over an untyped graph; see the module's docstring.

    `source` gives the walk its link to the text: ``node_spans`` (id(node) → span),
    ``node(typed, span)`` to register a rebuilt node under the same span, and
    ``text(span)`` for quoting. After `run`, `embeddings` and `heads` count the layers of
    those kinds in the unrolled model."""

    #: layers that work on the widened stream's copies themselves under hc / mhc / gr
    ON_COPIES = (L.EngramConfig, L.NextNConfig, L.DocCopyConfig)

    def __init__(self, source, d_model: int, residual):
        self.source, self.d_model = source, d_model
        kind = residual.type if residual is not None else None
        self.widened = kind is not None and kind != "vpgate"
        self.copies = kind in ("hc", "mhc", "gr")
        self.depth = 0              # residual branches around the node being typed
        self.places: list = []      # spans of the nodes being typed, innermost last
        self.taps = TapLedger(self.fail)
        self.seen_shared: dict = {}
        self.embeddings = 0
        self.heads = 0
        self.need_one_embedding: list = []   # (what, span) of layers that borrow the embedding
        self.rules = {
            ir.Layer: self._layer, ir.Seq: self._sequence, ir.Residual: self._branch,
            ir.Sum: self._parallel, ir.Prod: self._parallel, ir.Neg: self._negated,
            ir.Const: lambda node, kind: (node, None), ir.Identity: lambda node, kind: (node, kind),
            ir.Repeat: self._repeat, ir.Tap: self._tap_write, ir.Ref: self._tap_read,
        }

    # ---- errors
    def fail(self, message: str, hint: Optional[str] = None) -> BuxError:
        return BuxError(message, self.places[-1] if self.places else None, hint)

    # ---- entry
    def run(self, graph):
        first = next(ir.unrolled_layers(graph), None)
        if first is not None and first.config.type == "embed":
            kind: Any = TOKENS
        else:
            kind = STREAMS if self.widened else self.d_model
        typed, _ = self.visit(graph, kind)
        if self.need_one_embedding and self.embeddings != 1:
            what, span = self.need_one_embedding[0]
            raise BuxError(f"{what} needs exactly one embedding, found {self.embeddings}", span)
        return typed

    def visit(self, node, kind):
        """(typed node, kind that leaves it). Labelled nodes open a tap scope; shared ones
        are compared with the other uses of the same module."""
        span = self.source.node_spans.get(id(node))
        if span is not None:
            self.places.append(span)
        try:
            rule = self.rules[type(node)]
            if node.label is not None and not isinstance(node, ir.Layer):
                with self.taps.scope(node.label):
                    typed, out = rule(node, kind)
            else:
                typed, out = rule(node, kind)
            if span is not None:
                self.source.node(typed, span)
            if node.share is not None:
                module = typed
                if isinstance(node, ir.Layer) and isinstance(typed, ir.Seq):
                    module = typed.items[-1]      # behind the merge that was put before it
                self._same_as_other_uses(node.share, module)
            return typed, out
        finally:
            if span is not None:
                self.places.pop()

    def _same_as_other_uses(self, share: str, typed) -> None:
        outside = self.depth == 0
        if share not in self.seen_shared:
            self.seen_shared[share] = (typed, outside)
        first, first_outside = self.seen_shared[share]
        if ir.strip(first, widths=False) != ir.strip(typed, widths=False):
            both_layers = isinstance(first, ir.Layer) and isinstance(typed, ir.Layer)
            if both_layers and first.ports != typed.ports:
                raise self.fail(f"shared '{share}' is one module, so every use of it takes "
                                "the same ports")
            raise self.fail(f"shared '{share}' is used where it would need different widths")
        has_branches = any(isinstance(n, ir.Residual) for n in ir.walk(typed))
        if outside != first_outside and has_branches:
            raise self.fail(
                f"shared '{share}' has residual branches and is used both outside residual "
                "branches and inside one, where its branches are built another way",
                "define a separate block for the uses inside branches")

    # ---- composite nodes
    def _sequence(self, node, kind):
        items = []
        for item in node.items:
            typed, kind = self.visit(item, kind)
            items.append(typed)
        return ir.with_children(node, splice(items, ir.Seq, "items")), kind

    def _parallel(self, node, kind):
        typed, kinds = [], []
        for term in ir.children(node):
            t, out = self.visit(term, kind)
            typed.append(t)
            if out is not None and out not in kinds:   # a constant takes any width
                kinds.append(out)
        if not kinds:
            raise self.fail("parallel branches need at least one layer")
        if len(kinds) > 1:
            raise self.fail("parallel branches disagree on width: "
                            f"{', '.join(map(str, kinds))}")
        return ir.with_children(node, tuple(typed)), kinds[0]

    def _negated(self, node, kind):
        typed, out = self.visit(node.body, kind)
        return ir.with_children(node, (typed,)), out

    def _branch(self, node, kind):
        body = node.body
        if isinstance(body, ir.Layer) and isinstance(body.config, L.EngramConfig):
            raise self.fail("engram adds to the stream itself, so [engram] would add the "
                            "stream twice", "write it bare: ... engram ...")
        inside = kind
        if self.widened and self.depth == 0:
            # a top-level branch hangs off the widened stream and sees one copy's width
            if kind != STREAMS:
                extra = ", engram and nextn" if self.copies else ""
                raise self.fail(
                    "a residual branch needs the widened residual stream, but it was read "
                    "back into one before this",
                    f"only branches, taps{extra} keep it; save it with @h and go on from $h")
            inside = self.d_model
        elif not isinstance(kind, int):
            raise self.fail(f"a residual branch needs hidden states, but receives {kind}")
        self.depth += 1
        try:
            typed, out = self.visit(body, inside)
        finally:
            self.depth -= 1
        if out != inside:
            raise self.fail("a residual branch must keep the width, but this one maps "
                            f"{inside} to {out}")
        return ir.with_children(node, (typed,)), kind

    def _repeat(self, node, kind):
        span = self.source.node_spans.get(id(node.body))
        text = self.source.text(span) if span is not None else "the block"
        shown = f"({text})" if " " in text else text
        label = f"one pass of {shown}^{node.times}"
        with self.taps.scope(label):
            typed, out = self.visit(node.body, kind)
        if out != kind:
            raise self.fail("a repeated block must keep the width, but this one maps "
                            f"{kind} to {out}")
        touches_taps = any(isinstance(n, (ir.Tap, ir.Ref)) or (isinstance(n, ir.Layer) and n.ports)
                           for n in ir.walk(node.body))
        if touches_taps:
            # the other passes change nothing but the tap stacks: replay them for those
            for _ in range(node.times - 1):
                with self.taps.scope(label):
                    self.visit(node.body, kind)
        else:
            more = node.times - 1
            for n in ir.walk(node.body):
                if isinstance(n, ir.Layer) and n.config.type == "embed":
                    self.embeddings += more
                elif isinstance(n, ir.Layer) and n.config.type == "head":
                    self.heads += more
        return ir.with_children(node, (typed,)), kind

    # ---- taps in the graph
    def _tap_write(self, node, kind):
        self.taps.push(node.name, kind)
        return node, kind

    def _tap_read(self, node, kind):
        tap = node.name
        value = self.taps.take(tap, node.pop)
        if isinstance(value, PortValue):
            raise self.fail(f"tap '{tap}' holds the '{value.port}' port of a layer",
                            f"read it through the same port: layer({value.port}=${tap})")
        if value == STREAMS and self.depth > 0:
            raise self.fail(f"tap '{tap}' holds the widened residual stream, which only "
                            "exists outside residual branches",
                            f"read it back into one first: merge @{tap}")
        return node, value

    # ---- layers
    def _layer(self, node: ir.Layer, kind):
        config = node.config
        if kind == LOGITS:
            raise self.fail("nothing can follow the LM head",
                            "to go on after a head, read a tap: @h norm head $h ...")
        takes_streams = isinstance(config, (L.MergeConfig, L.ValueEmbeddingConfig)) or (
            self.copies and isinstance(config, self.ON_COPIES))
        if kind == STREAMS and not takes_streams:
            # a plain layer on the widened stream: read the stream back into one first
            merge = ir.Layer(config=L.MergeConfig(), width=STREAMS)
            typed, out = self._layer(node, self.d_model)
            span = self.source.node_spans.get(id(node))
            if span is not None:
                self.source.node(typed, span)
            return ir.Seq(items=(merge, typed)), out
        out = self._leaves(config, kind)
        reads_first = sorted(node.ports, key=lambda p: p.mode == "write")
        for port in reads_first:
            if port.mode == "write":
                self.taps.push(port.tap, PortValue(port.name))
                continue
            value = self.taps.take(port.tap, port.mode == "pop")
            if not isinstance(value, PortValue) or value.port != port.name:
                held = f"the '{value.port}' port" if isinstance(value, PortValue) else "hidden states"
                raise self.fail(f"port '{port.name}' reads tap '{port.tap}', which holds {held}")
        return node.model_copy(update={"width": kind}), out

    def _leaves(self, config, kind):
        """The kind that leaves a layer of `config` fed `kind` (and the layer's own checks)."""
        top_level_widened = self.widened and self.depth == 0
        if isinstance(config, L.MergeConfig):
            if kind != STREAMS:
                raise self.fail(
                    "merge reads a widened residual stream back into one, but there is none "
                    "here",
                    None if self.widened else
                    "widen it with residual = hc(...), mhc(...), gr(...), attnres(...) or msar(...)")
            return self.d_model
        if config.type == "embed":
            if kind != TOKENS:
                raise self.fail("an embedding takes token ids, so it must come first")
            self.embeddings += 1
            return STREAMS if top_level_widened else self.d_model
        if kind == TOKENS:
            raise self.fail(f"{config.type} needs hidden states, but receives token ids",
                            "start with an embedding")
        if isinstance(config, L.LMHeadConfig):
            self.heads += 1
            if config.tied and self.places:
                self.need_one_embedding.append(("a tied head", self.places[-1]))
            return LOGITS
        if isinstance(config, L.LinearConfig):
            return config.features
        if isinstance(config, L.NextNConfig):
            if self.places:
                self.need_one_embedding.append(("nextn", self.places[-1]))
            return STREAMS if top_level_widened else kind
        return kind
