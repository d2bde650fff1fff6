"""`bux render`: a model's graph drawn as text.

The default drawing is a circuit of the residual stream: the stream runs left to right on
one row (the wire), a branch leaves it below and comes back at ``⊕`` (a sum) or ``⊗`` (a
product). A labelled block shows as ``┤name├`` and is drawn once more under its own name,
so a deep hybrid stays one screen wide (``expand=True`` draws everything in place)::

    model
    ──embed──┤block├×2──norm──head──

    block
    ──┬────────────⊕──┬───────────⊕──
      └─norm──attn─┘  └─norm──ffn─┘

`outline` is a second view, one layer per line with the widths, for reading sizes::

    tokens
      │ embed                                   ← 64
      ╭─ ×2 ──────────────────────────────
      │ ├─[ rmsnorm → gqa(4/2 heads) ]─⊕

Reference: ``lang/render.py:1-242`` (the drawings are the command's output; the canvas
below is this package's own).
"""

from __future__ import annotations

from . import ir


def _label(layer: ir.Layer) -> str:
    c = layer.config
    t = c.type
    if t == "gqa":
        return f"gqa({c.num_heads}/{c.num_kv_heads} heads" + (f", window {c.sliding_window_size}" if c.sliding_window_size else "") + ")"
    if t in ("mlp", "gated_mlp"):
        return f"{t}({c.intermediate_size}, {c.activation})"
    if t == "moe":
        return f"moe({c.num_experts} experts, top {c.top_k}, {c.expert.intermediate_size})"
    if t == "head":
        return "head (tied)" if c.tied else "head"
    if hasattr(c, "num_heads") and hasattr(c, "head_dim"):
        return f"{t}({c.num_heads} heads × {c.head_dim})"
    return t


def _inline(node) -> str:
    if isinstance(node, ir.Layer):
        s = _label(node)
        ports = "".join(f" {p.name}{'→@' if p.mode == 'write' else '←$'}{p.tap}" for p in node.ports)
        return s + ports
    if isinstance(node, ir.Seq):
        return " → ".join(_inline(n) for n in node.items)
    if isinstance(node, ir.Residual):
        return f"[ {_inline(node.body)} ]⊕"
    if isinstance(node, ir.Sum):
        return "(" + " + ".join(_inline(n) for n in node.terms) + ")"
    if isinstance(node, ir.Prod):
        return "(" + " * ".join(_inline(n) for n in node.factors) + ")"
    if isinstance(node, ir.Neg):
        return f"-{_inline(node.body)}"
    if isinstance(node, ir.Const):
        return f"{node.value:g}"
    if isinstance(node, ir.Identity):
        return "·"
    if isinstance(node, ir.Repeat):
        return f"({_inline(node.body)})^{node.times}"
    if isinstance(node, ir.Tap):
        return f"@{node.name}"
    if isinstance(node, ir.Ref):
        return f"${node.name}{'!' if node.pop else ''}"
    return str(node)


def _lines(node, indent: str, out: list) -> None:
    if isinstance(node, ir.Seq):
        for n in node.items:
            _lines(n, indent, out)
    elif isinstance(node, ir.Repeat):
        share = " (shared weights)" if node.body.share is not None else ""
        out.append(f"{indent}╭─ ×{node.times}{share} " + "─" * 30)
        _lines(node.body, indent + "│ ", out)
        out.append(f"{indent}╰" + "─" * 36)
    elif isinstance(node, ir.Residual):
        out.append(f"{indent}├─[ {_inline(node.body)} ]─⊕")
    elif isinstance(node, ir.Layer):
        width = node.width if node.width is not None else ""
        tail = f"← {width}" if node.config.type in ("embed", "head", "linear", "merge") and width != "" else ""
        out.append(f"{indent}│ {_inline(node):<44}{tail}".rstrip())
    else:
        out.append(f"{indent}│ {_inline(node)}")


def outline(arch: ir.Architecture) -> str:
    """One layer per line along the stream, with the widths that change."""
    out = ["tokens"]
    _lines(arch.graph, "  ", out)
    head = f"d_model {arch.d_model}, vocab {arch.vocab_size}"
    if arch.residual is not None:
        head += f", residual {arch.residual.type}"
    return head + "\n" + "\n".join(out)


# ------------------------------------------------------------------------------ the circuit
class Sheet:
    """A rectangle of characters with one row marked as the wire (where the stream
    enters on the left and leaves on the right). Rows are padded when sheets meet:
    the wire row with ``─``, every other row with spaces."""

    def __init__(self, lines, wire: int = 0):
        self.lines, self.wire = list(lines), wire

    @classmethod
    def word(cls, text: str) -> "Sheet":
        return cls([text])

    @property
    def span(self) -> int:
        return max((len(x) for x in self.lines), default=0)

    def padded(self, width: int) -> list:
        return [x + ("─" if i == self.wire else " ") * (width - len(x)) for i, x in enumerate(self.lines)]

    def shifted(self, above: int, height: int) -> list:
        """The sheet's padded lines in a column of `height` rows whose wire is row `above`."""
        body = self.padded(self.span)
        top = above - self.wire
        return [body[y - top] if 0 <= y - top < len(body) else
                ("─" if y == above else " ") * self.span for y in range(height)]


def chain(sheets, link: str = "──") -> Sheet:
    """Sheets in a row, their wires joined by `link`."""
    above = max(s.wire for s in sheets)
    height = above + max(len(s.lines) - s.wire for s in sheets)
    lines = [""] * height
    for n, sheet in enumerate(sheets):
        column = sheet.shifted(above, height)
        for y in range(height):
            gap = "" if n == 0 else (link if y == above else " " * len(link))
            lines[y] += gap + column[y]
    return Sheet(lines, above)


def fan(arms, fed, joint: str) -> Sheet:
    """`arms` one under another between a fork (left) and a merge at `joint` (right, on the
    first arm's wire). An arm whose `fed` is false starts from a tap: no line from the fork."""
    width = max(a.span for a in arms)
    lines, wires = [], []
    for arm in arms:
        wires.append(len(lines) + arm.wire)
        lines += arm.padded(width)
    taps_in = [w for w, f in zip(wires, fed) if f]

    def left(y):
        if not taps_in:
            return "  "
        if y == taps_in[0]:
            return "┬─" if len(taps_in) > 1 else "──"
        if y == taps_in[-1]:
            return "└─"
        if y in taps_in:
            return "├─"
        return "│ " if taps_in[0] < y < taps_in[-1] else "  "

    def right(y):
        if y == wires[0]:
            return "─" + joint
        if y == wires[-1]:
            return "─┘"
        if y in wires:
            return "─┤"
        return " │" if wires[0] < y < wires[-1] else "  "

    return Sheet([left(y) + x + right(y) for y, x in enumerate(lines)], wires[0])


def boxed(sheet: Sheet, caption: str) -> Sheet:
    """`sheet` inside a frame titled `caption` (an unlabelled repeat: `` ×4 ``)."""
    inner = sheet.span + 2
    lines = ["╭─" + caption + "─" * max(0, inner - len(caption) - 1) + "╮"]
    for y, x in enumerate(sheet.padded(sheet.span)):
        lines.append(("┤─" + x + "─├") if y == sheet.wire else ("│ " + x + " │"))
    lines.append("╰" + "─" * inner + "╯")
    return Sheet(lines, sheet.wire + 1)


def _reads_a_tap_first(node) -> bool:
    while True:
        if isinstance(node, ir.Ref):
            return True
        if isinstance(node, ir.Seq):
            node = node.items[0]
        elif isinstance(node, ir.Neg):
            node = node.body
        else:
            return False


class Circuit:
    """Draws nodes as sheets; remembers the labelled blocks it folded to ``┤name├``."""

    def __init__(self, fold: bool):
        self.fold = fold
        self.blocks: dict = {}    # title -> node, in the order met
        self._titles: dict = {}   # structure (labels kept) -> title

    def name_of(self, layer: ir.Layer) -> str:
        from .printer import port_to_source

        c = layer.config
        text = layer.label or (c.fn if c.type == "act" else c.type)
        if layer.ports:
            text += "(" + ", ".join(port_to_source(p) for p in layer.ports) + ")"
        return text

    def folded(self, node):
        """``┤title├`` for a labelled composite when folding, else None. Two blocks that share
        a label but not a structure get titles of their own (``name``, ``name_2``, ...)."""
        if not self.fold or node.label is None or isinstance(node, ir.Layer):
            return None
        shape = ir.strip(node, labels=False).model_dump_json()
        title = self._titles.get(shape)
        if title is None:
            title, n = node.label, 2
            while title in self.blocks:
                title, n = f"{node.label}_{n}", n + 1
            self._titles[shape] = title
            self.blocks[title] = node
        return f"┤{title}├"

    def sheet(self, node) -> Sheet:
        tag = self.folded(node)
        if tag is not None:
            return Sheet.word(tag)
        draw = getattr(self, "_" + type(node).__name__.lower())
        return draw(node)

    def _layer(self, n):
        return Sheet.word(self.name_of(n))

    def _seq(self, n):
        return chain([self.sheet(k) for k in n.items])

    def _residual(self, n):
        return fan([Sheet.word(""), self.sheet(n.body)], [True, True], "⊕")

    def _sum(self, n):
        return self._arms(n.terms, "⊕")

    def _prod(self, n):
        numbers = [f for f in n.factors if isinstance(f, ir.Const)]
        rest = [f for f in n.factors if not isinstance(f, ir.Const)]
        body = self._arms(rest, "⊗") if len(rest) > 1 else self.sheet(rest[0])
        return chain([body, *(Sheet.word(f"×{c.value:g}") for c in numbers)]) if numbers else body

    def _neg(self, n):
        return chain([Sheet.word("−"), self.sheet(n.body)], "─")

    def _const(self, n):
        return Sheet.word(f"{n.value:g}")

    def _identity(self, n):
        return Sheet.word("")

    def _repeat(self, n):
        tag = self.folded(n.body)
        if tag is not None:
            return Sheet.word(f"{tag}×{n.times}")
        if isinstance(n.body, ir.Layer):
            return Sheet.word(f"{self.name_of(n.body)}×{n.times}")
        return boxed(self.sheet(n.body), f" ×{n.times} ")

    def _tap(self, n):
        return Sheet.word(f"@{n.name}")

    def _ref(self, n):
        return Sheet.word(f"${n.name}{'!' if n.pop else ''}")

    def _arms(self, nodes, joint):
        # arms fed by the fork first, so the fork sits where the stream enters
        ordered = sorted(nodes, key=_reads_a_tap_first)
        return fan([self.sheet(k) for k in ordered], [not _reads_a_tap_first(k) for k in ordered], joint)

    def titled(self, title: str, node) -> str:
        drawn = chain([Sheet.word(""), self.sheet(node), Sheet.word("")])
        return "\n".join([title, *(x.rstrip() for x in drawn.lines)])


def render(arch: ir.Architecture, *, expand: bool = False) -> str:
    """The model's circuit, then one drawing per labelled block it uses (none with `expand`,
    which draws every block in place). Drawings are separated by blank lines; the text ends
    with a newline. This is what ``bux render`` prints."""
    circuit = Circuit(fold=not expand)
    parts = [circuit.titled(arch.graph.label or "model", arch.graph.model_copy(update={"label": None}))]
    done = 0
    while done < len(circuit.blocks):      # drawing a block can fold further blocks
        title = list(circuit.blocks)[done]
        parts.append(circuit.titled(title, circuit.blocks[title].model_copy(update={"label": None})))
        done += 1
    return "\n\n".join(parts) + "\n"
