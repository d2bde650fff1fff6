"""What the studio's page draws: the file as the compiler reads it, as plain JSON.

`view(source, filename, picks)` checks the source and, when it compiles, describes the run
the picks select: the model as a tree of drawable nodes (each with a title, the numbers that
matter as chips, the definition it comes from and the span of the source it is written at),
a card of the model's size, the training (budget, learning-rate curve with its warm-up,
stable and decay parts, curriculum, data mixture, evals, checkpoints, settings) and the
sweep (axes with their alternatives as written, the runs they make, a search's dimensions).
Spans are offsets into the buffer, so the page can select the text a node is written at and
find the node under the cursor. Reference: ``studio/view.py``, ``studio/internals.py``.
"""

from __future__ import annotations

from typing import Optional

from ..config import layers as L
from ..lang import compiler, ir
from ..lang import syntax as S
from ..lang.lsp import features
from ..lang.printer import config_to_source, value_to_source
from . import internals

TITLES = {
    "embed": "Token embedding", "head": "Output head", "rmsnorm": "RMSNorm", "layernorm": "LayerNorm", "dyt": "Dynamic tanh",
    "mlp": "Feed-forward", "gated_mlp": "Gated feed-forward", "moe": "Mixture of experts", "gqa": "Grouped-query attention",
    "mla": "Multi-head latent attention", "csa": "Compressed sparse attention", "deltanet": "DeltaNet", "gdn": "Gated DeltaNet",
    "gdn2": "Gated DeltaNet-2", "kda": "Kimi delta attention", "gla": "Gated linear attention", "lightning": "Lightning attention",
    "rwkv7": "RWKV-7", "mamba": "Mamba", "mamba2": "Mamba-2", "conv": "Convolution", "short_conv": "Short convolution",
    "linear": "Linear", "act": "Activation", "scale": "Scale", "dropout": "Dropout", "value_embed": "Value embedding",
    "nextn": "Next-token input", "engram": "N-gram memory", "doc_copy": "Document copy", "merge": "Merge streams",
}


def _short(n) -> str:
    """1536 -> "1536", 500000.0 -> "500k", 1e7 -> "10M"."""
    if isinstance(n, float) and n.is_integer():
        n = int(n)
    if isinstance(n, int) and n >= 10000:
        for unit, size in (("B", 10 ** 9), ("M", 10 ** 6), ("k", 10 ** 3)):
            if n >= size:
                v = n / size
                return (f"{v:.0f}" if v.is_integer() else f"{v:.1f}") + unit
    return str(n)


def chips(c) -> list:
    """The numbers that matter about a layer, as short labels."""
    t, out = c.type, []

    def add(text):
        out.append(text)

    if t == "gqa":
        add(f"{c.num_heads} heads")
        if c.num_kv_heads != c.num_heads:
            add(f"{c.num_kv_heads} KV heads")
        if c.head_dim:
            add(f"head {c.head_dim}")
    elif t in ("mla", "csa"):
        add(f"{c.num_heads} heads")
        if t == "mla":
            add(f"latent {c.kv_lora_rank}")
        else:
            add(f"1:{c.compress_ratio} compressed")
    elif isinstance(c, L.LinearAttentionConfig):
        add(f"{c.num_heads} heads")
        add(f"head {c.head_dim}")
    elif t in ("mlp", "gated_mlp"):
        add(f"hidden {_short(c.intermediate_size)}")
        add(c.activation)
    elif t == "moe":
        add(f"{c.num_experts} experts")
        add(f"top {c.top_k}")
        add(f"hidden {_short(c.expert.intermediate_size)}")
        if c.num_shared_experts:
            add(f"{c.num_shared_experts} shared")
    elif t in ("mamba", "mamba2"):
        add(f"state {c.state_size}")
        add(f"×{c.expand}")
    elif t == "linear":
        add(f"{_short(c.features)} features")
    elif t == "act":
        add(c.fn)
    elif t == "head":
        if c.tied:
            add("tied")
    elif t in ("conv", "short_conv"):
        add(f"{c.size if t == 'conv' else c.conv_size} taps")
    if getattr(c, "sliding_window_size", None):
        add(f"window {_short(c.sliding_window_size)}")
    rope = getattr(c, "rope", None)
    if rope is not None:
        add(f"RoPE {_short(rope.base)}")
    if getattr(c, "indexer", None) is not None:
        add(f"sparse top {c.indexer.top_k}")
    for flag in ("qk_norm", "sinks", "gated", "softcap"):
        v = getattr(c, flag, None)
        if v not in (None, False):
            add(flag.replace("_", " ") + ("" if v is True or isinstance(v, L.Config) else f" {v:g}"))
    return out


class Drawing:
    """Turns an architecture's graph into the page's tree, numbering nodes in walk order."""

    def __init__(self, spans: dict, base: int, limit: int, d_model: int = 0):
        self.spans, self.base, self.limit, self.d_model = spans, base, limit, d_model
        self.count = 0

    def span(self, node) -> Optional[list]:
        s = self.spans.get(id(node))
        if s is None or s.start < self.base or s.end > self.limit:
            return None       # written in a module, or made by the compiler
        return [s.start - self.base, s.end - self.base]

    def node(self, n) -> dict:
        self.count += 1
        out = {"id": self.count, "kind": type(n).__name__.lower(), "span": self.span(n)}
        if getattr(n, "label", None):
            out["name"] = n.label
        if isinstance(n, ir.Layer):
            c = n.config
            out.update(type=c.type, title=TITLES.get(c.type, c.type), chips=chips(c), source=config_to_source(c),
                       ports=[{"name": p.name, "mode": p.mode, "tap": p.tap} for p in n.ports],
                       opens=c.type in internals.BUILDERS)
            if out["opens"]:
                out["inside"] = internals.inside(c, n.width if isinstance(n.width, int) else self.d_model)
            if getattr(n, "share", None):
                out["shared"] = n.share
        elif isinstance(n, ir.Seq):
            out["items"] = [self.node(k) for k in n.items]
        elif isinstance(n, ir.Residual):
            out["body"] = self.node(n.body)
        elif isinstance(n, ir.Sum):
            out["terms"] = [self.node(k) for k in n.terms]
        elif isinstance(n, ir.Prod):
            out["factors"] = [self.node(k) for k in n.factors]
        elif isinstance(n, ir.Neg):
            out["body"] = self.node(n.body)
        elif isinstance(n, ir.Const):
            out["value"] = n.value
        elif isinstance(n, ir.Repeat):
            out.update(times=n.times, body=self.node(n.body))
        elif isinstance(n, ir.Tap):
            out["tap"] = n.name
        elif isinstance(n, ir.Ref):
            out.update(tap=n.name, pop=n.pop)
        return out


def card(arch: ir.Architecture) -> dict:
    from collections import Counter

    layers = list(ir.unrolled_layers(arch.graph))
    kinds = Counter(l.config.type for l in layers)
    out = {"d_model": arch.d_model, "vocab_size": arch.vocab_size, "layers": len(layers),
           "by_type": sorted(kinds.items(), key=lambda kv: -kv[1]),
           "residual": arch.residual.type if arch.residual is not None else None}
    try:
        from ..train.trainer import count_params

        out["params"] = count_params(arch)
    except Exception:  # noqa: BLE001 - the count needs torch; the page shows the rest without it
        out["params"] = None
    return out


def schedule_points(train, points: int = 200) -> dict:
    """The learning rate over the steps (as a share of the peak), with where the warm-up ends
    and the decay starts."""
    from ..train import optim

    steps = train.steps
    xs = sorted({min(steps - 1, round(i * (steps - 1) / max(1, points - 1))) for i in range(points)}) if steps > 1 else [0]
    scale = optim.lr_multiplier(train)
    ys = [float(scale(x)) for x in xs]
    sch = train.schedule
    warm = getattr(sch, "warmup", 0) or 0
    warm = round(warm * steps) if isinstance(warm, float) and warm < 1 else int(warm)
    decay = getattr(sch, "decay", None)
    decay_from = None
    if decay is not None and sch.type in ("wsd", "power"):
        decay_from = steps - (round(decay * steps) if decay < 1 else int(decay))
    return {"type": sch.type, "steps": xs, "scale": ys, "peak": train.optimizer.lr, "warmup_end": warm, "decay_start": decay_from}


def training(train) -> dict:
    from ..config import training as T

    tokens = train.steps * train.batch * train.seq_len
    out = {"steps": train.steps, "batch": train.batch, "seq_len": train.seq_len, "tokens": tokens,
           "optimizer": config_to_source(train.optimizer), "schedule": schedule_points(train)}
    data = train.data
    if isinstance(data, T.MixtureConfig):
        total = sum(w.weight for w in data.sources) or 1.0
        out["data"] = [{"name": getattr(w, "name", None) or config_to_source(w.source), "weight": w.weight / total}
                       for w in data.sources]
    else:
        out["data"] = [{"name": config_to_source(data), "weight": 1.0}]
    out["evals"] = [{"name": e.name, "every": e.every} for e in T.evals(train)]
    out["checkpoint"] = None if train.checkpoint is None else {"every": train.checkpoint.every, "keep": train.checkpoint.keep}
    out["curriculum"] = [{"at": ph.at, "seq_len": ph.seq_len, "batch": ph.batch} for ph in (train.curriculum or ())]
    out["settings"] = {}
    for name, f in T.TrainConfig.model_fields.items():
        v = getattr(train, name)
        if not f.is_required() and v == f.get_default(call_default_factory=True):
            continue
        try:
            out["settings"][name] = value_to_source(v)
        except Exception:  # noqa: BLE001
            out["settings"][name] = str(v)
    return out


def alternations(program) -> list:
    """Every ``a | b`` of the program's statements, as the parser read it."""
    found = []

    def walk(e):
        if isinstance(e, S.Alt):
            found.append(e)
        for name in ("items", "options"):
            for k in getattr(e, name, ()) or ():
                walk(k)
        for name in ("body", "operand", "left", "right", "base", "value"):
            k = getattr(e, name, None)
            if isinstance(k, (S.Expr, S.Arg)):
                walk(k)
        for a in getattr(e, "args", ()) or ():
            walk(a.value)

    for layer in program.layers:
        for st in layer:
            if st.body is not None:
                walk(st.body)
    return found


def sweep(found: list, program, base: int, limit: int) -> dict:
    """The axes as written (each alternative with the span it is written at, so the page can
    edit one and leave the others' lines alone), the runs they make, a search's dimensions."""
    written = alternations(program)
    axes = []
    for a in (found[0].axes if found else ()):
        if a.labeled:
            mine = [w for w in written if w.labels and set(w.labels) == set(a.key)]
        else:
            mine = [w for w in written if w.span == a.span]
        places = []
        for w in mine:
            options = []
            for i, opt in enumerate(w.options):
                inside = base <= opt.span.start and opt.span.end <= limit
                options.append({"text": " ".join(program.source[opt.span.start:opt.span.end].split()),
                                "label": w.labels[i] if w.labels else None,
                                "span": [opt.span.start - base, opt.span.end - base] if inside else None})
            places.append({"where": w.where, "options": options})
        axes.append({"where": a.where, "labeled": a.labeled, "count": len(a.options), "places": places})
    dims = [{"where": d.where, "space": config_to_source(d.space)} for d in (found[0].dims if found else ())]
    return {"axes": axes, "dimensions": dims, "runs": len(found)}


def view(source: str, filename: str = "<buffer>", picks: Optional[dict] = None, run: int = 0) -> dict:
    """Everything the page shows for `source`; `run` picks one run of a sweep."""
    errors = [{"start": d.start, "end": d.end, "message": d.message} for d in features.diagnostics(source, filename)]
    out = {"errors": errors, "model": None, "card": None, "training": None, "sweep": None, "runs": []}
    if errors:
        return out
    try:
        program = compiler._load(source, filename, (), None, recover=False)
        found = compiler._useful(compiler.explore(program, "model", require=False))
    except S.BuxError as err:
        out["errors"] = [{"start": err.span.start if err.span else 0, "end": err.span.end if err.span else 1, "message": err.message}]
        return out
    if not found:
        return out
    main = next((f for f in program.files if f.filename == filename), program.files[0])
    run = max(0, min(run, len(found) - 1))
    chosen = found[run]
    # spans of the chosen run's nodes: evaluate it once more, keeping the evaluator
    ev, arch, train = compiler._evaluate(program, "model", chosen.choices, None, require=False)
    drawing = Drawing(ev.node_spans, main.start, main.stop, arch.d_model)
    out["model"] = drawing.node(arch.graph)
    out["card"] = card(arch)
    out["training"] = training(train) if train is not None else None
    out["sweep"] = sweep(found, program, main.start, main.stop)
    for i, f in enumerate(found[:256]):
        name = compiler._run_name(filename, tuple(a.part(f.choices[a.key]) for a in f.axes if a.key in f.choices)) \
            if f.train is not None else f"model {i}"
        out["runs"].append({"index": i, "name": name})
    out["run"] = run
    return out
