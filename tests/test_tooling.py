"""render, reference pages, language-server features, the stdio server, trackers (the studio: test_studio.py)."""
import io
import json
from pathlib import Path

from bux_b200.lang import compile_runs, reference
from bux_b200.lang.lsp import Server, features
from bux_b200.lang.render import outline, render

SMOKE = (Path(__file__).resolve().parent.parent / "examples" / "experiments" / "smoke.bux").read_text()


def test_outline_shows_the_repeat_and_branches():
    text = outline(compile_runs(SMOKE, filename="smoke.bux")[0].arch)
    assert "×2" in text and "gqa(4/2 heads)" in text and "⊕" in text and "head (tied)" in text


_DEFS = """d_model = 64
vocab_size = 32
norm = rmsnorm
attn = gqa(num_heads=4, num_kv_heads=2)
ffn = gated_mlp(intermediate_size=128, activation=swish)
head = head
"""


def _arch(text):
    from bux_b200.lang import compile

    return compile(_DEFS + text, filename="r.bux")


def test_render_draws_residual_branches_under_the_stream():
    arch = _arch("block = [norm attn] [norm (attn + ffn)]\nmodel = embed block^2 norm head\n")
    assert render(arch) == (
        "model\n"
        "──embed──┤block├×2──norm──head──\n"
        "\n"
        "block\n"
        "──┬────────────⊕──┬────────────────⊕──\n"
        "  └─norm──attn─┘  └─norm──┬─attn─⊕─┘\n"
        "                          └─ffn──┘\n"
    )
    wide = render(arch, expand=True)
    assert "┤block├" not in wide and "×2" in wide and wide.count("\n\n") == 0


def test_render_products_taps_and_blocks_of_one_label():
    gate = _arch("swiglu = (linear(features=128) swish * linear(features=128)) linear(features=d_model)\n"
                 "model = embed [norm swiglu] head\n")
    assert ("swiglu\n"
            "──┬─linear──swish─⊗──linear──\n"
            "  └─linear────────┘\n") in render(gate)
    two = render(_arch("inner(f) = [norm f]\nouter(g) = inner(g) scale\nmodel = embed outer(attn) outer(ffn) head\n"))
    assert "┤inner(g)_2├" in two and "norm──ffn" in two
    taps = render(_arch("a = gqa(num_heads=4, num_kv_heads=4)\nmodel = embed [a(v=@v)] [a(v=$v!)] head\n"))
    assert "a(v=$v!)" in taps and "a(v=@v)" in taps
    scaled = render(_arch("model = embed (_ * 2.0 + attn) @skip [ffn] [$skip! scale] head\n"))
    assert "×2" in scaled and "@skip" in scaled and "$skip!" in scaled


def test_render_every_example_architecture():
    root = Path(__file__).resolve().parent.parent / "examples" / "architectures"
    from bux_b200.lang import compile

    for path in sorted(root.glob("*.bux")):
        arch = compile(path.read_text(), filename=str(path))
        assert render(arch).endswith("\n") and render(arch, expand=True)


def test_reference_lists_every_layer_and_setting():
    text = reference.reference()
    for name in ("gqa", "moe", "kda", "mamba2", "adamw", "checkpoint", "mesh"):
        assert f"`{name}`" in text


_SRC = """d_model = 64
vocab_size = 32
norm = rmsnorm
attn = gqa(num_heads=4, num_kv_heads=2, rope=rope(base=500000.0))
local = attn(sliding_window_size=128)
ffn = gated_mlp(intermediate_size=128, activation=swish)
layer(mixer) = [norm mixer] [norm ffn]
L = layer(local)
G = layer(attn(v=@v))
model = embed @h "LG"^2 [$h! scale] norm head
optimizer = adamw(lr=1e-3)
data = synthetic
seq_len = 8
batch = 2
steps = 1
"""


def _at(src, needle, inside=0):
    return src.index(needle) + inside


def _labels(src, offset, path=None):
    return [c.label for c in features.complete(src, offset, path)]


def test_diagnostics_report_every_mistake_at_its_place(tmp_path):
    assert features.diagnostics(_SRC) == []
    bad = _SRC.replace("num_heads=4", "num_heads=3").replace("activation=swish", "activation=swosh")
    found = features.diagnostics(bad)
    assert len(found) >= 2 and all(bad.count("\n", 0, d.start) in (3, 5) for d in found[:2])
    # a mistake inside a module shows at the `use` that brought the module in
    (tmp_path / "blocks.bux").write_text("attn = gqa(num_heads=3, num_kv_heads=2)\n")
    main = "use blocks\n" + _SRC.replace("attn = gqa(num_heads=4, num_kv_heads=2, rope=rope(base=500000.0))\n", "")
    (d,) = [d for d in features.diagnostics(main, str(tmp_path / "main.bux")) if "blocks.bux" in d.message]
    assert main[d.start:d.end] == "blocks" and "blocks.bux:1" in d.message


def test_hover_says_what_a_name_is():
    def text(needle, inside=0, src=_SRC):
        h = features.hover(src, _at(src, needle, inside))
        return h.text if h else None

    gqa = text("gqa(")
    assert gqa.startswith("**gqa** — layer") and "`num_kv_heads: int" in gqa and "Key/value heads" in gqa
    assert "`base: float = 10000.0`" in text("base=") and "Theta" in text("base=")       # a dotted class's field
    assert "sliding_window_size" in text("sliding_window_size=128") and "most recent keys" in text("sliding_window_size=128")
    use = text("local)")                                         # a use of a definition
    assert "local = attn(sliding_window_size=128)" in use and "evaluates to `gqa(" in use and "a `gqa`" in use
    assert "macro of `mixer`" in text("layer(local)")
    assert text("mixer]") == "parameter `mixer` of the macro `layer`"
    assert "**swish** — activation" in text("swish")
    assert text("steps = 1").startswith("**steps** — training setting") and "here: `1`" in text("steps = 1")
    tap = text("@h", 1)
    assert "written (the stream pushed) on line 10" in tap and "popped on line 10" in tap
    assert "written by a layer's port on line 9" in text("@v", 1)
    assert "port `v`" in text("v=@v")
    bare = text("softmax", src=_SRC.replace("model =", "e = moe(num_experts=4, top_k=1, expert=ffn, router=softmax)\nmodel ="))
    assert "an option of `router`" in bare
    name = text("mything", src=_SRC.replace("data = synthetic", "data = text(path=mything)"))
    assert "is not defined" in name and "string" in name


def test_hover_names_the_module_a_definition_comes_from(tmp_path):
    (tmp_path / "blocks.bux").write_text("# shared blocks\nmynorm = rmsnorm(eps=1e-5)\n")
    main = "use blocks\n" + _SRC.replace("norm = rmsnorm\n", "norm = mynorm\n")
    h = features.hover(main, _at(main, "mynorm"), str(tmp_path / "main.bux"))
    assert "mynorm = rmsnorm(eps=1e-5)" in h.text and "blocks.bux`, line 2" in h.text
    file, start, end = features.definition(main, _at(main, "mynorm"), str(tmp_path / "main.bux"))
    assert file.endswith("blocks.bux") and (tmp_path / "blocks.bux").read_text()[start:end] == "mynorm"


def test_definition_goes_to_the_name():
    file, start, end = features.definition(_SRC, _at(_SRC, "local)"))
    assert _SRC[start:end] == "local" and _SRC[:start].endswith("\n") and _SRC[end:].startswith(" = attn")
    _, start, end = features.definition(_SRC, _at(_SRC, "$h!", 1))
    assert _SRC[start:end] == "@h"


def test_completion_offers_what_fits():
    # settings of the layer being called, through definitions, without those already given
    src = _SRC.replace("local = attn(sliding_window_size=128)", "local = attn(sliding_window_size=128, ")
    got = _labels(src, _at(src, "sliding_window_size=128, ") + len("sliding_window_size=128, "))
    assert "num_kv_heads" in got and "softcap" in got and "sliding_window_size" not in got and "v" in got
    # dotted keys
    src = _SRC.replace("rope=rope(base=500000.0)", "rope.")
    got = _labels(src, _at(src, "rope.") + 5)
    assert {"base", "fraction", "scaling"} <= set(got) and "num_heads" not in got
    # values a setting's type allows
    src = _SRC.replace("activation=swish", "activation=")
    assert {"swish", "gelu", "relu2"} <= set(_labels(src, _at(src, "activation=") + len("activation=")))
    src = _SRC.replace("num_kv_heads=2,", "num_kv_heads=2, qk_norm=,")
    got = _labels(src, _at(src, "qk_norm=") + len("qk_norm="))
    assert got[0] == "norm" or "norm" in got[:3]
    assert {"rmsnorm", "layernorm", "norm", "none"} <= set(got) and "gqa" not in got
    src = _SRC.replace("model =", "e = moe(num_experts=4, top_k=1, expert=ffn, router=)\nmodel =")
    assert set(_labels(src, _at(src, "router=") + 7)) == {"softmax", "sigmoid", "sqrtsoftplus"}
    # macro parameters
    src = _SRC.replace("L = layer(local)", "L = layer(")
    assert _labels(src, _at(src, "L = layer(") + len("L = layer("))[0] == "mixer"
    # fields after `name.`, with their current values
    src = _SRC + "attn."
    items = features.complete(src, len(src))
    heads = next(c for c in items if c.label == "num_heads")
    assert heads.detail == "= 4" and heads.insert == "num_heads"
    # tap names after @ and $
    src = _SRC.replace("[$h! scale]", "[$ scale]")
    assert _labels(src, _at(src, "[$ scale]") + 2) == ["h", "v"]
    # one-letter definitions inside patterns
    src = _SRC.replace('"LG"^2', '"L"^2')
    assert _labels(src, _at(src, '"L"') + 2) == ["G", "L"]
    # expressions: definitions first, then builtins, filtered by what is typed
    src = _SRC.replace("model = embed", "model = em")
    assert _labels(src, _at(src, "model = em") + len("model = em")) == ["embed"]
    src = _SRC + "sch"
    assert _labels(src, len(src)) == ["schedule"]
    src = _SRC + "schedule = "
    assert {"wsd", "cosine", "constant"} <= set(_labels(src, len(src)))


def _frame(msg):
    body = json.dumps({"jsonrpc": "2.0", **msg}).encode()
    return f"Content-Length: {len(body)}\r\n\r\n".encode() + body


def test_server_over_stdio():
    uri = "file:///x.bux"
    inp = io.BytesIO(b"".join(_frame(m) for m in [
        {"id": 1, "method": "initialize", "params": {}},
        {"method": "textDocument/didOpen", "params": {"textDocument": {"uri": uri, "text": "model = embed head\nd_model = 8\n"}}},
        {"id": 2, "method": "textDocument/hover", "params": {"textDocument": {"uri": uri}, "position": {"line": 0, "character": 9}}},
        {"method": "textDocument/didChange", "params": {"textDocument": {"uri": uri}, "contentChanges": [{"text": "model = embed he\nd_model = 8\n"}]}},
        {"id": 4, "method": "textDocument/completion", "params": {"textDocument": {"uri": uri}, "position": {"line": 0, "character": 16}}},
        {"id": 3, "method": "shutdown"}, {"method": "exit"}]))
    out = io.BytesIO()
    Server(inp, out).serve()
    raw = out.getvalue()
    msgs = []
    while raw:
        head, _, rest = raw.partition(b"\r\n\r\n")
        n = int(head.split(b":")[1])
        msgs.append(json.loads(rest[:n]))
        raw = rest[n:]
    assert msgs[0]["result"]["capabilities"]["hoverProvider"]
    diag = next(m for m in msgs if m.get("method") == "textDocument/publishDiagnostics")
    assert diag["params"]["diagnostics"]  # the file has no vocab_size / optimizer ...
    hover = next(m for m in msgs if m.get("id") == 2)["result"]
    assert hover["contents"]["value"].startswith("**embed** — layer") and hover["range"]["start"] == {"line": 0, "character": 8}
    items = next(m for m in msgs if m.get("id") == 4)["result"]["items"]
    assert [i["label"] for i in items] == ["head"] and items[0]["kind"] == 7


def test_trackers_forward_every_logged_step_to_their_package(tmp_path, monkeypatch):
    """W&B and TensorBoard sinks against stand-ins for the packages (neither is installed here):
    a W&B run resumes under the id kept in the run's folder; TensorBoard writes scalars only."""
    import sys
    import types

    from bux_b200.config import training as T
    from bux_b200.lang import compile_runs
    from bux_b200.train import trackers

    calls = {"init": [], "log": [], "scalars": [], "closed": 0}
    wandb = types.ModuleType("wandb")
    wandb.util = types.SimpleNamespace(generate_id=lambda: "abc123")

    class _Run:
        def log(self, values, step):
            calls["log"].append((step, dict(values)))

        def finish(self):
            calls["closed"] += 1

    def init(**kw):
        calls["init"].append(kw)
        return _Run()

    wandb.init = init
    monkeypatch.setitem(sys.modules, "wandb", wandb)
    tb = types.ModuleType("torch.utils.tensorboard")

    class SummaryWriter:
        def __init__(self, folder):
            calls["tb_folder"] = folder

        def add_scalar(self, name, value, step):
            calls["scalars"].append((name, value, step))

        def close(self):
            calls["closed"] += 1

    tb.SummaryWriter = SummaryWriter
    monkeypatch.setitem(sys.modules, "torch.utils.tensorboard", tb)
    run = compile_runs(SMOKE, filename="smoke.bux")[0]
    configs = [T.WandbConfig(project="p", tags=("a",)), T.TensorBoardConfig()]
    sinks = trackers.build(configs, tmp_path, run)
    for s in sinks:
        s.write(3, {"loss": 1.5, "note": "text"})
        s.close()
    assert calls["init"][0]["id"] == "abc123" and calls["init"][0]["resume"] == "allow" and calls["init"][0]["project"] == "p"
    assert (tmp_path / "wandb_id").read_text() == "abc123"
    assert calls["log"] == [(3, {"loss": 1.5, "note": "text"})]
    assert calls["scalars"] == [("loss", 1.5, 3)] and calls["tb_folder"].endswith("tensorboard") and calls["closed"] == 2
    # a second start of the same run takes the id on file
    wandb.util = types.SimpleNamespace(generate_id=lambda: "other")
    trackers.build(configs[:1], tmp_path, run)
    assert calls["init"][1]["id"] == "abc123"


def test_the_textmate_grammar_lists_every_builtin_and_matches_a_file():
    import re

    from bux_b200.lang.lsp.editors.__main__ import names

    folder = Path(__file__).resolve().parent.parent / "bux_b200" / "lang" / "lsp" / "editors"
    grammar = json.loads((folder / "bux.tmLanguage.json").read_text())
    builtin = next(r for r in grammar["repository"]["expression"]["patterns"] if r.get("name") == "support.function.builtin.bux")
    listed = set(builtin["match"][len("\\b("):-len(")\\b")].split("|"))
    assert listed == set(names()[0])                       # regenerate after adding a layer
    setting, define = (re.compile(r["match"], re.M) for r in grammar["repository"]["definition"]["patterns"])
    assert [m.group(2) for m in setting.finditer(_SRC)][:2] == ["d_model", "vocab_size"]
    assert "layer" in [m.group(2) for m in define.finditer(_SRC)]
    tap = next(r for r in grammar["repository"]["expression"]["patterns"] if r.get("name") == "variable.other.tap.bux")
    assert re.findall(tap["match"], _SRC) == ["@v", "@h", "$h!"]
    assert json.loads((folder / "template.json").read_text())["programArgs"]["default"] == "bux-lsp"


def test_check_prints_the_summary_of_a_run_a_sweep_and_a_module(tmp_path, capsys):
    from bux_b200.__main__ import main

    smoke = str(Path(__file__).resolve().parent.parent / "examples" / "experiments" / "smoke.bux")
    assert main(["check", smoke, "optimizer.lr = 1e-3 | 3e-3"]) == 0
    assert capsys.readouterr().out.splitlines() == [
        "d_model=64 vocab_size=512 layers=11",
        "rmsnorm×5  gqa×2  gated_mlp×2  embed×1  head×1",
        "50 steps × 8 × 64 tokens = 25.6k tokens",
        "optimizer=adamw(lr=0.001) schedule=wsd(warmup=10)",
        "data=synthetic()",
        "sweep: 2 runs over optimizer.lr (1e-3 | 3e-3)"]
    recipe = tmp_path / "recipe.bux"
    recipe.write_text("optimizer = adamw(lr=1e-3)\nschedule = wsd(warmup=10)\nbudget = 100\nsteps = budget\n")
    assert main(["check", str(recipe)]) == 0
    assert capsys.readouterr().out.strip() == "a module: it defines optimizer, schedule, budget, steps, and no model"
    recipe.write_text("optimizer = adamw(lr=1e-3, weight_dacay=0.1)\n")      # a module's definitions are still checked
    assert main(["check", str(recipe)]) == 1
    assert "did you mean 'weight_decay'" in capsys.readouterr().err
    assert features.diagnostics("optimizer = adamw(lr=1e-3)\nsteps = 10\n") == []     # the editor takes a module too
