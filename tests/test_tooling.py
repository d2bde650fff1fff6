"""render, reference pages, language-server features and the stdio server."""
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


def test_features():
    src = "d_model = 64\nvocab_size = 32\nattn = gqa(num_heads=4, num_kv_heads=2)\nmodel = embed [rmsnorm attn] rmsnorm head\noptimizer = adamw(lr=1e-3)\ndata = synthetic\nseq_len = 8\nbatch = 2\nsteps = 1\n"
    assert features.diagnostics(src) == []
    bad = src.replace("num_heads=4", "num_heads=3")
    diags = features.diagnostics(bad)
    assert diags and diags[0]["range"]["start"]["line"] == 2
    assert "num_heads" in features.hover(src, 2, 8)                     # on `gqa`
    assert "line 3" in features.hover(src, 3, 24)                       # on the use of `attn`
    assert features.definition(src, 3, 24)["start"] == {"line": 2, "character": 0}
    labels = [c["label"] for c in features.completion(src[:src.index("num_kv")], 2, len("attn = gqa(num_heads=4, "))]
    assert "num_kv_heads" in labels and "sliding_window_size" in labels
    tops = [c["label"] for c in features.completion("model = em", 0, 10)]
    assert "embed" in tops and all(t.startswith("em") for t in tops)


def _frame(msg):
    body = json.dumps({"jsonrpc": "2.0", **msg}).encode()
    return f"Content-Length: {len(body)}\r\n\r\n".encode() + body


def test_server_over_stdio():
    uri = "file:///x.bux"
    inp = io.BytesIO(b"".join(_frame(m) for m in [
        {"id": 1, "method": "initialize", "params": {}},
        {"method": "textDocument/didOpen", "params": {"textDocument": {"uri": uri, "text": "model = embed head\nd_model = 8\n"}}},
        {"id": 2, "method": "textDocument/hover", "params": {"textDocument": {"uri": uri}, "position": {"line": 0, "character": 9}}},
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
    assert next(m for m in msgs if m.get("id") == 2)["result"]["contents"]["value"].startswith("embed")


def test_studio_api(tmp_path):
    import threading
    import urllib.request
    from http.server import ThreadingHTTPServer

    from bux_b200.studio import Studio
    from bux_b200.studio.server import set_value

    assert set_value("a = 1\nb = f(\n  x)\nc = 2\n", "b", "g()") == "a = 1\nb = g()\nc = 2\n"
    assert set_value("a = 1\n", "steps", "9").endswith("steps = 9\n")
    f = tmp_path / "s.bux"
    f.write_text(SMOKE)
    studio = Studio(f, out=tmp_path / "runs")
    server = ThreadingHTTPServer(("127.0.0.1", 0), studio.handler())
    port = server.server_address[1]
    threading.Thread(target=server.serve_forever, daemon=True).start()
    try:
        def call(path, body=None, token=studio.token):
            req = urllib.request.Request(f"http://127.0.0.1:{port}{path}?token={token}",
                                         data=None if body is None else json.dumps(body).encode())
            with urllib.request.urlopen(req) as r:
                return json.loads(r.read())

        view = call("/api/view")
        assert view["runs"][0]["id"] == "5a4f0f7d85" and view["runs"][0]["params"] == 155968 and "×2" in view["graph"]
        edited = call("/api/set", {"name": "steps", "value": "20"})
        assert not edited["diagnostics"] and "steps = 20" in f.read_text().replace("    ", " ").replace("  ", " ")
        broken = call("/api/source", {"source": SMOKE.replace("num_heads=4", "num_heads=3")})
        assert broken["diagnostics"] and "num_heads=3" not in f.read_text()   # the file keeps its last good text
        try:
            call("/api/view", token="nope")
            raise AssertionError("a bad token must be refused")
        except urllib.error.HTTPError as e:
            assert e.code == 403
    finally:
        server.shutdown()


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
