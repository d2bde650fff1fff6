"""The studio's Python side: the view of a file, the inspector, the palette, structural
edits as text splices, and the HTTP API (saving, conflicts, tokens)."""
import json
import threading
import urllib.error
import urllib.request
from pathlib import Path

import pytest

from bux_b200.lang import compile_runs
from bux_b200.studio import edits, forms, palette, view

SRC = """# a small run
d_model = 64
vocab_size = 512
norm = rmsnorm
attn = gqa(num_heads=4, num_kv_heads=2, rope=rope(base=10000.0))   # the mixer
ffn = gated_mlp(intermediate_size=128, activation=swish)
layer(mixer) = [norm mixer] [norm ffn]
block = layer(attn)
model = embed block^2 norm head(tied=true)
data = synthetic
optimizer = adamw(lr=3e-3 | 1e-3)
schedule = wsd(warmup=10)
seq_len = 64
batch = 8
steps = 50
"""


def _span(src, text, nth=0):
    at = -1
    for _ in range(nth + 1):
        at = src.index(text, at + 1)
    return at, at + len(text)


def _ok(src):
    return compile_runs(src, filename="s.bux")


def test_view_describes_the_run_the_picks_select():
    v = view.view(SRC, "s.bux")
    assert v["errors"] == [] and v["card"]["layers"] == 11 and v["card"]["params"] > 0
    model = v["model"]
    assert model["kind"] == "seq" and [k["kind"] for k in model["items"]] == ["layer", "repeat", "layer", "layer"]
    repeat = model["items"][1]
    assert repeat["times"] == 2 and SRC[slice(*repeat["span"])] == "block^2" and repeat["body"]["name"] == "block"
    attn = repeat["body"]["items"][0]["body"]["items"][1]
    assert attn["title"] == "Grouped-query attention" and attn["chips"][:2] == ["4 heads", "2 KV heads"] and "RoPE 10k" in attn["chips"]
    assert SRC[slice(*attn["span"])] == "mixer"            # where the macro writes it
    inside = attn["inside"]                                 # what the layer opens into
    assert inside["kind"] == "seq" and inside["items"][0]["kind"] == "prod" and len(inside["items"][0]["factors"]) == 3
    assert any(i.get("title") == "Softmax attention" for i in inside["items"]) and "64 → 4 × 16" in json.dumps(inside, ensure_ascii=False)
    ffn = repeat["body"]["items"][1]["body"]["items"][1]
    assert ffn["inside"]["items"][0]["kind"] == "prod" and ffn["inside"]["items"][-1]["title"] == "Down projection"
    t = v["training"]
    assert t["tokens"] == 50 * 8 * 64 and t["schedule"]["warmup_end"] == 10 and t["schedule"]["decay_start"] == 40
    assert max(t["schedule"]["scale"]) == 1.0 and t["schedule"]["scale"][-1] < 0.05
    (axis,) = v["sweep"]["axes"]
    assert [o["text"] for o in axis["places"][0]["options"]] == ["3e-3", "1e-3"] and v["sweep"]["runs"] == 2
    assert SRC[slice(*axis["places"][0]["options"][1]["span"])] == "1e-3"
    assert len(v["runs"]) == 2 and view.view(SRC, "s.bux", run=1)["training"]["optimizer"] == "adamw(lr=0.001)"
    bad = view.view(SRC.replace("num_heads=4", "num_heads=3"), "s.bux")
    assert bad["model"] is None and bad["errors"][0]["start"] > 0


def test_inspector_lists_fields_and_says_why_one_cannot_be_set():
    got = forms.inspect(SRC, *_span(SRC, "attn", 1), "s.bux")       # `attn` inside layer(attn)
    assert got["type"] == "gqa" and got["why"] is None
    by = {f["name"]: f for f in got["fields"]}
    assert by["num_heads"]["value"] == "4" and by["num_heads"]["written"] and by["num_heads"]["kind"] == "int"
    assert by["softcap"]["written"] is False and by["softcap"]["kind"] == "float" and by["softcap"]["optional"]
    assert by["rope"]["kind"] == "config" and "rope" in by["rope"]["types"] and "Rotary" in by["rope"]["note"]
    assert by["value_residual"]["kind"] == "choice" and "learned" in by["value_residual"]["options"]
    macro = forms.inspect(SRC, *_span(SRC, "mixer", 2), "s.bux")     # the parameter inside the macro's body
    assert "parameter of the macro 'layer'" in macro["why"]
    block = forms.inspect(SRC, *_span(SRC, "block", 1), "s.bux")
    assert block["fields"] == [] and "block" in block["why"]


def test_palette_offers_insertable_text():
    groups = {g["group"]: g["items"] for g in palette.palette(SRC, "s.bux")}
    assert {"attn", "ffn", "norm", "block"} <= {i["name"] for i in groups["This file"]}
    for group, items in groups.items():
        for item in ([] if group == "This file" else items):
            if item["name"] in ("embed", "head", "nextn", "value_embed", "engram", "doc_copy"):
                continue
            src = SRC.replace("[norm ffn]", f"[norm ffn] [norm {item['insert']}]") if item["name"] not in ("csa",) else SRC
            assert _ok(src), item


def test_edits_are_splices_that_keep_the_rest_of_the_file():
    # a field where it is written, through the macro call's argument
    s, e = _span(SRC, "attn", 1)
    out = edits.set_field(SRC, s, e, "num_kv_heads", "4", "s.bux")
    assert "num_kv_heads=4, rope=rope(base=10000.0))   # the mixer" in out and out.count("\n") == SRC.count("\n") and _ok(out)
    out = edits.set_field(SRC, s, e, "softcap", "30.0", "s.bux")             # added
    assert "rope=rope(base=10000.0), softcap=30.0)   # the mixer" in out and _ok(out)
    out = edits.set_field(out, *_span(out, "attn", 1), "softcap", None, "s.bux")   # and removed again
    assert out == SRC
    out = edits.set_field(SRC, s, e, "rope.base", "500000.0", "s.bux")        # a dotted key, inside rope(...)
    assert "rope=rope(base=500000.0)" in out and _ok(out)
    out = edits.set_field(SRC, *_span(SRC, "norm", 2), "eps", "1e-5", "s.bux")  # ``norm = rmsnorm`` gets its call
    assert "norm = rmsnorm(eps=1e-5)\n" in out and _ok(out)
    with pytest.raises(edits.EditError, match="parameter of the macro"):
        edits.set_field(SRC, *_span(SRC, "mixer", 2), "num_heads", "8", "s.bux")
    # top-level settings, with CRLF kept
    assert "steps = 100\n" in edits.set_setting(SRC, "steps", "100") and "clip = 0.5\n" in edits.set_setting(SRC, "clip", "0.5")
    crlf = SRC.replace("\n", "\r\n")
    assert "steps = 7\r\n" in edits.set_setting(crlf, "steps", "7") and "\n\n" not in edits.set_setting(crlf, "steps", "7")
    # the graph's shape
    s, e = _span(SRC, "[norm ffn]")
    out = edits.insert(SRC, s, e, "[norm gated_mlp(intermediate_size=32, activation=gelu)]", True, "s.bux")
    assert "[norm ffn] [norm gated_mlp(intermediate_size=32, activation=gelu)]" in out and len(_ok(out)) == 2
    assert "[norm mixer]\n" in edits.delete(SRC, s, e, "s.bux") + "\n" or "[norm mixer]" in edits.delete(SRC, s, e, "s.bux")
    s, e = _span(SRC, "norm", 4)                                              # the final norm of the model
    wrapped = edits.wrap(SRC, s, e, "s.bux")
    assert "block^2 [norm] head" in wrapped and edits.unwrap(wrapped, s, e + 2, "s.bux") == SRC
    assert "block^6 norm" in edits.set_repeat(SRC, *_span(SRC, "block^2"), 6, "s.bux")
    assert "embed^3 block" in edits.set_repeat(SRC, *_span(SRC, "embed", 0), 3, "s.bux")
    # a sweep's alternatives
    s, e = _span(SRC, "1e-3")
    assert "lr=3e-3 | 2e-3)" in edits.alt_replace(SRC, s, e, "2e-3")
    assert "lr=3e-3 | 1e-3 | 3e-4)" in edits.alt_add(SRC, s, e, "3e-4") and len(_ok(edits.alt_add(SRC, s, e, "3e-4"))) == 3
    assert "lr=3e-3)" in edits.alt_remove(SRC, s, e) and "lr=1e-3)" in edits.alt_remove(SRC, *_span(SRC, "3e-3"))
    lined = SRC.replace("attn = gqa(num_heads=4, num_kv_heads=2, rope=rope(base=10000.0))   # the mixer",
                        "attn = mha: gqa(num_heads=4, num_kv_heads=4)   # full\n     | mqa: gqa(num_heads=4, num_kv_heads=1)")
    s, e = _span(lined, "gqa(num_heads=4, num_kv_heads=1)")
    more = edits.alt_add(lined, s, e, "gqa(num_heads=4, num_kv_heads=2)", "gqa")
    assert "\n     | gqa: gqa(num_heads=4, num_kv_heads=2)\n" in more and "# full" in more and len(_ok(more)) == 6
    less = edits.alt_remove(more, *_span(more, "gqa(num_heads=4, num_kv_heads=1)"))
    assert "mqa" not in less and "# full" in less and len(_ok(less)) == 4
    assert edits.apply(SRC, {"op": "set_setting", "name": "batch", "value": "16"}).count("batch = 16") == 1
    # one field of a setting's call: the rest of the call stays as written
    shaped = SRC.replace("schedule = wsd(warmup=10)", "schedule = wsd(warmup=10, final=0.1)   # cool down to a tenth")
    out = edits.apply(shaped, {"op": "set_setting_field", "name": "schedule", "key": "decay", "value": "0.300", "kind": "wsd"}, "s.bux")
    assert "schedule = wsd(warmup=10, final=0.1, decay=0.300)   # cool down to a tenth" in out and _ok(out)
    out = edits.apply(out, {"op": "set_setting_field", "name": "schedule", "key": "warmup", "value": "25", "kind": "wsd"}, "s.bux")
    assert "wsd(warmup=25, final=0.1, decay=0.300)" in out
    bare = SRC.replace("schedule = wsd(warmup=10)\n", "")
    assert "schedule = wsd(warmup=5)" in edits.set_setting_field(bare, "schedule", "warmup", "5", "wsd", "s.bux")


def test_a_setting_written_in_a_module_is_changed_by_an_amendment(tmp_path):
    (tmp_path / "parts.bux").write_text("attn = gqa(num_heads=4, num_kv_heads=2)\n")
    main = "use parts\n" + SRC.replace("attn = gqa(num_heads=4, num_kv_heads=2, rope=rope(base=10000.0))   # the mixer\n", "")
    path = str(tmp_path / "main.bux")
    s, e = _span(main, "attn", 0)
    out = edits.set_field(main, s, e, "num_heads", "8", path)
    assert out.startswith("use parts\nattn.num_heads = 8\n")
    again = edits.set_field(out, *_span(out, "attn", 1), "num_heads", "2", path)
    assert again.count("attn.num_heads") == 1 and "attn.num_heads = 2" in again
    assert forms.inspect(main, s, e, path)["module"].endswith("parts.bux")


def _balanced(js: str) -> list:
    """A crude check of a JavaScript source: brackets pair up outside strings, template
    literals, comments and regular expressions (no JavaScript engine is installed here)."""
    stack, problems, i, n = [], [], 0, len(js)
    pairs = {")": "(", "]": "[", "}": "{"}
    prev = ""
    while i < n:
        ch = js[i]
        if js.startswith("//", i):
            i = js.find("\n", i) if js.find("\n", i) >= 0 else n
            continue
        if js.startswith("/*", i):
            i = js.find("*/", i) + 2
            continue
        if ch in "\"'":
            j = i + 1
            while j < n and js[j] != ch:
                j += 2 if js[j] == "\\" else 1
                if j < n and js[j - 1] == "\n" and js[j - 2] != "\\":
                    problems.append(f"a string runs over a line end near {js[i:i + 30]!r}")
                    break
            i, prev = j + 1, ch
            continue
        if ch == "`":
            j = i + 1
            while j < n and js[j] != "`":
                if js[j] == "\\":
                    j += 2
                elif js.startswith("${", j):
                    depth, j = 1, j + 2
                    while j < n and depth:
                        depth += {"{": 1, "}": -1}.get(js[j], 0)
                        j += 1
                else:
                    j += 1
            i, prev = j + 1, "`"
            continue
        if ch == "/" and prev in "(,=:[!&|?{};\n" + "":
            j = i + 1
            in_class = False
            while j < n and (js[j] != "/" or in_class):
                if js[j] == "\\":
                    j += 1
                elif js[j] == "[":
                    in_class = True
                elif js[j] == "]":
                    in_class = False
                j += 1
            i, prev = j + 1, "/"
            continue
        if ch in "([{":
            stack.append((ch, js.count("\n", 0, i) + 1))
        elif ch in ")]}":
            if not stack or stack[-1][0] != pairs[ch]:
                problems.append(f"line {js.count(chr(10), 0, i) + 1}: unmatched {ch}")
                break
            stack.pop()
        if not ch.isspace():
            prev = ch
        i += 1
    problems += [f"line {line}: {ch} never closed" for ch, line in stack]
    return problems


def test_the_page_is_served_with_its_modules_and_the_api_guards_the_file(tmp_path):
    from http.server import ThreadingHTTPServer

    from bux_b200.studio import Studio
    from bux_b200.studio.server import STATIC

    for js in STATIC.glob("*.js"):
        assert _balanced(js.read_text()) == [], js.name
        for name in __import__("re").findall(r'from "\./([\w.-]+)"', js.read_text()):
            assert (STATIC / name).exists(), (js.name, name)
    f = tmp_path / "s.bux"
    f.write_bytes(SRC.replace("\n", "\r\n").encode())                 # a file with CRLF line ends
    studio = Studio(f, out=tmp_path / "runs")
    server = ThreadingHTTPServer(("127.0.0.1", 0), studio.handler({"127.0.0.1"}))
    port = server.server_address[1]
    threading.Thread(target=server.serve_forever, daemon=True).start()

    def call(path, body=None, token=studio.token, raw=False, host=None):
        req = urllib.request.Request(f"http://127.0.0.1:{port}{path}?t={token}", data=None if body is None else json.dumps(body).encode(),
                                     headers={"Host": host} if host else {})
        with urllib.request.urlopen(req) as r:
            return r.read() if raw else json.loads(r.read())

    try:
        page = call("/", raw=True).decode()
        assert '<script type="module" src="/static/app.js">' in page
        assert b"export const api" in call("/static/api.js", raw=True)
        for bad in (lambda: call("/api/file", token="nope"), lambda: call("/", token="nope", raw=True),
                    lambda: call("/static/../server.py", raw=True), lambda: call("/api/file", host="evil.example")):
            with pytest.raises(urllib.error.HTTPError) as err:
                bad()
            assert err.value.code in (400, 403, 404)
        loaded = call("/api/file")
        assert loaded["source"] == SRC and "\r" not in loaded["source"]
        v = call("/api/view", {"source": loaded["source"], "run": 1})
        assert v["errors"] == [] and v["run"] == 1 and v["card"]["layers"] == 11
        edited = call("/api/edit", {"source": loaded["source"], "edit": {"op": "set_setting", "name": "steps", "value": "20"}})
        assert "steps = 20\n" in edited["source"]
        refused = call("/api/edit", {"source": loaded["source"], "edit": {"op": "set_field", "start": 0, "end": 3, "key": "x", "value": "1"}})
        assert "drawing is behind" in refused["error"]
        form = call("/api/inspect", {"source": loaded["source"], "start": SRC.index("attn", SRC.index("layer(attn)")), "end": SRC.index("attn", SRC.index("layer(attn)")) + 4})
        assert form["type"] == "gqa"
        assert any(c["label"] == "num_kv_heads" for c in call("/api/complete", {"source": "a = gqa(", "offset": 8}))
        assert call("/api/hover", {"source": loaded["source"], "offset": SRC.index("gqa(")})["text"].startswith("**gqa**")
        saved = call("/api/save", {"source": edited["source"], "mtime": loaded["mtime"]})
        assert b"steps = 20\r\n" in f.read_bytes() and b"\n\n" not in f.read_bytes().replace(b"\r\n", b"")   # CRLF kept
        with pytest.raises(urllib.error.HTTPError) as err:                          # a stale page cannot overwrite
            call("/api/save", {"source": "x", "mtime": loaded["mtime"]})
        assert err.value.code == 409
        call("/api/save", {"source": loaded["source"], "mtime": loaded["mtime"], "overwrite": True})
        assert call("/api/file")["mtime"] != saved["mtime"]
        runs = call("/api/runs")
        assert runs["state"] == "idle" and [r["state"] for r in runs["runs"]] == [None, None]
        fresh = Studio(tmp_path / "new.bux")
        assert compile_runs(fresh.source(), filename="new.bux")                    # the template of a new file compiles
    finally:
        server.shutdown()
