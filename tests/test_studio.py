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
