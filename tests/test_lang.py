"""The .bux language: parsing, evaluation, lowering, sweeps, ids, errors, printing."""
import glob
import os

import pytest

from bux_b200.lang import BuxError, check, compile, compile_runs, compile_spaces
from bux_b200.lang import ir
from bux_b200.lang.printer import run_to_source

SMOKE = """
d_model    = 64
vocab_size = 512
norm  = rmsnorm
attn  = gqa(num_heads=4, num_kv_heads=2, rope=rope())
ffn   = gated_mlp(intermediate_size=4 * d_model, activation=swish)
block = [norm attn] [norm ffn]
model = embed block^2 norm head(tied=true)
data      = synthetic
optimizer = adamw(lr=3e-3)
schedule  = wsd(warmup=10)
seq_len   = 64
batch     = 8
steps     = 50
"""
REF = os.environ.get("BUX_REFERENCE_EXAMPLES", "")  # the reference's examples folder, when there is one


def test_golden_run_ids():
    assert compile_runs(SMOKE, filename="smoke.bux")[0].id == "5a4f0f7d85"
    assert compile_runs(SMOKE, filename="smoke.bux", overrides=["optimizer.lr = 1e-2"])[0].id == "54d678be8d"
    assert compile_runs(SMOKE, filename="smoke.bux", overrides=["seed=1"])[0].id == "9d2a4a5bf8"


def test_id_ignores_how_a_run_is_watched_and_split():
    base = compile_runs(SMOKE, filename="smoke.bux")[0].id
    for extra in (["mesh = mesh(fsdp=2)", "methods.remat = full", "compiler.preset = o1"],
                  ["checkpoint = checkpoint(every=10)", "eval = eval(data=synthetic, every=10)"],
                  ["log = log(every=3)"]):
        assert compile_runs(SMOKE, filename="smoke.bux", overrides=extra)[0].id == base


def test_widths_and_layers():
    arch = compile(SMOKE)
    layers = list(arch.layers())
    assert [l.config.type for l in layers][:3] == ["embed", "rmsnorm", "gqa"]
    assert [l.width for l in layers][:3] == ["tokens", 64, 64]
    assert len(layers) == 1 + 2 * 4 + 2


def test_numbers_and_si_suffixes():
    arch = compile("d_model = 1k\nvocab_size = 64k\nmodel = embed rmsnorm head\n")
    assert arch.d_model == 1000 and arch.vocab_size == 64000
    arch = compile("d_model = 8 * 8 // 2\nvocab_size=10\nmodel = embed head")
    assert arch.d_model == 32


def test_sweep_axes_cross_and_labels_zip():
    runs = compile_runs(SMOKE, filename="s.bux", overrides=["optimizer.lr = 1e-3 | 3e-3", "seed = 0 | 1"])
    assert len(runs) == 4
    assert runs[0].name == "s[optimizer.lr=1e-3, seed=0]"
    src = SMOKE.replace("d_model    = 64", "d_model = s: 64 | m: 128") + "optimizer.lr = s: 4e-3 | m: 3e-3\n"
    runs = compile_runs(src, filename="w.bux")
    assert [r.name for r in runs] == ["w[s]", "w[m]"]
    assert runs[1].arch.d_model == 128 and runs[1].train.optimizer.lr == 3e-3


def test_partial_label_overlap_is_an_error():
    src = SMOKE.replace("d_model    = 64", "d_model = s: 64 | m: 128") + "optimizer.lr = s: 4e-3 | l: 3e-3\n"
    with pytest.raises(BuxError, match="share some labels"):
        compile_runs(src)


def test_amendments_macros_patterns_shared():
    src = """
d_model = 32
vocab_size = 16
attn = gqa(num_heads=4, num_kv_heads=4)
attn.num_kv_heads = 2
attn.rope = rope(base=5000)
layer(mixer, f=mlp(intermediate_size=64, activation=gelu)) = [rmsnorm mixer] [rmsnorm f]
A = layer(attn)
M = layer(attn, gated_mlp(intermediate_size=32, activation=swish))
shared out = head
model = embed "AM"^2 rmsnorm out
"""
    arch = compile(src)
    types = [l.config.type for l in arch.layers()]
    assert types.count("gqa") == 4 and types.count("mlp") == 2 and types.count("gated_mlp") == 2
    gqa = next(l.config for l in arch.layers() if l.config.type == "gqa")
    assert gqa.num_kv_heads == 2 and gqa.rope.base == 5000


def test_taps_and_unet():
    src = """
d_model = 16
vocab_size = 8
b = [rmsnorm mlp(intermediate_size=32, activation=relu)]
model = embed (b @skip)^2 ([$skip! scale] b)^2 head
"""
    arch = compile(src)
    assert any(isinstance(n, ir.Tap) for n in ir.walk(arch.graph))
    with pytest.raises(BuxError, match="read before anything writes"):
        compile("d_model=16\nvocab_size=8\nmodel = embed [$nope] head")


def test_error_messages_point_at_the_source():
    with pytest.raises(BuxError) as e:
        compile("d_model = 64\nvocab_size = 8\nmodel = embed nrom head\n", filename="tiny.bux")
    text = str(e.value)
    assert "unknown layer or block 'nrom'" in text and "tiny.bux:3:15" in text and "^^^^" in text
    with pytest.raises(BuxError, match="has no setting 'num_head'"):
        compile("d_model=8\nvocab_size=8\nmodel = embed gqa(num_head=2) head")
    with pytest.raises(BuxError, match="must keep the width"):
        compile("d_model=8\nvocab_size=8\nmodel = embed [linear(features=4)] head")
    with pytest.raises(BuxError, match="nothing can follow the LM head"):
        compile("d_model=8\nvocab_size=8\nmodel = embed head rmsnorm")
    with pytest.raises(BuxError, match="needs exactly one embedding"):
        compile("d_model=8\nvocab_size=8\nmodel = rmsnorm head(tied=true)")


def test_check_collects_every_error():
    report = check("d_model = 8\nvocab_size = 8\na = gqa(num_heads=3, num_kv_heads=2)\nmodel = embed nrom head\n")
    assert len(report.errors) >= 2


def test_residual_algebra_inserts_merge():
    src = "d_model=16\nvocab_size=8\nresidual = hc(expansion=2)\nmodel = embed [rmsnorm] rmsnorm head"
    arch = compile(src)
    types = [l.config.type for l in arch.layers()]
    assert "merge" in types and types.index("merge") < len(types) - 1


def test_data_mixture_and_objective():
    src = SMOKE.replace("data      = synthetic", 'web = tokens(path="a*.bin")\ncode = tokens(path="b*.bin")\n'
                        "data = 0.75 * web + 0.25 * code")
    run = compile_runs(src)[0]
    assert [w.weight for w in run.train.data.sources] == [0.75, 0.25]


def test_search_dimensions():
    src = SMOKE.replace("adamw(lr=3e-3)", "adamw(lr=log_uniform(1e-4, 1e-2))")
    [space] = compile_spaces(src, filename="tune.bux")
    assert list(space.dimensions) == ["optimizer.lr"]
    assert space.trial({"optimizer.lr": 3e-4}).name == "tune[optimizer.lr=3e-4]"


def test_printer_round_trips():
    run = compile_runs(SMOKE, filename="smoke.bux")[0]
    text = run_to_source(run)
    assert text.startswith("# smoke, run 5a4f0f7d85")
    assert compile_runs(text, filename="smoke.bux")[0].id == run.id


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference examples not mounted")
def test_every_reference_example_compiles():
    bad = []
    for path in sorted(glob.glob(f"{REF}/**/*.bux", recursive=True)):
        src = open(path).read()
        try:
            compile_runs(src, filename=path)
        except BuxError as err:
            if "defines a model, not a run" in err.message:
                compile(src, filename=path)
            elif "no definition named 'model'" not in err.message:
                bad.append((path, err.message))
    assert not bad, bad[:5]


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference examples not mounted")
def test_every_reference_architecture_builds():
    """Every file of the reference's model zoo becomes a module tree (on the meta device)."""
    import torch

    from bux_b200.models import Model

    bad = []
    for path in sorted(glob.glob(f"{REF}/architectures/**/*.bux", recursive=True)):
        src = open(path).read()
        try:
            try:
                arch = compile_runs(src, filename=path)[0].arch
            except BuxError:
                arch = compile(src, filename=path)
            with torch.device("meta"):
                Model(arch)
        except Exception as err:  # noqa: BLE001 - every failure is listed
            bad.append((path, f"{type(err).__name__}: {err}"))
    assert not bad, bad[:5]


def test_own_examples_compile_and_build():
    import torch

    from bux_b200.models import Model

    root = os.path.join(os.path.dirname(os.path.dirname(__file__)), "examples")
    paths = sorted(glob.glob(f"{root}/**/*.bux", recursive=True))
    assert len(paths) >= 25
    for path in paths:
        src = open(path).read()
        try:
            archs = [run.arch for run in compile_runs(src, filename=path)]
        except BuxError as err:
            assert "defines a model, not a run" in err.message, (path, str(err))
            archs = [compile(src, filename=path)]
        with torch.device("meta"):
            for arch in archs:
                Model(arch)
