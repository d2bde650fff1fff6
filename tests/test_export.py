"""Export: a trained run → a Hugging Face folder that computes the same logits, in the
bux format and, for standard decoders, in the family's own format read by transformers."""
import json

import pytest
import torch

from bux_b200.export import check as C
from bux_b200.export import export, native, weights as W
from bux_b200.lang import compile_runs
from bux_b200.train.trainer import train

BASE = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, rope=rope(){qk})
f = {ffn}
block = [n a] [n f]
model = embed block^2 n head(tied=false)
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 16
batch = 4
steps = 3
checkpoint = checkpoint(every=3)
precision = precision(compute=float32)
log = log(every=100)
{extra}
"""
DENSE = "gated_mlp(intermediate_size=48, activation=swish)"
MOE = "moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish))"


def _trained(tmp_path, qk="", ffn=DENSE, extra=""):
    run = compile_runs(BASE.format(qk=qk, ffn=ffn, extra=extra), filename="e.bux")[0]
    tr = train(run, out=tmp_path / "runs", device="cpu", quiet=True)
    (folder,) = list((tmp_path / "runs").iterdir())
    return run, tr, folder


def test_weight_names_split_and_fuse_back(tmp_path):
    run, tr, _ = _trained(tmp_path, ffn=MOE)
    t = W.tensors(tr.model)
    names = set(t)
    assert any(n.endswith(".q.weight") for n in names) and not any("qkv" in n for n in names)
    assert any(n.endswith("experts.gate") for n in names) and any(n.endswith("experts.down") for n in names)
    back = W.fused(tr.model, t)
    own = tr.model.state_dict()
    assert set(back) == set(own)
    assert all(torch.equal(back[k], own[k]) for k in own)


def test_detects_standard_families():
    fam = lambda qk, ffn, extra="": native.detect(compile_runs(BASE.format(qk=qk, ffn=ffn, extra=extra), filename="e.bux")[0].arch)
    assert fam("", DENSE) == "llama"
    assert fam(", qk_norm=rmsnorm", DENSE) == "qwen3"
    assert fam(", qk_norm=rmsnorm", MOE) == "qwen3_moe"
    assert fam(", sinks=true", DENSE) is None
    assert fam(", bias=true", DENSE) is None and fam(", bias=true, output_bias=false", DENSE) == "qwen2"
    assert fam(", sliding_window_size=8", DENSE) == "mistral" and fam(", sliding_window_size=8, bias=true, output_bias=false", DENSE) is None
    assert fam("", MOE) == "mixtral" and fam("", MOE.replace("top_k=2,", "top_k=2, normalize_top_k=false,")) is None
    assert fam(", paired=true", DENSE) is None and fam(", exclusive=true", DENSE) is None
    with_pointer = BASE.format(qk="", ffn=DENSE, extra="").replace("head(tied=false)", "head(tied=false, pointer=copy_pointer(dim=8))")
    assert native.detect(compile_runs(with_pointer, filename="e.bux")[0].arch) is None
    assert fam(", qk_norm=rmsnorm", MOE.replace("top_k=2,", "top_k=2, latent_size=16,")) is None
    assert fam(", qk_norm=rmsnorm", MOE.replace("top_k=2,", "top_k=2, expert_norm=rmsnorm,")) is None
    assert fam(", qk_norm=rmsnorm", MOE.replace("top_k=2,", "top_k=2, random_logits=true,")) == "qwen3_moe"
    assert fam("", DENSE, "residual = hc(expansion=2)") is None


def test_bux_format_round_trip(tmp_path):
    run, tr, folder = _trained(tmp_path, qk=", sinks=true")   # not a standard family
    out = export(folder, tmp_path / "hf", dtype="float32", check=True, echo=lambda *_: None)
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["model_type"] == "bux" and cfg["bux"]["run"] == run.id and cfg["bux_layer_types"].count("gqa") == 2 and cfg["layer_types"] == ["full_attention"] * 2
    assert (out / "modeling_bux.py").exists() and (out / "model.safetensors").exists()
    report = C.compare(tr.model, out)
    report.check()
    assert [r.implementation for r in report.results] == ["bux"] and report.max_error < 1e-4
    assert report.results[0].greedy["cache"] == report.results[0].greedy["bux"] and report.results[0].padded


@pytest.mark.parametrize("qk,ffn,family", [
    ("", DENSE, "llama"), (", qk_norm=rmsnorm", DENSE, "qwen3"), (", qk_norm=rmsnorm", MOE, "qwen3_moe"),
    (", sliding_window_size=5", DENSE, "mistral"), (", bias=true, output_bias=false", DENSE, "qwen2"), ("", MOE, "mixtral"),
    ("LLAMA3", DENSE, "llama"), ("YARN", DENSE, "qwen3"), ("PI", DENSE, "llama")])
def test_standard_families_load_in_transformers(tmp_path, qk, ffn, family):
    scaled = {"LLAMA3": "rope(scaling=llama3(factor=4.0, original_max_len=8))",
              "YARN": "rope(scaling=yarn(factor=4.0, original_max_len=8)), qk_norm=rmsnorm",
              "PI": "rope(scaling=pi(factor=2.0))"}.get(qk)
    if scaled:     # a scaled RoPE: the family's rope_parameters must mean what the layer computes
        global BASE
        run = compile_runs(BASE.replace("rope=rope(){qk}", "rope=" + scaled).format(ffn=ffn, extra=""), filename="e.bux")[0]
        tr = train(run, out=tmp_path / "runs", device="cpu", quiet=True)
        (folder,) = list((tmp_path / "runs").iterdir())
    else:
        run, tr, folder = _trained(tmp_path, qk=qk, ffn=ffn)
    out = export(folder, tmp_path / "hf", dtype="float32", echo=lambda *_: None)
    assert json.loads((out / "config.json").read_text())["model_type"] == family
    report = C.compare(tr.model, out, tolerance=2e-3)   # transformers' own implementation of the family
    report.check()                                       # logits, greedy with and without its cache, left padding
    assert [r.implementation for r in report.results] == ["eager", "sdpa"]


@pytest.mark.parametrize("qk", [", k_eq_v=true, differential=true", ", paired=true", ", exclusive=learned, power_scale=0.5",
                                ", gated=true, gate_input_rank=4, gate_cross_head=true, kv_conv_size=3"])
def test_less_common_attention_settings_round_trip(tmp_path, qk):
    """The exported model rebuilds the graph from the architecture, so every setting of the
    layer survives the export; the fused projection splits only into the parts it has."""
    run, tr, folder = _trained(tmp_path, qk=qk)
    assert native.detect(run.arch) is None
    out = export(folder, tmp_path / "hf", dtype="float32", check=True, echo=lambda *_: None)
    report = C.compare(tr.model, out)
    report.check()
    assert report.max_error < 1e-4
    names = set(W.tensors(tr.model))
    assert ("k_eq_v" in qk) == (not any(n.endswith(".v.weight") for n in names))


def test_exported_folder_loads_without_the_package(tmp_path):
    """The exported folder carries the Python sources it needs: a process that cannot import
    `bux_b200` loads it with transformers alone and computes the trained model's logits."""
    import subprocess
    import sys

    run, tr, folder = _trained(tmp_path, qk=", sinks=true")
    out = export(folder, tmp_path / "hf", dtype="float32", echo=lambda *_: None)
    assert (out / "bux_runtime" / "models" / "model.py").exists()
    assert not list((out / "bux_runtime").rglob("*.cu")) and not list((out / "bux_runtime").rglob("*.so"))
    ids = torch.arange(12).reshape(1, 12) % 64
    want = tr.model.logits(ids, training=False).float()
    torch.save({"ids": ids, "want": want}, tmp_path / "probe.pt")
    script = f"""
import sys
sys.path = [p for p in sys.path if p not in ('', {str(__import__('os').path.dirname(__import__('os').path.dirname(__import__('os').path.abspath(__file__))))!r})]
try:
    import bux_b200
    raise SystemExit("bux_b200 is importable here: the test proves nothing")
except ImportError:
    pass
import torch
from transformers import AutoModelForCausalLM
model = AutoModelForCausalLM.from_pretrained({str(out)!r}, trust_remote_code=True)
probe = torch.load({str(tmp_path / 'probe.pt')!r})
got = model(probe["ids"]).logits
err = (got - probe["want"]).abs().max().item()
print("max_abs_error", err)
assert err < 1e-4, err
"""
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, cwd=str(tmp_path),
                          env={k: v for k, v in __import__("os").environ.items() if k != "PYTHONPATH"})
    assert proc.returncode == 0, proc.stdout + proc.stderr


def test_decoding_over_a_key_value_cache_equals_whole_sequence_passes():
    """`DecodeCache`: a prompt in one call and tokens one at a time give the logits of passes
    over the whole sequence, with sinks, a window, q/k norms, a value residual through a port,
    experts, and a left-padded row beside a full one; graphs with other state are refused."""
    from bux_b200.models import Model
    from bux_b200.models.cache import DecodeCache, supports

    src = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, rope=rope(), sinks=true, qk_norm=rmsnorm, softcap=20.0, value_residual=learned)
w = a(sliding_window_size=4)
e = moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish))
model = embed [n a(v=@v)] [n e] ([n w(v=$v)] [n gated_mlp(intermediate_size=48, activation=gelu)])^2 n head
"""
    from bux_b200.lang import compile

    arch = compile(src, filename="c.bux")
    assert supports(arch) is None
    model = C.perturbed(Model(arch, dtype=torch.float32), scale=0.05).eval()
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 64, (2, 10), generator=g)
    mask = torch.ones(2, 10, dtype=torch.int32)
    mask[1, :3] = 0                                                   # the second row is left-padded by three
    pos = (mask.cumsum(-1) - 1).clamp_min(0)
    with torch.no_grad():
        whole = model(ids, pos, mask, training=False).heads[0].logits().float()
        cache = DecodeCache()
        first = model(ids[:, :6], pos[:, :6], mask[:, :6], training=False, cache=cache).heads[0].logits().float()
        steps = [model(ids[:, t:t + 1], pos[:, t:t + 1], mask[:, t:t + 1], training=False, cache=cache).heads[0].logits().float()
                 for t in range(6, 10)]
    got = torch.cat([first, *steps], dim=1)
    real = mask.bool()
    assert torch.allclose(got[real], whole[real], atol=2e-5), (got[real] - whole[real]).abs().max()
    assert cache.length == 10
    for bad, why in (("a = gqa(num_heads=4, num_kv_heads=2, indexer=indexer(num_heads=2, head_dim=8, top_k=2))", "indexer"),
                     ("a = csa(num_heads=2, head_dim=16, compress_ratio=4)", "csa"), ("residual = hc(expansion=2)\na = gqa(num_heads=4, num_kv_heads=2)", "hc")):
        other = compile("d_model=32\nvocab_size=64\n" + bad + "\nmodel = embed [rmsnorm a] rmsnorm head\n", filename="c.bux")
        assert why in supports(other)


@pytest.mark.parametrize("mixer", ["gdn(num_heads=2, head_dim=16)", "kda(num_heads=2, head_dim=16)", "deltanet(num_heads=2, head_dim=16)",
                                   "gla(num_heads=2, head_dim=16)", "lightning(num_heads=2, head_dim=16)",
                                   "gdn2(num_heads=2, head_dim=16)", "short_conv(conv_size=3)", "conv(size=4)",
                                   "rwkv7(num_heads=2, head_dim=16)", "mamba(state_size=8)", "mamba2(state_size=16, head_dim=16)",
                                   "mla(num_heads=2, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=8, rope=rope())"])
def test_recurrent_mixers_and_convolutions_continue_from_the_cache(mixer):
    """A hybrid of one recurrent mixer (or a convolution) and attention decodes token by token to
    the logits of whole-sequence passes: the recurrent state and the convolutions' last inputs
    live in the cache; a left-padded row restarts both at its first real token."""
    from bux_b200.lang import compile
    from bux_b200.models import Model
    from bux_b200.models.cache import DecodeCache, supports

    arch = compile(f"""
d_model=32
vocab_size=64
n = rmsnorm
r = {mixer}
a = gqa(num_heads=4, num_kv_heads=2, rope=rope())
f = gated_mlp(intermediate_size=48, activation=swish)
model = embed ([n r] [n f] [n a] [n f])^2 n head
""", filename="h.bux")
    assert supports(arch) is None
    model = C.perturbed(Model(arch, dtype=torch.float32), scale=0.05).eval()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 64, (2, 9), generator=g)
    mask = torch.ones(2, 9, dtype=torch.int32)
    mask[1, :2] = 0
    pos = (mask.cumsum(-1) - 1).clamp_min(0)
    with torch.no_grad():
        whole = model(ids, pos, mask, training=False).heads[0].logits().float()
        cache = DecodeCache()
        parts = [model(ids[:, :5], pos[:, :5], mask[:, :5], training=False, cache=cache).heads[0].logits().float()]
        parts += [model(ids[:, t:t + 1], pos[:, t:t + 1], mask[:, t:t + 1], training=False, cache=cache).heads[0].logits().float()
                  for t in range(5, 9)]
    got, real = torch.cat(parts, dim=1), mask.bool()
    assert torch.allclose(got[real], whole[real], atol=5e-5), (got[real] - whole[real]).abs().max()
    assert "engram" in supports(compile("d_model=32\nvocab_size=64\nmodel = embed [rmsnorm engram(head_dim=8, table_size=64)] rmsnorm head\n", filename="h.bux"))


def test_exported_model_samples_and_stops_at_the_end_token(tmp_path):
    run, tr, folder = _trained(tmp_path, qk=", sinks=true")
    out = export(folder, tmp_path / "hf", dtype="float32", echo=lambda *_: None)
    hf = C.load_exported(out)
    ids = torch.arange(6).reshape(1, 6) % 64
    greedy = hf.generate(ids, max_new_tokens=5)
    assert torch.equal(greedy, hf.generate(ids, max_new_tokens=5, use_cache=False))
    assert torch.equal(greedy, hf.generate(ids, max_new_tokens=5, do_sample=True, top_k=1))          # top-1 sampling is greedy
    g = lambda: torch.Generator().manual_seed(3)
    a = hf.generate(ids, max_new_tokens=8, do_sample=True, temperature=1.5, top_p=0.9, generator=g())
    b = hf.generate(ids, max_new_tokens=8, do_sample=True, temperature=1.5, top_p=0.9, generator=g())
    assert torch.equal(a, b) and a.shape == (1, 14)
    eos = int(greedy[0, 7])                                   # the second decoded token ends the row
    stopped = hf.generate(ids, max_new_tokens=5, eos_token_id=eos, pad_token_id=63)
    assert stopped.shape[1] <= 8 or (stopped[0, 8:] == 63).all()
    assert stopped[0, :8].tolist() == greedy[0, :8].tolist() or eos in stopped[0, 6:8].tolist()


def test_a_file_exports_its_model_without_weights(tmp_path, capsys):
    """``bux export FILE.bux OUT``: config (and code), no weights; the model is only built on the
    meta device, so a model far larger than this machine's memory exports."""
    from pathlib import Path

    from bux_b200.__main__ import main

    root = Path(__file__).resolve().parent.parent / "examples" / "architectures"
    out = tmp_path / "llama"
    (out).mkdir()
    (out / "model.safetensors").write_bytes(b"left by an earlier export")
    assert main(["export", str(root / "llama3_70b.bux"), str(out)]) == 0
    assert "70.6B parameters exported" in capsys.readouterr().out and "without weights" 
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["model_type"] == "llama" and cfg["num_hidden_layers"] == 80 and not (out / "model.safetensors").exists()
    out = tmp_path / "hybrid"
    assert main(["export", str(root / "hybrid_gdn.bux"), str(out), "d_model = 512", "--dtype", "float32"]) == 0
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["model_type"] == "bux" and cfg["hidden_size"] == 512 and cfg["bux"]["run"] is None and cfg["torch_dtype"] == "float32"
    assert (out / "modeling_bux.py").exists() and (out / "bux_runtime" / "models" / "cache.py").exists()
