"""The serving plugin's plan: which vLLM decoder an exported IR is, its config fields and
the tensor renaming (no vLLM engine is started here)."""
import json

import torch

from bux_b200.export import native, weights as W
from bux_b200.lang import compile_runs
from bux_b200.models import Model
from bux_vllm_b200 import plan

SRC = """
d_model=32
vocab_size=64
n = rmsnorm
a = gqa(num_heads=4, num_kv_heads=2, rope=rope(){qk})
block = [n a] [n {ffn}]
model = embed block^2 n head(tied=false)
data = synthetic
optimizer = adamw(lr=1e-3)
seq_len = 16
batch = 4
steps = 3
"""
DENSE = "gated_mlp(intermediate_size=48, activation=swish)"
MOE = "moe(num_experts=4, top_k=2, expert=gated_mlp(intermediate_size=16, activation=swish))"


def _arch(qk="", ffn=DENSE):
    return compile_runs(SRC.format(qk=qk, ffn=ffn), filename="v.bux")[0].arch


def test_plan_agrees_with_the_exporter():
    for qk, ffn in (("", DENSE), (", qk_norm=rmsnorm", DENSE), (", qk_norm=rmsnorm", MOE), (", sinks=true", DENSE),
                    (", sliding_window_size=8", DENSE), (", bias=true, output_bias=false", DENSE), (", bias=true", DENSE),
                    ("", MOE), ("", MOE.replace("top_k=2,", "top_k=2, normalize_top_k=false,")),
                    (", sliding_window_size=8, qk_norm=rmsnorm", DENSE), (", paired=true", DENSE)):
        arch = _arch(qk, ffn)
        fam, why = plan.family(json.loads(arch.model_dump_json()))
        assert fam == native.detect(arch), (qk, ffn, why)
    fam, why = plan.family(json.loads(_arch(", sinks=true").model_dump_json()))
    assert fam is None and "sinks" in why


import pytest


@pytest.mark.parametrize("qk,ffn,fam", [
    (", qk_norm=rmsnorm", MOE, "qwen3_moe"), ("", MOE, "mixtral"), (", bias=true, output_bias=false", DENSE, "qwen2"),
    (", sliding_window_size=8", DENSE, "mistral"), ("SCALED", DENSE, "llama")])
def test_renaming_matches_the_native_export(qk, ffn, fam):
    if qk == "SCALED":
        arch = compile_runs(SRC.replace("rope=rope(){qk}", "rope=rope(scaling=llama3(factor=4.0, original_max_len=8))")
                            .format(ffn=ffn), filename="v.bux")[0].arch
    else:
        arch = _arch(qk, ffn)
    model = Model(arch, dtype=torch.float32)
    exported = W.tensors(model)
    want_cfg, want = native.convert(fam, arch, exported, torch.float32)
    got = {}
    for name, t in exported.items():
        for new, piece in plan.rename(f"model.{name}", t, fam):
            got[new] = piece
    assert set(got) == set(want)
    assert all(torch.equal(got[k], want[k]) for k in want)
    assert plan.family(json.loads(arch.model_dump_json()))[0] == fam
    fields = plan.hf_fields(json.loads(arch.model_dump_json()), fam)
    for k, v in fields.items():
        assert want_cfg[k] == v, k


def test_every_family_names_a_module_of_the_installed_vllm():
    """Without starting vLLM: the module and class the plugin would import for each family are
    in the installed package, and transformers has the config class."""
    import importlib.util

    import transformers

    from bux_vllm_b200 import model

    assert set(model._MODULES) == set(plan.FAMILIES)
    for fam, (module, cls, cfg) in model._MODULES.items():
        assert cls == plan.FAMILIES[fam] and hasattr(transformers, cfg), fam
        spec = importlib.util.find_spec(module)
        if spec is None:      # vLLM is not installed here: nothing to compare with
            continue
        assert f"class {cls}(" in open(spec.origin).read(), (fam, module)
