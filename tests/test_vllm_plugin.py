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
    for qk, ffn in (("", DENSE), (", qk_norm=rmsnorm", DENSE), (", qk_norm=rmsnorm", MOE), (", sinks=true", DENSE)):
        arch = _arch(qk, ffn)
        fam, why = plan.family(json.loads(arch.model_dump_json()))
        assert fam == native.detect(arch), (qk, ffn, why)
    fam, why = plan.family(json.loads(_arch(", sinks=true").model_dump_json()))
    assert fam is None and "sinks" in why


def test_renaming_matches_the_native_export():
    arch = _arch(", qk_norm=rmsnorm", MOE)
    model = Model(arch, dtype=torch.float32)
    exported = W.tensors(model)
    want_cfg, want = native.convert("qwen3_moe", arch, exported, torch.float32)
    got = {}
    for name, t in exported.items():
        for new, piece in plan.rename(f"model.{name}", t, "qwen3_moe"):
            got[new] = piece
    assert set(got) == set(want)
    assert all(torch.equal(got[k], want[k]) for k in want)
    fields = plan.hf_fields(json.loads(arch.model_dump_json()), "qwen3_moe")
    for k, v in fields.items():
        assert want_cfg[k] == v, k
