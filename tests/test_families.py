"""The model families of the example files, shrunk to toy sizes, build and take a step on
CPU; the full-size files compile and are counted on the meta device."""
from pathlib import Path

import pytest
import torch

from bux_b200.lang import compile_runs
from bux_b200.train.trainer import Trainer, count_params

ROOT = Path(__file__).resolve().parent.parent
TAIL = """
data = synthetic
optimizer = adamw(lr=1e-2)
seq_len = 32
batch = 2
steps = 2
precision = precision(compute=float32)
"""


def _toy(name: str, overrides: list):
    src = (ROOT / "examples" / "architectures" / f"{name}.bux").read_text() + TAIL
    return compile_runs(src, filename=f"{name}.bux", overrides=overrides)[0]


@pytest.mark.parametrize("name,overrides", [
    ("llama3_8b", ["d_model = 64", "vocab_size = 128"]),
    ("qwen3_30b_a3b", ["d_model = 64", "vocab_size = 128"]),
    ("gpt_oss_20b", ["d_model = 64", "vocab_size = 128"]),
])
def test_family_steps_on_cpu(name, overrides):
    src = (ROOT / "examples" / "architectures" / f"{name}.bux").read_text()
    # shrink by text: heads, widths, experts and depth
    import re

    small = re.sub(r"num_heads=\d+", "num_heads=4", src)
    small = re.sub(r"num_kv_heads=\d+", "num_kv_heads=2", small)
    small = re.sub(r"head_dim=\d+", "head_dim=16", small)
    small = re.sub(r"intermediate_size=\d+", "intermediate_size=32", small)
    small = re.sub(r"num_experts=\d+", "num_experts=4", small)
    small = re.sub(r"top_k=\d+", "top_k=2", small)
    small = re.sub(r"\^\d+", "^2", small)
    small = re.sub(r"d_model\s*=\s*\d+", "d_model = 64", small)
    small = re.sub(r"vocab_size\s*=\s*\d+", "vocab_size = 128", small)
    small = re.sub(r"original_max_len=\d+", "original_max_len=16", small)
    run = compile_runs(small + TAIL, filename=f"{name}.bux")[0]
    tr = Trainer(run, device="cpu")
    batch = next(iter(tr.batches()))
    losses = [tr.train_step(batch)["loss"].item() for _ in range(3)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]


@pytest.mark.parametrize("file,params", [("llama3_8b_fsdp8", 8.03e9), ("qwen3_30b_a3b_mxfp8", 30.5e9),
                                         ("gpt_oss_20b_ep8", 20.9e9)])
def test_benchmark_files_compile_at_full_size(file, params):
    path = ROOT / "examples" / "benchmarks" / f"{file}.bux"
    run = compile_runs(path.read_text(), filename=str(path))[0]
    assert count_params(run.arch) == pytest.approx(params, rel=0.02)
