"""Writes a Hugging Face folder: ``config.json`` (carries the IR), ``configuration_bux.py``,
``modeling_bux.py``, ``model.safetensors``, and a model card. Architectures that are a
standard decoder (``native.detect``) are also written in that family's own format, so a
stock serving stack loads them without any plugin. Reference: ``export/huggingface.py:40``."""

from __future__ import annotations

import json
import shutil
from pathlib import Path

import torch

from . import native
from . import weights as W

HERE = Path(__file__).resolve().parent


def layer_types(arch) -> list:
    return [layer.config.type for layer in arch.layers()]


def cache_types(arch) -> list:
    """What each token mixer keeps between decoding steps, in transformers' vocabulary."""
    out = []
    for layer in arch.layers():
        c = layer.config
        if c.type in ("gqa", "mla", "csa"):
            out.append("sliding_attention" if getattr(c, "sliding_window_size", None) else "full_attention")
        elif c.type in ("conv", "short_conv", "engram"):
            out.append("conv")
        elif c.type in native.MIXERS:
            out.append("linear_attention")
    return out


def save(run, model, folder, dtype=torch.bfloat16, step=None, family: str = "auto") -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch = run.arch
    fam = native.detect(arch) if family == "auto" else (None if family == "bux" else family)
    tensors = {f"model.{k}": v for k, v in W.tensors(model, dtype=dtype).items() if not k.endswith("inv_freq")}
    if fam is not None:
        config, tensors = native.convert(fam, arch, W.tensors(model, dtype=dtype), dtype)
    else:
        config = bux_config(arch, dtype, {"run": run.id, "name": run.name, "step": step})
        for name in ("configuration_bux.py", "modeling_bux.py"):
            shutil.copy(HERE / "hf" / name, folder / name)
        vendor_runtime(folder)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"),
              metadata={"format": "pt"})
    (folder / "README.md").write_text(card(run, step, fam))
    return folder


def save_architecture(arch, folder, dtype=torch.bfloat16, name: str = "model", family: str = "auto") -> tuple:
    """Write `arch` without weights: its ``config.json`` (and, in the bux format, its code), but
    no ``model.safetensors`` (one an earlier export left there is removed). A serving stack can
    run it on random weights to time an architecture before anything is trained. The model is
    only ever built on the ``meta`` device (shapes, no memory), so a hundred billion parameters
    export in seconds. Returns (folder, number of parameters)."""
    from ..models import Model

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    with torch.device("meta"):
        model = Model(arch, dtype=dtype)
    params = model.num_params()
    fam = native.detect(arch) if family == "auto" else (None if family == "bux" else family)
    if fam is not None:
        config, _ = native.convert(fam, arch, W.tensors(model, dtype=dtype), dtype)
    else:
        config = bux_config(arch, dtype, {"run": None, "name": name, "step": None})
        for file in ("configuration_bux.py", "modeling_bux.py"):
            shutil.copy(HERE / "hf" / file, folder / file)
        vendor_runtime(folder)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    (folder / "model.safetensors").unlink(missing_ok=True)
    return folder, params


def bux_config(arch, dtype, origin: dict) -> dict:
    """``config.json`` of the bux format: what transformers and serving stacks read, and the IR."""
    return {
        "model_type": "bux", "architectures": ["BuxForCausalLM"],
        "auto_map": {"AutoConfig": "configuration_bux.BuxConfig",
                     "AutoModelForCausalLM": "modeling_bux.BuxForCausalLM"},
        "vocab_size": arch.vocab_size, "hidden_size": arch.d_model,
        "num_hidden_layers": sum(1 for t in layer_types(arch) if t in native.MIXERS),
        "layer_types": cache_types(arch), "bux_layer_types": layer_types(arch),
        "tie_word_embeddings": any(getattr(l.config, "tied", False) for l in arch.layers()),
        "torch_dtype": str(dtype).removeprefix("torch."),
        "bux": {"architecture": json.loads(arch.model_dump_json()), **origin,
                "dtype": str(dtype).removeprefix("torch.")},
    }


def vendor_runtime(folder: Path) -> Path:
    """Copy this package's Python sources into ``<folder>/bux_runtime`` so that the exported
    folder loads where the package is not installed (the reference copies its torch layers,
    ``export/hf/*.py``, for the same reason: ``export/huggingface.py:40-170`` there). Only
    ``.py`` files travel: no native sources, no built library, no studio assets."""
    package = HERE.parent
    target = Path(folder) / "bux_runtime"
    if target.exists():
        shutil.rmtree(target)
    skip = {"csrc", "_ext", "studio", "__pycache__"}
    for src in sorted(package.rglob("*.py")):
        rel = src.relative_to(package)
        if skip & set(rel.parts):
            continue
        dst = target / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copy(src, dst)
    return target


def card(run, step, family) -> str:
    from ..lang.printer import run_to_source

    how = (f"a standard `{family}` checkpoint: any stack that serves that family loads it"
           if family else "a `bux` checkpoint: load it with `trust_remote_code=True` (the folder carries the "
                          "Python sources it needs), or serve it with the `bux_vllm_b200` plugin")
    return (f"# {run.name}\n\nExported from run `{run.id}`" + (f" at step {step}" if step is not None else "")
            + f". This folder is {how}.\n\n```bux\n{run_to_source(run)}\n```\n")
