"""`bux export --check`: runs the trained model and the exported folder on the same
tokens and compares the logits. Reference: ``export/check.py:95``."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def load_exported(folder):
    folder = Path(folder)
    kind = json.loads((folder / "config.json").read_text())["model_type"]
    if kind == "bux":
        from .hf.modeling_bux import BuxForCausalLM

        return BuxForCausalLM.from_pretrained(folder)
    from transformers import AutoModelForCausalLM

    return AutoModelForCausalLM.from_pretrained(folder, dtype=torch.float32).eval()


@torch.no_grad()
def compare(model, folder, tokens: int = 64, rows: int = 2, seed: int = 0, atol: float = None) -> dict:
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, model.arch.vocab_size, (rows, tokens), generator=g)
    pos = torch.arange(tokens).expand(rows, tokens)
    want = model(ids, pos, None, training=False).heads[0].logits().float()
    other = load_exported(folder)
    got = other(input_ids=ids).logits.float()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    tol = atol if atol is not None else 2e-2 * max(scale, 1.0)
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean().item()
    return {"max_abs_error": err, "logit_scale": scale, "argmax_agreement": agree, "ok": err <= tol}
