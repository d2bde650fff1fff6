"""`bux export --check`: the exported folder against the trained model, in float32.

`compare` loads the folder back (transformers' own class for a standard family, once per
attention implementation; the folder's `BuxForCausalLM` otherwise) and measures

* every head's logits on a batch of random tokens, against the model's;
* greedy decoding with the loaded model's cache, without it, and by full forwards of the
  trained model: the three must give the same tokens;
* a left-padded batch: a prompt decoded beside a shorter one must decode as it does alone.

`Report.check()` raises with what disagrees; ``bux export --check`` exits 1 on it.
Reference: ``export/check.py:33-257``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

import torch


@dataclass
class Result:
    implementation: str      # transformers' attention implementation, or "bux" for the folder's own class
    error: float             # largest |difference| of any head's logits over the largest |logit|
    agreement: float         # share of positions whose argmax token is the same
    greedy: dict             # "cache", "no cache", "bux": one row of tokens each, prompt included
    padded: bool             # a left-padded batch decodes as each prompt alone


@dataclass
class Report:
    results: list = field(default_factory=list)
    tolerance: float = 1e-4
    logit_scale: float = 1.0
    exact: bool = True   # the folder holds float32: its greedy tokens must be the trained model's

    @property
    def max_error(self) -> float:
        return max((r.error for r in self.results), default=0.0)

    def problems(self) -> list:
        out = []
        for r in self.results:
            if not r.error <= self.tolerance:
                out.append(f"{r.implementation}: logits off by {r.error:.2e} (relative), tolerance {self.tolerance:.0e}")
            # weights stored in 16 bits may break a near-tie otherwise than float32 does: there the
            # cache is held to the folder's own cacheless decoding instead of the trained model's
            ref, name = (r.greedy["bux"], "the trained model") if self.exact else (r.greedy["no cache"], "without the cache")
            for how in ("cache", "no cache"):
                if r.greedy[how] != ref:
                    out.append(f"{r.implementation} greedy, {how}: {r.greedy[how]}, {name} {ref}")
            if not r.padded:
                out.append(f"{r.implementation}: a left-padded batch decodes otherwise than its prompts alone")
        return out

    @property
    def ok(self) -> bool:
        return not self.problems()

    def check(self) -> None:
        found = self.problems()
        assert not found, "; ".join(found)


def perturbed(model, seed: int = 1, scale: float = 0.1):
    """Add noise to every parameter in place, so that gains at one and biases at zero (where
    fresh weights start) cannot hide a tensor the export dropped or misplaced."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(scale * torch.randn(p.shape, generator=g).to(p.dtype).to(p.device))
    return model


def kind_of(folder) -> str:
    return json.loads((Path(folder) / "config.json").read_text())["model_type"]


def load_exported(folder, implementation: str = "eager"):
    """The folder as a causal LM in float32; every weight of the checkpoint must find its
    place (transformers would only warn and draw the missing ones at random)."""
    folder = Path(folder)
    if kind_of(folder) == "bux":
        from .hf.modeling_bux import BuxForCausalLM

        return BuxForCausalLM.from_pretrained(folder)
    from transformers import AutoModelForCausalLM

    model, info = AutoModelForCausalLM.from_pretrained(folder, dtype=torch.float32, attn_implementation=implementation,
                                                       output_loading_info=True)
    unmatched = {k: v for k, v in info.items() if k != "error_msgs" and v}
    assert not unmatched, f"weights without a match: {unmatched}"
    return model.eval()


def _own_heads(model, ids) -> list:
    pos = torch.arange(ids.shape[1]).expand_as(ids)
    return [h.logits().float() for h in model(ids, pos, None, training=False).heads]


def _own_greedy(model, prompt, steps: int) -> list:
    ids = prompt.clone()
    for _ in range(steps):
        nxt = _own_heads(model, ids)[0][:, -1].argmax(-1, keepdim=True)
        ids = torch.cat([ids, nxt], dim=1)
    return ids[0].tolist()


def _generate(hf, ids, mask, steps: int, cache: bool = True):
    return hf.generate(ids, attention_mask=mask, max_new_tokens=steps, do_sample=False, use_cache=cache,
                       eos_token_id=None, pad_token_id=0)


def _padded(hf, tokens, length: int, steps: int) -> bool:
    short = max(length // 2, 1)
    rows = [tokens[0, :length], tokens[1 % len(tokens), :short]]
    ids = torch.zeros(2, length, dtype=torch.long)
    mask = torch.zeros(2, length, dtype=torch.long)
    for i, row in enumerate(rows):
        ids[i, length - len(row):], mask[i, length - len(row):] = row, 1
    both = _generate(hf, ids, mask, steps)
    for i, row in enumerate(rows):
        alone = _generate(hf, row[None], torch.ones(1, len(row), dtype=torch.long), steps)
        if both[i, length:].tolist() != alone[0, len(row):].tolist():
            return False
    return True


@torch.no_grad()
def compare(model, folder, *, implementations=None, rows: int = 2, tokens: int = 12, steps: int = 6,
            tolerance: float = None, seed: int = 0) -> Report:
    """Compare the trained `model` (float32, evaluation mode) with the export at `folder`."""
    model.eval()
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, model.arch.vocab_size, (rows, tokens), generator=g)
    want = _own_heads(model, ids)
    prompt = ids[:1, : tokens // 2]
    greedy = _own_greedy(model, prompt, steps)
    native = kind_of(folder) != "bux"
    stored = json.loads((Path(folder) / "config.json").read_text()).get("torch_dtype") or \
        json.loads((Path(folder) / "config.json").read_text()).get("dtype") or "float32"
    if tolerance is None:   # a folder stored in 16 bits cannot agree to float32's last digits
        tolerance = 1e-4 if str(stored) == "float32" else 3e-2
    report = Report(tolerance=tolerance, logit_scale=max(float(w.abs().max()) for w in want),
                    exact=str(stored) == "float32")
    for impl in implementations or (("eager", "sdpa") if native else ("bux",)):
        hf = load_exported(folder, impl)
        got = [hf(input_ids=ids).logits.float()] if native else hf(ids, all_heads=True)
        pairs = list(zip(got, want))   # a standard family has the first head only
        error = max(float((a - b).abs().max()) / max(float(b.abs().max()), 1e-6) for a, b in pairs)
        agree = min(float((a.argmax(-1) == b.argmax(-1)).float().mean()) for a, b in pairs)
        ones = torch.ones_like(prompt)
        runs = {"cache": _generate(hf, prompt, ones, steps, True)[0].tolist(),
                "no cache": _generate(hf, prompt, ones, steps, False)[0].tolist(), "bux": greedy}
        report.results.append(Result(impl, error, agree, runs, _padded(hf, ids, tokens // 2, steps)))
    return report
