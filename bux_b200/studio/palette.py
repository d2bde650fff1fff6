"""The palette: every layer and activation the page can insert, with the text that is
inserted (required settings filled with a small sensible value, so the file still
compiles) and a note. The file's own definitions come first. Reference: ``studio/palette.py``."""

from __future__ import annotations

from typing import Optional

from ..config import layers as L
from ..lang import reference
from ..lang.lsp import features

GROUPS = {
    "Attention": ("gqa", "mla", "csa"),
    "Recurrent": ("gdn", "gdn2", "kda", "deltanet", "gla", "lightning", "rwkv7", "mamba", "mamba2"),
    "Feed-forward": ("gated_mlp", "mlp", "moe"),
    "Norms": ("rmsnorm", "layernorm", "dyt"),
    "Projections": ("linear", "scale", "conv", "short_conv", "dropout"),
    "Model ends": ("embed", "head", "nextn", "value_embed", "engram", "doc_copy"),
}
_FILLS = {"num_heads": "4", "num_kv_heads": "2", "head_dim": "64", "intermediate_size": "4 * d_model", "activation": "swish",
          "num_experts": "8", "top_k": "2", "expert": "gated_mlp(intermediate_size=d_model, activation=swish)",
          "features": "d_model", "state_size": "64", "size": "4", "rate": "0.1", "kv_lora_rank": "64", "qk_nope_head_dim": "32",
          "qk_rope_head_dim": "16", "v_head_dim": "32", "compress_ratio": "4", "table_size": "65536", "fn": "gelu"}


def insert_text(tag: str) -> str:
    cls = L.LAYERS[tag]
    need = [n for n, f in cls.model_fields.items() if n != "type" and f.is_required()]
    if not need:
        return tag
    return f"{tag}(" + ", ".join(f"{n}={_FILLS.get(n, '1')}" for n in need) + ")"


def palette(source: str = "", path: Optional[str] = None) -> list:
    groups = []
    if source:
        ix = features.Index(source, path)
        mine = [{"name": n, "insert": n, "note": ix.written(st)} for n, (st, _) in ix.names.items()
                if st.params is None and n not in features._TOP and (ix.leads_to(n) in L.LAYERS or ix.leads_to(n) is None)]
        if mine:
            groups.append({"group": "This file", "items": mine})
    for group, tags in GROUPS.items():
        groups.append({"group": group, "items": [{"name": t, "insert": insert_text(t), "note": reference.docs.SUMMARY.get(t, "")}
                                                 for t in tags]})
    groups.append({"group": "Activations", "items": [{"name": a, "insert": a, "note": "elementwise"} for a in L.ACTIVATIONS]})
    return groups
