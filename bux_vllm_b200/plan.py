"""IR → a served family: which of vLLM's decoders an exported architecture is, the
family's config fields, and the renaming of exported tensor names into the family's.
Pure Python over the JSON of ``config.bux["architecture"]`` (no bux import)."""

from __future__ import annotations

import re
from typing import Iterator, Optional

FAMILIES = {"llama": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM"}


def _layer(node, kind=None):
    return node.get("kind") == "layer" and (kind is None or node["config"]["type"] == kind)


def _plain_norm(c) -> bool:
    return (c["type"] == "rmsnorm" and c.get("affine", True) and not c.get("bias") and not c.get("zero_centered")
            and not c.get("scale_input"))


def parts(arch: dict) -> Optional[dict]:
    """{"attn", "ffn", "norm", "layers", "tied"} of an ``embed ([norm attn] [norm ffn])^n norm head`` graph."""
    g = arch["graph"]
    if arch.get("residual") is not None or g.get("kind") != "seq" or len(g["items"]) != 4:
        return None
    emb, rep, norm, head = g["items"]
    if not (_layer(emb, "embed") and rep.get("kind") == "repeat" and _layer(norm) and _layer(head, "head")):
        return None
    body = rep["body"]
    if body.get("kind") != "seq" or len(body["items"]) != 2:
        return None
    found = []
    for br in body["items"]:
        if br.get("kind") != "residual" or br["body"].get("kind") != "seq" or len(br["body"]["items"]) != 2:
            return None
        a, b = br["body"]["items"]
        if not (_layer(a) and _layer(b) and _plain_norm(a["config"])):
            return None
        found.append(b["config"])
    if not _plain_norm(norm["config"]):
        return None
    return {"attn": found[0], "ffn": found[1], "norm": norm["config"], "layers": rep["times"],
            "tied": bool(head["config"].get("tied")), "embed": emb["config"], "head": head["config"]}


def family(arch: dict) -> tuple:
    """(family or None, why not)."""
    p = parts(arch)
    if p is None:
        return None, "the graph is not embed ([norm attn] [norm ffn])^n norm head"
    a, f = p["attn"], p["ffn"]
    if a["type"] != "gqa":
        return None, f"token mixer '{a['type']}' has no served counterpart in this plugin"
    rope = a.get("rope")
    odd = [k for k in ("sinks", "gated", "softcap", "sliding_window_size", "bias", "scale", "output_norm",
                       "differential", "k_eq_v", "indexer", "kv_conv_size") if a.get(k)]
    if rope is None or rope.get("layout", "half") != "half" or rope.get("fraction", 1.0) != 1.0 or rope.get("scaling"):
        odd.append("rope")
    if odd:
        return None, f"gqa settings without a served counterpart: {', '.join(odd)}"
    qk = a.get("qk_norm") is not None
    if f["type"] == "gated_mlp" and f.get("activation") == "swish" and not f.get("bias"):
        return ("qwen3" if qk else "llama"), ""
    if f["type"] == "moe" and qk and f.get("router", "softmax") == "softmax" and not f.get("num_shared_experts"):
        return "qwen3_moe", ""
    return None, f"feed-forward '{f['type']}' has no served counterpart in this plugin"


def hf_fields(arch: dict, fam: str) -> dict:
    p = parts(arch)
    a, f = p["attn"], p["ffn"]
    d = arch["d_model"]
    out = {
        "vocab_size": arch["vocab_size"], "hidden_size": d, "num_hidden_layers": p["layers"],
        "num_attention_heads": a["num_heads"], "num_key_value_heads": a["num_kv_heads"],
        "head_dim": a.get("head_dim") or d // a["num_heads"], "rms_norm_eps": p["norm"].get("eps", 1e-6),
        "rope_theta": a["rope"].get("base", 10000.0), "hidden_act": "silu", "attention_bias": False,
        "max_position_embeddings": 131072, "tie_word_embeddings": p["tied"],
    }
    if fam == "qwen3_moe":
        x = f["expert"]
        out.update(intermediate_size=x["intermediate_size"], moe_intermediate_size=x["intermediate_size"],
                   num_experts=f["num_experts"], num_experts_per_tok=f["top_k"],
                   norm_topk_prob=bool(f.get("normalize_top_k", True)), decoder_sparse_step=1, mlp_only_layers=[])
    else:
        out.update(intermediate_size=f["intermediate_size"])
    return out


_BLOCK = re.compile(r"^model\.graph\.items\.1\.items\.(\d+)\.items\.(\d)\.body\.items\.(\d)\.(.+)$")


def rename(name: str, tensor, fam: str) -> Iterator:
    """Exported (name, tensor) → the family's (name, tensor) pairs (stacked experts fan out)."""
    if name == "model.graph.items.0.tokens.embedding":
        yield "model.embed_tokens.weight", tensor
        return
    if name == "model.graph.items.2.scale":
        yield "model.norm.weight", tensor
        return
    if name == "model.graph.items.3.proj.weight":
        yield "lm_head.weight", tensor
        return
    m = _BLOCK.match(name)
    if m is None:
        return
    i, branch, item, leaf = int(m[1]), int(m[2]), int(m[3]), m[4]
    pre = f"model.layers.{i}"
    if item == 0 and leaf == "scale":
        yield f"{pre}.{'input_layernorm' if branch == 0 else 'post_attention_layernorm'}.weight", tensor
    elif branch == 0:
        if leaf in ("q.weight", "k.weight", "v.weight", "o.weight"):
            yield f"{pre}.self_attn.{leaf[0]}_proj.weight", tensor
        elif leaf in ("q_norm.scale", "k_norm.scale"):
            yield f"{pre}.self_attn.{leaf[:6]}.weight", tensor
    elif leaf in ("gate.weight", "up.weight", "down.weight"):
        yield f"{pre}.mlp.{leaf.split('.')[0]}_proj.weight", tensor
    elif leaf == "router.weight":
        yield f"{pre}.mlp.gate.weight", tensor
    elif leaf in ("experts.gate", "experts.up", "experts.down"):
        which = leaf.split(".")[1]
        for e in range(tensor.shape[0]):
            yield f"{pre}.mlp.experts.{e}.{which}_proj.weight", tensor[e]
