"""IR → a served family: which of vLLM's decoders an exported architecture is, the
family's config fields, and the renaming of exported tensor names into the family's.
Pure Python over the JSON of ``config.bux["architecture"]`` (no bux import)."""

from __future__ import annotations

import re
from typing import Iterator, Optional

FAMILIES = {"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "qwen2": "Qwen2ForCausalLM",
            "qwen3": "Qwen3ForCausalLM", "mixtral": "MixtralForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM"}


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
    out_bias = a.get("bias") if a.get("output_bias") is None else a.get("output_bias")
    odd = [k for k in ("sinks", "gated", "softcap", "scale", "output_norm", "differential", "k_eq_v", "indexer",
                       "kv_conv_size", "paired", "exclusive", "power_scale", "log_scale", "relative_bias") if a.get(k)]
    if out_bias:
        odd.append("output_bias")
    if rope is None or rope.get("layout", "half") != "half" or rope.get("fraction", 1.0) != 1.0:
        odd.append("rope")
    elif (rope.get("scaling") or {}).get("attention_factor_on", "rotary") != "rotary":
        odd.append("rope.scaling.attention_factor_on")
    if odd:
        return None, f"gqa settings without a served counterpart: {', '.join(odd)}"
    qk = a.get("qk_norm") is not None
    window, bias = a.get("sliding_window_size") is not None, bool(a.get("bias"))
    if sum((qk, window, bias)) > 1:
        return None, "more than one of qk_norm, sliding_window_size and bias: no served family has both"
    if f["type"] == "gated_mlp" and f.get("activation") == "swish" and not f.get("bias"):
        return ("qwen3" if qk else "qwen2" if bias else "mistral" if window else "llama"), ""
    if (f["type"] == "moe" and not window and not bias and f.get("router", "softmax") == "softmax"
            and not f.get("num_shared_experts")):
        if qk:
            return "qwen3_moe", ""
        if f.get("normalize_top_k", True):
            return "mixtral", ""
        return None, "Mixtral renormalises the picked weights: normalize_top_k=false has no served counterpart"
    return None, f"feed-forward '{f['type']}' has no served counterpart in this plugin"


def rope_parameters(rope: dict) -> dict:
    out = {"rope_type": "default", "rope_theta": rope.get("base", 10000.0)}
    sc = rope.get("scaling")
    if not sc:
        return out
    if sc["type"] == "pi":
        out.update(rope_type="linear", factor=sc["factor"])
    elif sc["type"] == "llama3":
        out.update(rope_type="llama3", factor=sc["factor"], original_max_position_embeddings=sc.get("original_max_len", 8192),
                   low_freq_factor=sc.get("low_freq_factor", 1.0), high_freq_factor=sc.get("high_freq_factor", 4.0))
    else:
        out.update(rope_type="yarn", factor=sc["factor"], original_max_position_embeddings=sc["original_max_len"],
                   beta_fast=sc.get("beta_fast", 32.0), beta_slow=sc.get("beta_slow", 1.0))
        if sc.get("attention_factor") is not None:
            out["attention_factor"] = sc["attention_factor"]
    return out


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
        "rope_parameters": rope_parameters(a["rope"]),
    }
    if a["rope"].get("scaling"):
        out["rope_scaling"] = {k: v for k, v in out["rope_parameters"].items() if k != "rope_theta"}
    if fam == "mistral":
        out["sliding_window"] = a["sliding_window_size"]
    if fam == "mixtral":
        x = f["expert"]
        out.update(intermediate_size=x["intermediate_size"], num_local_experts=f["num_experts"],
                   num_experts_per_tok=f["top_k"], sliding_window=None)
    elif fam == "qwen3_moe":
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
        elif leaf in ("q.bias", "k.bias", "v.bias"):
            yield f"{pre}.self_attn.{leaf[0]}_proj.bias", tensor
        elif leaf in ("q_norm.scale", "k_norm.scale"):
            yield f"{pre}.self_attn.{leaf[:6]}.weight", tensor
    elif leaf in ("gate.weight", "up.weight", "down.weight"):
        yield f"{pre}.mlp.{leaf.split('.')[0]}_proj.weight", tensor
    elif leaf == "router.weight":
        yield f"{pre}.{'block_sparse_moe' if fam == 'mixtral' else 'mlp'}.gate.weight", tensor
    elif leaf in ("experts.gate", "experts.up", "experts.down"):
        which = leaf.split(".")[1]
        for e in range(tensor.shape[0]):
            if fam == "mixtral":
                yield f"{pre}.block_sparse_moe.experts.{e}.{ {'gate': 'w1', 'up': 'w3', 'down': 'w2'}[which] }.weight", tensor[e]
            else:
                yield f"{pre}.mlp.experts.{e}.{which}_proj.weight", tensor[e]
