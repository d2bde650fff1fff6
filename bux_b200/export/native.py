"""Standard decoder families: when an architecture is exactly one of them, the export is
written in that family's own Hugging Face format (config fields and tensor names), so
stock `transformers` and stock vLLM load and serve it with their own kernels.

Families: ``llama`` (pre-norm GQA + SwiGLU), ``mistral`` (llama with one sliding window for
every layer), ``qwen2`` (llama with biases on q, k and v), ``qwen3`` (llama with per-head q/k
RMSNorm), ``mixtral`` (llama with softmax top-k routed SwiGLU experts, the picked weights
renormalised) and ``qwen3_moe`` (the same on qwen3's attention). RoPE scalings (``pi``,
``llama3``, ``yarn``) are written as the family's ``rope_parameters``.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..config import layers as L
from ..lang import ir

MIXERS = ("gqa", "mla", "csa", "gla", "deltanet", "gdn", "kda", "gdn2", "lightning", "rwkv7", "mamba", "mamba2",
          "conv", "short_conv")


def _block_parts(block) -> Optional[tuple]:
    """(norm, gqa, norm, ffn) configs of a ``[norm attn] [norm ffn]`` block, else None."""
    if not isinstance(block, ir.Seq) or len(block.items) != 2:
        return None
    out = []
    for br in block.items:
        if not isinstance(br, ir.Residual) or not isinstance(br.body, ir.Seq) or len(br.body.items) != 2:
            return None
        a, b = br.body.items
        if not (isinstance(a, ir.Layer) and isinstance(b, ir.Layer)):
            return None
        out += [a.config, b.config]
    return tuple(out)


def _plain_norm(c) -> bool:
    return (isinstance(c, L.NormalizationConfig) and c.type == "rmsnorm" and c.affine and not c.bias
            and not c.zero_centered and not c.scale_input)


def detect(arch: ir.Architecture) -> Optional[str]:
    if arch.residual is not None:
        return None
    g = arch.graph
    if not isinstance(g, ir.Seq) or len(g.items) != 4:
        return None
    emb, rep, norm, head = g.items
    if not (isinstance(emb, ir.Layer) and emb.config.type == "embed" and isinstance(rep, ir.Repeat)
            and isinstance(norm, ir.Layer) and _plain_norm(norm.config)
            and isinstance(head, ir.Layer) and head.config.type == "head"):
        return None
    e = emb.config
    if (e.max_positions is not None or e.scale_by_sqrt_dim or e.norm is not None or head.config.softcap
            or head.config.bias or head.config.pointer is not None):
        return None
    parts = _block_parts(rep.body)
    if parts is None or rep.body.share is not None:
        return None
    n1, attn, n2, ffn = parts
    if not (_plain_norm(n1) and _plain_norm(n2) and isinstance(attn, L.GQAConfig)):
        return None
    a = attn
    plain = (a.rope is not None and a.rope.layout == "half" and a.rope.fraction == 1.0
             and not a.sinks and not a.gated and a.softcap is None
             and not (a.bias if a.output_bias is None else a.output_bias)   # no family here biases the output projection
             and a.scale is None and a.output_norm is None and not a.qk_norm_all_heads
             and all(getattr(a, f) in (None, False) for f in ("kv_conv_size", "differential", "k_eq_v", "indexer")))
    # every other setting of the layer changes what it computes: only its defaults are a standard family
    allowed = {"type", "num_heads", "num_kv_heads", "head_dim", "v_head_dim", "rope", "qk_norm", "fused_qkv",
               "value_residual", "value_embed_gate", "bias", "output_bias", "sliding_window_size"}
    plain = plain and all(getattr(a, name) == field.default for name, field in type(a).model_fields.items()
                          if name not in allowed and not field.is_required())
    if not plain:
        return None
    qk = a.qk_norm is not None and _plain_norm(a.qk_norm)
    if a.qk_norm is not None and not qk:
        return None
    # one variation at a time is a family; two at once (a window and biases, ...) is none of them
    variations = [bool(a.bias), a.sliding_window_size is not None, qk]
    if sum(variations) > 1 or (a.v_head_dim not in (None, a.head_dim or arch.d_model // a.num_heads)):
        return None
    if isinstance(a.rope.scaling, L.YaRNConfig) and a.rope.scaling.attention_factor_on != "rotary":
        return None
    if isinstance(ffn, L.MLPConfig):
        ok = (ffn.type == "gated_mlp" and ffn.activation == "swish" and not ffn.bias and ffn.limit is None
              and not ffn.up_offset and ffn.up_softcap is None)
        if not ok:
            return None
        return "qwen3" if qk else "qwen2" if a.bias else "mistral" if a.sliding_window_size is not None else "llama"
    if isinstance(ffn, L.MoEConfig) and not a.bias and a.sliding_window_size is None:
        x = ffn.expert
        ok = (ffn.router == "softmax" and not ffn.num_shared_experts and ffn.num_groups == 1
              and not ffn.router_bias and ffn.load_balancing not in ("aux_free", "smebu")
              and ffn.routed_scaling_factor == 1.0 and ffn.router_logit_scale == 1.0
              and x.type == "gated_mlp" and x.activation == "swish" and x.limit is None and not x.up_offset
              and not x.bias and x.up_softcap is None)
        # what the family's format can say, or what only training uses; anything else off its default is not the family
        allowed = {"type", "num_experts", "top_k", "expert", "normalize_top_k", "aux_loss_coef", "aux_loss_scope",
                   "random_logits", "load_balancing", "bias_update_rate", "bias_softclamp", "bias_momentum"}
        ok = ok and all(getattr(ffn, name) == field.default for name, field in type(ffn).model_fields.items()
                        if name not in allowed and not field.is_required())
        if not ok:
            return None
        if qk:
            return "qwen3_moe"
        return "mixtral" if ffn.normalize_top_k else None      # Mixtral always renormalises the picked weights
    return None


def rope_parameters(rope) -> dict:
    """A RoPE config in the families' ``rope_parameters`` form."""
    out = {"rope_type": "default", "rope_theta": rope.base}
    sc = rope.scaling
    if isinstance(sc, L.PositionInterpolationConfig):
        out.update(rope_type="linear", factor=sc.factor)
    elif isinstance(sc, L.Llama3RoPEScalingConfig):
        out.update(rope_type="llama3", factor=sc.factor, original_max_position_embeddings=sc.original_max_len,
                   low_freq_factor=sc.low_freq_factor, high_freq_factor=sc.high_freq_factor)
    elif isinstance(sc, L.YaRNConfig):
        out.update(rope_type="yarn", factor=sc.factor, original_max_position_embeddings=sc.original_max_len,
                   beta_fast=sc.beta_fast, beta_slow=sc.beta_slow)
        if sc.attention_factor is not None:
            out["attention_factor"] = sc.attention_factor
    return out


def convert(family: str, arch: ir.Architecture, t: dict, dtype) -> tuple:
    """(config.json dict, tensors under the family's names) from the exported tensors `t`."""
    emb, rep, norm, head = arch.graph.items
    n1, attn, n2, ffn = _block_parts(rep.body)
    d = arch.d_model
    hd = attn.head_dim or d // attn.num_heads
    layers = rep.times
    out = {"model.embed_tokens.weight": t["graph.items.0.tokens.embedding"],
           "model.norm.weight": t["graph.items.2.scale"]}
    tied = head.config.tied
    if not tied:
        out["lm_head.weight"] = t["graph.items.3.proj.weight"]
    for i in range(layers):
        src = f"graph.items.1.items.{i}.items"
        dst = f"model.layers.{i}"
        out[f"{dst}.input_layernorm.weight"] = t[f"{src}.0.body.items.0.scale"]
        out[f"{dst}.post_attention_layernorm.weight"] = t[f"{src}.1.body.items.0.scale"]
        at = f"{src}.0.body.items.1"
        for p in "qkvo":
            out[f"{dst}.self_attn.{p}_proj.weight"] = t[f"{at}.{p}.weight"]
        if family in ("qwen3", "qwen3_moe"):
            out[f"{dst}.self_attn.q_norm.weight"] = t[f"{at}.q_norm.scale"]
            out[f"{dst}.self_attn.k_norm.weight"] = t[f"{at}.k_norm.scale"]
        if family == "qwen2":
            for p in "qkv":
                out[f"{dst}.self_attn.{p}_proj.bias"] = t[f"{at}.{p}.bias"]
        ff = f"{src}.1.body.items.1"
        if family in ("qwen3_moe", "mixtral"):
            gate, up, down = t[f"{ff}.experts.gate"], t[f"{ff}.experts.up"], t[f"{ff}.experts.down"]
            moe = f"{dst}.mlp" if family == "qwen3_moe" else f"{dst}.block_sparse_moe"
            names = ("gate_proj", "up_proj", "down_proj") if family == "qwen3_moe" else ("w1", "w3", "w2")
            out[f"{moe}.gate.weight"] = t[f"{ff}.router.weight"]
            for e in range(gate.shape[0]):
                for name, w in zip(names, (gate, up, down)):
                    out[f"{moe}.experts.{e}.{name}.weight"] = w[e]
        else:
            for p in ("gate", "up", "down"):
                out[f"{dst}.mlp.{p}_proj.weight"] = t[f"{ff}.{p}.weight"]
    cfg = {
        "vocab_size": arch.vocab_size, "hidden_size": d, "num_hidden_layers": layers,
        "num_attention_heads": attn.num_heads, "num_key_value_heads": attn.num_kv_heads, "head_dim": hd,
        "rms_norm_eps": n1.eps, "rope_theta": attn.rope.base, "hidden_act": "silu", "attention_bias": False,
        "attention_dropout": 0.0, "max_position_embeddings": 131072, "tie_word_embeddings": bool(tied),
        "torch_dtype": str(dtype).removeprefix("torch."), "use_cache": True,
        "rope_parameters": rope_parameters(attn.rope),
    }
    if attn.rope.scaling is not None:
        cfg["rope_scaling"] = {k: v for k, v in cfg["rope_parameters"].items() if k != "rope_theta"}   # the older key
    if family == "llama":
        cfg.update(model_type="llama", architectures=["LlamaForCausalLM"], intermediate_size=ffn.intermediate_size,
                   mlp_bias=False)
    elif family == "mistral":
        cfg.update(model_type="mistral", architectures=["MistralForCausalLM"], intermediate_size=ffn.intermediate_size,
                   sliding_window=attn.sliding_window_size)
    elif family == "qwen2":
        cfg.update(model_type="qwen2", architectures=["Qwen2ForCausalLM"], intermediate_size=ffn.intermediate_size,
                   use_sliding_window=False, sliding_window=None)
    elif family == "mixtral":
        cfg.update(model_type="mixtral", architectures=["MixtralForCausalLM"], intermediate_size=ffn.expert.intermediate_size,
                   num_local_experts=ffn.num_experts, num_experts_per_tok=ffn.top_k, sliding_window=None,
                   output_router_logits=False, router_aux_loss_coef=ffn.aux_loss_coef or 0.0, router_jitter_noise=0.0)
    elif family == "qwen3":
        cfg.update(model_type="qwen3", architectures=["Qwen3ForCausalLM"], intermediate_size=ffn.intermediate_size)
    else:
        cfg.update(model_type="qwen3_moe", architectures=["Qwen3MoeForCausalLM"],
                   intermediate_size=ffn.expert.intermediate_size, moe_intermediate_size=ffn.expert.intermediate_size,
                   num_experts=ffn.num_experts, num_experts_per_tok=ffn.top_k, norm_topk_prob=bool(ffn.normalize_top_k),
                   decoder_sparse_step=1, mlp_only_layers=[], output_router_logits=False,
                   router_aux_loss_coef=getattr(ffn, "aux_loss_coef", 0.0) or 0.0)
    return cfg, {k: v.to(dtype) if v.is_floating_point() else v for k, v in out.items()}
