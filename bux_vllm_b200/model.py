"""``BuxForCausalLM`` for vLLM: builds the vLLM decoder the exported IR describes and
loads the exported tensors into it under that decoder's names."""

from __future__ import annotations

import copy
import importlib
from typing import Iterable

import torch
from torch import nn

from . import plan

# family → (vLLM's module, its class, transformers' config class): the modules vLLM's own registry names
_MODULES = {"llama": ("vllm.model_executor.models.llama", "LlamaForCausalLM", "LlamaConfig"),
            "mistral": ("vllm.model_executor.models.mistral", "MistralForCausalLM", "MistralConfig"),
            "qwen2": ("vllm.model_executor.models.qwen2", "Qwen2ForCausalLM", "Qwen2Config"),
            "qwen3": ("vllm.model_executor.models.qwen3", "Qwen3ForCausalLM", "Qwen3Config"),
            "mixtral": ("vllm.model_executor.models.mixtral", "MixtralForCausalLM", "MixtralConfig"),
            "qwen3_moe": ("vllm.model_executor.models.qwen3_moe", "Qwen3MoeForCausalLM", "Qwen3MoeConfig")}


class BuxForCausalLM(nn.Module):
    def __init__(self, *, vllm_config, prefix: str = ""):
        super().__init__()
        import transformers

        hf = vllm_config.model_config.hf_config
        arch = hf.bux["architecture"]
        fam, why = plan.family(arch)
        if fam is None:
            raise NotImplementedError(f"bux_vllm_b200 cannot serve this architecture: {why}. Export it with "
                                      f"`bux export` in a standard family's format, or serve it with transformers.")
        module, cls, cfg_cls = _MODULES[fam]
        config = getattr(transformers, cfg_cls)(**plan.hf_fields(arch, fam))
        config.architectures = [cls]
        if getattr(hf, "torch_dtype", None) is not None:
            config.torch_dtype = hf.torch_dtype
        inner_cfg = copy.copy(vllm_config)
        inner_cfg.model_config = copy.copy(vllm_config.model_config)
        inner_cfg.model_config.hf_config = config
        if hasattr(inner_cfg.model_config, "hf_text_config"):
            inner_cfg.model_config.hf_text_config = config
        self.family = fam
        self.inner = getattr(importlib.import_module(module), cls)(vllm_config=inner_cfg, prefix=prefix)
        for name in ("packed_modules_mapping", "supported_lora_modules", "embedding_modules"):
            if hasattr(self.inner, name):
                setattr(self, name, getattr(self.inner, name))

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            inner = self._modules.get("inner")
            if inner is not None and name != "inner":
                return getattr(inner, name)
            raise

    def forward(self, input_ids, positions, *args, **kwargs):
        return self.inner(input_ids, positions, *args, **kwargs)

    def embed_input_ids(self, input_ids, *args, **kwargs):
        """Token embeddings (vLLM's model interface; older releases call it `get_input_embeddings`)."""
        fn = getattr(self.inner, "embed_input_ids", None) or self.inner.get_input_embeddings
        return fn(input_ids, *args, **kwargs)

    def get_input_embeddings(self, input_ids, *args, **kwargs):
        return self.embed_input_ids(input_ids, *args, **kwargs)

    def compute_logits(self, *args, **kwargs):
        return self.inner.compute_logits(*args, **kwargs)

    def load_weights(self, weights: Iterable) -> set:
        def renamed():
            for name, tensor in weights:
                yield from plan.rename(name, tensor, self.family)

        loaded = self.inner.load_weights(renamed())
        return {f"inner.{n}" for n in loaded} if loaded is not None else None
