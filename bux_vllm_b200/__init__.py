"""bux exports in vLLM.

A checkpoint that `bux_b200.export` wrote in a standard family's format (llama, mistral,
qwen2, qwen3, mixtral, qwen3_moe) needs nothing from here: vLLM serves it as that family. This plugin is for
folders in the ``bux`` format (``model_type: "bux"``, the architecture carried as its
IR): it registers the config with transformers and ``BuxForCausalLM`` with vLLM, a model
that recognises which of vLLM's own decoder implementations the IR describes, builds
that one (paged attention, fused MoE, tensor parallelism all vLLM's), and renames the
exported tensors into it while loading. Graphs outside those families are refused with
the list of layers that have no served counterpart.

vLLM loads the plugin through the ``vllm.general_plugins`` entry point (`register`).
Reference: ``src/bux_vllm/__init__.py:17``, ``src/bux_vllm/model.py:421``.
"""


def register() -> None:
    from transformers import AutoConfig
    from vllm import ModelRegistry

    from .config import BuxConfig

    try:
        AutoConfig.register("bux", BuxConfig, exist_ok=True)
    except TypeError:  # older transformers: no exist_ok
        try:
            AutoConfig.register("bux", BuxConfig)
        except ValueError:
            pass
    ModelRegistry.register_model("BuxForCausalLM", "bux_vllm_b200.model:BuxForCausalLM")
