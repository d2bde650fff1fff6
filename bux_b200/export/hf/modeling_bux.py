"""``BuxForCausalLM``: an exported bux model as a Hugging Face causal LM.

The graph is rebuilt from ``config.bux`` (the architecture's IR) by the ``bux_b200``
package, which must be importable; weights load from ``model.safetensors`` under the
exported names (every projection on its own) and are fused back on load."""

import torch
from transformers import PreTrainedModel
from transformers.modeling_outputs import CausalLMOutput

try:
    from .configuration_bux import BuxConfig
except ImportError:  # loaded as a loose file by trust_remote_code
    from configuration_bux import BuxConfig


class BuxForCausalLM(PreTrainedModel):
    config_class = BuxConfig
    base_model_prefix = "model"
    supports_gradient_checkpointing = False

    def __init__(self, config: BuxConfig):
        super().__init__(config)
        from bux_b200.lang import ir
        from bux_b200.models import Model

        arch = ir.Architecture.model_validate(config.bux["architecture"])
        dtype = getattr(torch, str(config.bux.get("dtype", "float32")))
        self.model = Model(arch, dtype=dtype)

    def _init_weights(self, module):  # weights always come from the checkpoint
        pass

    @classmethod
    def from_pretrained(cls, path, *args, **kwargs):
        from pathlib import Path

        from safetensors.torch import load_file

        from bux_b200.export import weights as W

        config = BuxConfig.from_pretrained(path)
        self = cls(config)
        exported = load_file(str(Path(path) / "model.safetensors"))
        exported = {k.removeprefix("model."): v for k, v in exported.items()}
        state = W.fused(self.model, exported)
        own = self.model.state_dict()
        self.model.load_state_dict({k: v.to(own[k].dtype) for k, v in state.items() if k in own}, strict=False)
        return self.eval()

    def forward(self, input_ids, position_ids=None, labels=None, **kwargs):
        if position_ids is None:
            position_ids = torch.arange(input_ids.shape[1], device=input_ids.device).expand_as(input_ids)
        ctx = self.model(input_ids, position_ids, None, training=False)
        logits = ctx.heads[0].logits().float()
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]),
                                                     labels[:, 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutput(loss=loss, logits=logits)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 16, **kwargs):
        """Greedy decoding by whole-sequence passes (no cache): for checks, not serving."""
        for _ in range(max_new_tokens):
            nxt = self(input_ids).logits[:, -1].argmax(-1, keepdim=True)
            input_ids = torch.cat([input_ids, nxt], dim=1)
        return input_ids
