"""``BuxForCausalLM``: an exported bux model as a Hugging Face causal LM.

The folder is self-contained: beside this file the exporter writes ``bux_runtime/``, a copy
of the framework's Python sources (the language's IR, the layer schemas, every layer in
plain PyTorch, the weight-name mapping), so loading needs torch, transformers and
safetensors only. Where the ``bux_b200`` package itself is installed it is used instead
(its sm_100a kernels then run on a B200). The graph is rebuilt from ``config.bux`` (the
architecture's IR); weights load from ``model.safetensors`` under the exported names (every
projection on its own) and are fused back on load."""

import importlib
import sys
from pathlib import Path

import torch
from transformers import PreTrainedModel
from transformers.modeling_outputs import CausalLMOutput

try:
    from .configuration_bux import BuxConfig
except ImportError:  # loaded as a loose file by trust_remote_code
    from configuration_bux import BuxConfig


def runtime(folder=None):
    """The package that builds the model: the installed ``bux_b200`` when there is one, else
    the ``bux_runtime`` copy that sits in the exported folder (kernels off: plain PyTorch)."""
    try:
        return importlib.import_module("bux_b200")
    except ImportError:
        pass
    for place in (folder, Path(__file__).resolve().parent):
        if place is not None and (Path(place) / "bux_runtime" / "__init__.py").exists():
            if str(place) not in sys.path:
                sys.path.insert(0, str(place))
            rt = importlib.import_module("bux_runtime")
            importlib.import_module("bux_runtime.ops.functional").set_kernels(False)
            return rt
    raise ImportError("neither the bux_b200 package nor the exported folder's bux_runtime copy was found")


class BuxForCausalLM(PreTrainedModel):
    config_class = BuxConfig
    base_model_prefix = "model"
    supports_gradient_checkpointing = False

    def __init__(self, config: BuxConfig):
        super().__init__(config)
        rt = runtime(getattr(config, "_name_or_path", None) or None)
        ir = importlib.import_module(rt.__name__ + ".lang.ir")
        models = importlib.import_module(rt.__name__ + ".models")
        arch = ir.Architecture.model_validate(config.bux["architecture"])
        dtype = getattr(torch, str(config.bux.get("dtype", "float32")))
        self.model = models.Model(arch, dtype=dtype)

    def _init_weights(self, module):  # weights always come from the checkpoint
        pass

    @classmethod
    def from_pretrained(cls, path, *args, **kwargs):
        from safetensors.torch import load_file

        rt = runtime(path)
        W = importlib.import_module(rt.__name__ + ".export.weights")
        config = BuxConfig.from_pretrained(path)
        config._name_or_path = str(path)
        self = cls(config)
        exported = load_file(str(Path(path) / "model.safetensors"))
        exported = {k.removeprefix("model."): v for k, v in exported.items()}
        state = W.fused(self.model, exported)
        own = self.model.state_dict()
        self.model.load_state_dict({k: v.to(own[k].dtype) for k, v in state.items() if k in own}, strict=False)
        return self.eval()

    @staticmethod
    def _placed(input_ids, attention_mask, position_ids):
        """Positions and document ids of a (possibly left-padded) batch: positions count the
        real tokens of a row from 0; padding is a document of its own that nothing real attends."""
        if attention_mask is None:
            if position_ids is None:
                position_ids = torch.arange(input_ids.shape[1], device=input_ids.device).expand_as(input_ids)
            return position_ids, None
        mask = attention_mask.to(torch.long)
        if position_ids is None:
            position_ids = (mask.cumsum(-1) - 1).clamp_min(0)
        return position_ids, (None if bool(mask.all()) else mask.to(torch.int32))

    def forward(self, input_ids, attention_mask=None, position_ids=None, labels=None, all_heads=False, **kwargs):
        position_ids, segments = self._placed(input_ids, attention_mask, position_ids)
        ctx = self.model(input_ids, position_ids, segments, training=False)
        if all_heads:   # every head of the graph (multi-token-prediction heads after the first)
            return [h.logits().float() for h in ctx.heads]
        logits = ctx.heads[0].logits().float()
        loss = None
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]),
                                                     labels[:, 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutput(loss=loss, logits=logits)

    @staticmethod
    def _next(logits, do_sample: bool, temperature: float, top_k, top_p, generator):
        """The next token of each row from its last position's logits: the largest, or a draw
        after temperature, top-k and nucleus (top-p) filtering."""
        if not do_sample:
            return logits.argmax(-1, keepdim=True)
        logits = logits / max(float(temperature), 1e-6)
        if top_k:
            kth = logits.topk(min(int(top_k), logits.shape[-1]), dim=-1).values[..., -1:]
            logits = logits.masked_fill(logits < kth, float("-inf"))
        if top_p is not None and top_p < 1.0:
            ordered, order = logits.sort(dim=-1, descending=True)
            mass = ordered.softmax(-1).cumsum(-1)
            drop = mass - ordered.softmax(-1) >= top_p          # keep the token that crosses top_p
            logits = logits.masked_fill(drop.scatter(-1, order, drop), float("-inf"))
        return torch.multinomial(logits.softmax(-1), 1, generator=generator)

    @torch.no_grad()
    def generate(self, input_ids, attention_mask=None, max_new_tokens: int = 16, use_cache: bool = True,
                 do_sample: bool = False, temperature: float = 1.0, top_k=None, top_p=None, eos_token_id=None,
                 pad_token_id=None, generator=None, **kwargs):
        """Decode `max_new_tokens` tokens: greedily, or by sampling (`do_sample`, `temperature`,
        `top_k`, `top_p`, `generator`). With `use_cache` (and a graph `models.cache` can carry
        between tokens) the prompt runs once and every new token alone; otherwise every step is a
        pass over the whole sequence. Rows may be left-padded (`attention_mask`); a row that has
        produced `eos_token_id` is filled with `pad_token_id` from then on. For checks and light
        generation: serving goes through vLLM."""
        rt = runtime(getattr(self.config, "_name_or_path", None) or None)
        caching = importlib.import_module(rt.__name__ + ".models.cache")
        cached = use_cache and caching.supports(self.model.arch) is None
        mask = torch.ones_like(input_ids) if attention_mask is None else attention_mask.to(input_ids.dtype)
        positions = (mask.cumsum(-1) - 1).clamp_min(0)
        done = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        fill = pad_token_id if pad_token_id is not None else (eos_token_id if eos_token_id is not None else 0)
        cache = caching.DecodeCache() if cached else None
        new, new_positions, new_mask = input_ids, positions, mask
        for _ in range(max_new_tokens):
            if cached:
                ctx = self.model(new, new_positions, new_mask.to(torch.int32), training=False, cache=cache)
                last = ctx.heads[0].logits()[:, -1].float()
            else:
                last = self(input_ids, attention_mask=mask).logits[:, -1]
            nxt = self._next(last, do_sample, temperature, top_k, top_p, generator)
            if eos_token_id is not None:
                nxt = torch.where(done.unsqueeze(-1), torch.full_like(nxt, fill), nxt)
                done = done | (nxt.squeeze(-1) == eos_token_id)
            input_ids = torch.cat([input_ids, nxt], dim=1)
            mask = torch.cat([mask, torch.ones_like(mask[:, :1])], dim=1)
            new, new_positions, new_mask = nxt, positions[:, -1:] + 1, torch.ones_like(nxt)
            positions = torch.cat([positions, new_positions], dim=1)
            if eos_token_id is not None and bool(done.all()):
                break
        return input_ids
