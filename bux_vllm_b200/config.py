"""The Hugging Face config of ``model_type: "bux"`` (a copy of the exported
``configuration_bux.py``: the plugin runs in vLLM's environment, without the export)."""

from transformers import PretrainedConfig


class BuxConfig(PretrainedConfig):
    model_type = "bux"

    def __init__(self, bux=None, vocab_size=None, hidden_size=None, num_hidden_layers=None,
                 layer_types=None, bux_layer_types=None, tie_word_embeddings=False, **kwargs):
        self.bux = bux or {}
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.num_hidden_layers = num_hidden_layers
        self.layer_types = layer_types or []
        self.bux_layer_types = bux_layer_types or []
        super().__init__(tie_word_embeddings=tie_word_embeddings, **kwargs)
