"""Incremental decoding: the state a graph carries between tokens, kept between calls.

``Model(..., cache=DecodeCache())`` runs the given tokens as the continuation of what the
cache holds: every `gqa` and `mla` layer appends its new keys and values and attends over all of
them, the recurrent mixers (DeltaNet, Gated DeltaNet, GDN-2, KDA, GLA, Lightning, RWKV-7,
Mamba, Mamba-2) continue their state, causal convolutions keep their last inputs, everything else
runs per token as always. A prompt is one call, each decoded token one
more. Rows may be left-padded: the cache keeps which of its positions are real tokens, and
padding is never attended. `supports(arch)` says whether an architecture can decode this way
(and why not): layers that carry other state between tokens (compressed and sparse
attention, n-gram memory, the copy layers) and layers that read keys another layer
cached are run by whole-sequence passes instead. The attention here is the
plain PyTorch statement: it is for checks and light generation, not for serving.
Reference: the caches of ``export/hf/attention.py`` there.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..lang import ir

_PER_TOKEN = {"embed", "head", "rmsnorm", "layernorm", "dyt", "mlp", "gated_mlp", "moe", "linear", "act", "scale",
              "dropout", "value_embed", "merge"}
_CONTINUED = {"deltanet", "gdn", "gdn2", "kda", "gla", "lightning", "rwkv7", "mamba", "mamba2", "conv", "short_conv"}


def supports(arch: ir.Architecture) -> Optional[str]:
    """None when `arch` can decode with a `DecodeCache`, else the reason it cannot."""
    if arch.residual is not None:
        return f"the residual algebra '{arch.residual.type}' is not run incrementally here"
    for layer in ir.unrolled_layers(arch.graph):
        c = layer.config
        if c.type == "gqa":
            for what in ("paired", "indexer", "relative_bias", "kv_conv_size"):
                if getattr(c, what) not in (None, False):
                    return f"gqa({what}=...) needs more than cached keys and values"
            if any(p.name == "kv" and p.mode != "write" for p in layer.ports):
                return "a layer that reads another layer's keys and values (the kv port) has no cache of its own"
        elif c.type == "mla":
            if c.indexer is not None:
                return "mla(indexer=...) needs more than cached keys and values"
        elif c.type == "head":
            if c.pointer is not None:
                return "a copy pointer looks back over the whole context"
        elif c.type not in _PER_TOKEN and c.type not in _CONTINUED:
            return f"'{c.type}' carries state between tokens that is not cached here"
    return None


class DecodeCache:
    """Keys and values of every attention layer, and which cached positions are real tokens."""

    def __init__(self):
        self.keys: dict = {}
        self.values: dict = {}
        self.states: dict = {}     # recurrent mixers: the state after the last cached token
        self.tails: dict = {}      # causal convolutions: their last inputs
        self.real: Optional[torch.Tensor] = None      # [b, s] bool: False where a row is padded
        self.new_real: Optional[torch.Tensor] = None  # the same for the tokens of the call in flight

    @property
    def length(self) -> int:
        return 0 if self.real is None else self.real.shape[1]

    def begin(self, real: torch.Tensor) -> None:
        """A call starts: `real` [b, t] says which of its tokens are not padding."""
        self.new_real = real
        self.real = real if self.real is None else torch.cat([self.real, real], dim=1)

    def extend(self, layer, k: torch.Tensor, v: torch.Tensor) -> tuple:
        """Append a layer's new keys and values ([b, t, g, d]); returns all of them."""
        key = id(layer)
        if key in self.keys:
            k = torch.cat([self.keys[key], k], dim=1)
            v = torch.cat([self.values[key], v], dim=1)
        self.keys[key], self.values[key] = k, v
        return k, v

    def segments(self) -> tuple:
        """(ids of the call's tokens, ids of every cached position): padding is document 0, real
        tokens document 1, so attention confined to equal ids never reads padding."""
        return self.new_real.to(torch.int32), self.real.to(torch.int32)
