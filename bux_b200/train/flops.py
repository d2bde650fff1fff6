"""Model FLOPs per token, counted from the architecture: 2·m·n·k per matmul a token
passes through (routed experts at top_k), attention at the keys a query actually sees
(causal: (S+1)/2 on average; sliding window: at most the window), times 3 for forward +
backward. Embedding lookups count nothing.

Reference: ``train/flops.py:40-232`` (there counted on the traced program; the rules
are the same, and the totals agree: Qwen3-30B-A3B at 4096 → 23.1 GFLOP/token).
"""

from __future__ import annotations

from ..config import layers as L
from ..lang import ir

PEAK = {"B300": 2.25e15, "B200": 2.25e15, "H200": 989e12, "H100": 989e12, "A100": 312e12}


def device_peak(device) -> float:
    """Dense bf16 peak FLOP/s of `device`, 0 when unknown (then no MFU is logged)."""
    import torch

    if getattr(device, "type", "cpu") != "cuda":
        return 0.0
    name = torch.cuda.get_device_name(device)
    for key, peak in PEAK.items():
        if key in name:
            return peak
    return 0.0


def keys_seen(seq_len: int, window=None, positions=None, top_k=None) -> float:
    """Average number of keys a query attends: query i of its document sees ``i + 1`` keys,
    at most `window`, at most `top_k` picks. Without `positions` every row is one document of
    `seq_len` tokens; with the batch's position ids (which restart at every document of a
    packed row) the average is over the documents as they are (reference: ``train/flops.py:49-99``,
    the mask's share of the square)."""
    import numpy as np

    if positions is None:
        seen = np.arange(1, seq_len + 1, dtype=np.float64)
    else:
        seen = np.asarray(positions, dtype=np.float64).reshape(-1) + 1.0
    for cap in (window, top_k):
        if cap:
            seen = np.minimum(seen, float(cap))
    return float(seen.mean())


def _attention_flops(heads: int, qk_dim: int, v_dim: int, seq_len: int, window, positions=None, top_k=None) -> float:
    return 2.0 * heads * (qk_dim + v_dim) * keys_seen(seq_len, window, positions, top_k)


def _indexer_flops(ix, w: int, seq_len: int, positions=None) -> float:
    """The scorer of a sparse attention layer: its projections, and a score for every key a
    query could see (all of them: that is what picking means), per block when it pools."""
    if ix is None:
        return 0.0
    proj = 2.0 * w * (ix.num_heads * ix.head_dim + ix.head_dim) + (2.0 * w * ix.num_heads if ix.weighted else 0.0)
    keys = keys_seen(seq_len, None, positions) / max(1, ix.block_size or 1)
    return proj + 2.0 * ix.num_heads * ix.head_dim * keys


def layer_forward_flops(c, width, d_model: int, vocab: int, seq_len: int, positions=None) -> float:
    """Forward FLOPs per token of one layer (`positions`: a batch's position ids, for packed rows)."""
    w = width if isinstance(width, int) else d_model
    t = c.type
    if t in ("mlp", "gated_mlp"):
        mats = 3 if t == "gated_mlp" else 2
        return 2.0 * mats * w * c.intermediate_size
    if t == "moe":
        e = c.expert
        mats = 3 if e.type == "gated_mlp" else 2
        per = 2.0 * mats * w * e.intermediate_size
        total = per * c.top_k + 2.0 * w * c.num_experts
        if c.num_shared_experts:
            s = c.shared_expert or c.expert
            total += 2.0 * (3 if s.type == "gated_mlp" else 2) * w * s.intermediate_size * c.num_shared_experts
        return total
    if t == "gqa":
        d = c.head_dim or w // c.num_heads
        dv = c.v_head_dim or d
        proj = 2.0 * w * (c.num_heads * d + c.num_kv_heads * (d + dv)) + 2.0 * c.num_heads * dv * w
        if c.gated:
            proj += 2.0 * w * (c.num_heads if c.gate_per_head else c.num_heads * dv)
        picks = c.indexer.top_k * (c.indexer.block_size or 1) if c.indexer is not None else None
        return (proj + _attention_flops(c.num_heads, d, dv, seq_len, c.sliding_window_size, positions, picks)
                + _indexer_flops(c.indexer, w, seq_len, positions))
    if t == "csa":
        d = c.head_dim
        q = 2.0 * w * c.num_heads * d if c.q_lora_rank is None else 2.0 * (w * c.q_lora_rank + c.q_lora_rank * c.num_heads * d)
        kv = 2.0 * w * d * (1.0 + 2.0 / c.compress_ratio)         # the window's latent, and the compressor's share per token
        o = 2.0 * c.num_heads * d * w if c.o_lora_rank is None else 2.0 * (c.num_heads * d * c.o_lora_rank + c.o_lora_rank * w)
        local = keys_seen(seq_len, c.sliding_window_size, positions)
        far = keys_seen(seq_len, None, positions) / c.compress_ratio
        if c.indexer is not None:
            far = min(far, float(c.indexer.top_k))
        return q + kv + o + 2.0 * c.num_heads * 2 * d * (local + far) + _indexer_flops(c.indexer, w, seq_len / c.compress_ratio)
    if t == "mla":
        qk = c.qk_nope_head_dim + c.qk_rope_head_dim
        q = 2.0 * w * c.num_heads * qk if c.q_lora_rank is None else \
            2.0 * (w * c.q_lora_rank + c.q_lora_rank * c.num_heads * qk)
        kv = 2.0 * w * (c.kv_lora_rank + c.qk_rope_head_dim) + \
            2.0 * c.kv_lora_rank * c.num_heads * (c.qk_nope_head_dim + c.v_head_dim)
        o = 2.0 * c.num_heads * c.v_head_dim * w
        picks = c.indexer.top_k * (c.indexer.block_size or 1) if c.indexer is not None else None
        return (q + kv + o + _attention_flops(c.num_heads, qk, c.v_head_dim, seq_len, c.sliding_window_size, positions, picks)
                + _indexer_flops(c.indexer, w, seq_len, positions))
    if t == "head":
        return 2.0 * w * vocab
    if t == "linear":
        return 2.0 * w * c.features
    if t == "nextn":
        return 2.0 * (2 * w) * w          # the stream and the next token's embedding, joined and projected
    if t in ("conv", "short_conv"):
        return 2.0 * w * (c.size if t == "conv" else c.conv_size)
    if isinstance(c, L.LinearAttentionConfig):
        d = c.head_dim
        hv = c.num_v_heads or c.num_heads
        dv = c.v_head_dim or d
        proj = 2.0 * w * (2 * c.num_heads * d + 2 * hv * dv) + 2.0 * hv * dv * w
        state = 4.0 * hv * d * dv  # state update and read per token
        return proj + state
    if isinstance(c, L.StateSpaceConfig):
        inner = c.expand * w
        return 2.0 * w * inner * 3 + 2.0 * inner * c.state_size * 3
    return 0.0


def flops_per_token(arch: ir.Architecture, seq_len: int, positions=None) -> float:
    """Training FLOPs per token: 3 × the forward's (a backward is two products per forward
    product). What a rerun of the forward costs under remat is hardware work, not model work,
    and is not counted: MFU stays comparable between remat policies. With `positions` (a
    packed batch's position ids) attention is counted at the keys the documents' queries see."""
    total = 0.0
    for layer in arch.layers():
        total += layer_forward_flops(layer.config, layer.width, arch.d_model, arch.vocab_size or 0, seq_len, positions)
    return 3.0 * total
