"""RoPE frequencies: plain, position interpolation, Llama-3 and YaRN scaling.

Reference: ``architecture/attention/rope.py:31-130`` (`frequencies`, `logit_gain`).
Returns inverse frequencies (one per rotated pair) and the gain YaRN applies.
"""

from __future__ import annotations

import math

import torch


def rotated_dims(head_dim: int, fraction: float) -> int:
    r = int(head_dim * fraction)
    return r - (r % 2)


def inverse_frequencies(c, head_dim: int, device=None) -> tuple:
    """(inv_freq [R/2] fp32, gain) for a ``rope(...)`` config `c`."""
    r = rotated_dims(head_dim, c.fraction)
    exponents = torch.arange(0, r, 2, dtype=torch.float32, device=device) / r
    inv = c.base ** (-exponents)
    gain = 1.0
    s = c.scaling
    if s is None:
        return inv, gain
    if s.type == "pi":
        return inv / s.factor, gain
    wavelengths = 2 * math.pi / inv
    if s.type == "llama3":
        low = s.original_max_len / s.low_freq_factor
        high = s.original_max_len / s.high_freq_factor
        smooth = (s.original_max_len / wavelengths - s.low_freq_factor) / (
            s.high_freq_factor - s.low_freq_factor)
        mixed = (1 - smooth) * inv / s.factor + smooth * inv
        out = torch.where(wavelengths > low, inv / s.factor, torch.where(wavelengths < high, inv, mixed))
        return out, gain
    if s.type == "yarn":
        def turns_to_dim(turns: float) -> float:
            return r * math.log(s.original_max_len / (turns * 2 * math.pi)) / (2 * math.log(c.base))

        lo = max(math.floor(turns_to_dim(s.beta_fast)), 0)
        hi = min(math.ceil(turns_to_dim(s.beta_slow)), r // 2 - 1)
        ramp = ((torch.arange(r // 2, dtype=torch.float32, device=device) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        keep = 1 - ramp  # 1: extrapolate (keep), 0: interpolate (divide by factor)
        out = inv / s.factor * (1 - keep) + inv * keep
        gain = s.attention_factor if s.attention_factor is not None else 0.1 * math.log(s.factor) + 1.0
        return out, gain
    raise ValueError(s.type)


def tables(positions: torch.Tensor, inv_freq: torch.Tensor, gain: float = 1.0):
    """cos, sin of shape positions.shape + (R/2,), fp32; `gain` scales both (YaRN)."""
    ang = positions.float().unsqueeze(-1) * inv_freq.to(positions.device)
    return ang.cos() * gain, ang.sin() * gain
