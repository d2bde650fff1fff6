"""NVFP4 matmuls: E2M1 values in blocks of 16 along a row, one E4M3 scale per block, one
fp32 scale per tensor; the recipe NVIDIA describes for pretraining and the reference
registers as the format ``nvfp4`` (``architecture/precision/nvfp4.py:46-140`` there):

* activations are quantised in 1 x 16 blocks, to nearest;
* weights in 16 x 16 tiles, so that W and W^T hold the same values;
* output gradients are rounded stochastically (unbiased);
* the two operands of the weight gradient, x^T and dy^T, are contracted over tokens, and a
  random-sign Hadamard transform of every 16 tokens is applied to both first (it cancels in
  the product and spreads a block's outliers over the block).

Here the quantisers are plain PyTorch (`quantize`) with a CUDA kernel for the 1 x 16 case
(`bux_b200.ops.kernels.quant_nvfp4`, `cvt.rn.satfinite.e2m1x2` on sm_100a, bit-equal to
`quantize`), and the products run on the bf16 tensor cores over the dequantised operands:
block scale times E2M1 value is exact in bf16, the two tensor scales multiply the result.
The numerics are NVFP4's; an FP4 tensor-core GEMM (`kind::mxf4nvf4`) is not written.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch

BLOCK = 16
E2M1_MAX = 6.0
E4M3_MAX = 448.0
_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


class Blocks(NamedTuple):
    values: torch.Tensor        # fp32 on the E2M1 grid, [R, C]
    scales: torch.Tensor        # fp32 holding E4M3 values, [R, C/16]
    tensor_scale: torch.Tensor  # fp32 scalar: x ≈ values · scales · tensor_scale

    def dequantized(self, with_tensor_scale: bool = True) -> torch.Tensor:
        r, c = self.values.shape
        out = (self.values.view(r, c // BLOCK, BLOCK) * self.scales.unsqueeze(-1)).view(r, c)
        return out * self.tensor_scale if with_tensor_scale else out


def hadamard_matrix(device=None) -> torch.Tensor:
    """Sylvester's 16 x 16 Hadamard matrix with its rows' signs drawn once (seed 0), over 4:
    orthogonal."""
    i = torch.arange(BLOCK)
    bits = (i[:, None] & i[None, :])
    pop = sum((bits >> b) & 1 for b in range(4))
    sylvester = torch.where(pop % 2 == 0, 1.0, -1.0)
    g = torch.Generator().manual_seed(0)
    signs = torch.where(torch.rand(BLOCK, generator=g) < 0.5, -1.0, 1.0)
    return (signs[:, None] * sylvester / 4).to(device=device, dtype=torch.float32)


def hadamard_rows(x: torch.Tensor) -> torch.Tensor:
    """Each 16 consecutive values of a row, transformed."""
    r, c = x.shape
    h = hadamard_matrix(x.device)
    return (x.float().view(r, c // BLOCK, BLOCK) @ h.t()).view(r, c)


def round_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest value of the E2M1 grid (ties to the even mantissa), magnitudes clamped to 6."""
    a = x.abs().clamp(max=E2M1_MAX)
    # spacing 0.5 below 2, 1 below 4, 2 below 6: round in units of the local spacing
    step = torch.where(a < 2.0, 0.5, torch.where(a < 4.0, 1.0, 2.0))
    q = torch.round(a / step) * step          # torch.round rounds half to even
    return torch.copysign(q, x)


def round_e2m1_stochastic(x: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """Round up or down to a grid neighbour with probability by distance (`noise` in [0, 1))."""
    a = x.abs().clamp(max=E2M1_MAX)
    step = torch.where(a < 2.0, 0.5, torch.where(a < 4.0, 1.0, 2.0))
    low = torch.floor(a / step) * step
    up = (a - low) / step > noise
    return torch.copysign(torch.where(up, low + step, low).clamp(max=E2M1_MAX), x)


def quantize(x: torch.Tensor, *, tiles: bool = False, stochastic: bool = False, hadamard: bool = False,
             seed: int = 0) -> Blocks:
    """x [R, C] (C % 16 == 0; with `tiles` R % 16 == 0 too) in NVFP4 along its rows."""
    x = x.float()
    if hadamard:
        x = hadamard_rows(x)
    r, c = x.shape
    amax = x.abs().max().clamp_min(1e-30)
    tensor_scale = amax / (E2M1_MAX * E4M3_MAX)
    if tiles:
        block_amax = x.abs().view(r // BLOCK, BLOCK, c // BLOCK, BLOCK).amax((1, 3))
        block_amax = block_amax.repeat_interleave(BLOCK, dim=0)
    else:
        block_amax = x.abs().view(r, c // BLOCK, BLOCK).amax(-1)
    scales = (block_amax / (E2M1_MAX * tensor_scale)).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn).float()
    denom = (scales * tensor_scale).unsqueeze(-1)
    scaled = torch.where(denom > 0, x.view(r, c // BLOCK, BLOCK) / denom.clamp_min(1e-30), torch.zeros(()).to(x))
    if stochastic:
        g = torch.Generator(device=x.device).manual_seed(int(seed))
        noise = torch.rand(scaled.shape, generator=g, device=x.device)
        values = round_e2m1_stochastic(scaled, noise)
    else:
        values = round_e2m1(scaled)
    return Blocks(values.view(r, c), scales, tensor_scale)


def _matmul(a: Blocks, b: Blocks) -> torch.Tensor:
    """dequant(a) · dequant(b)^T: exact block products in bf16, tensor scales on the result."""
    x, w = a.dequantized(False), b.dequantized(False)
    if x.is_cuda:
        from . import kernels as K
        from .functional import kernels_on

        xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
        if kernels_on(xb) and xb.shape[1] % 8 == 0:
            out = K.gemm_bf16(xb.contiguous(), wb.contiguous(), out_dtype=torch.float32)
        else:
            out = xb.float() @ wb.float().t()
    else:
        out = x @ w.t()
    return out * (a.tensor_scale * b.tensor_scale)


class _LinearNVFP4(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, seed, passes):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.shape, ctx.seed, ctx.passes = x.shape, seed, passes
        if "fprop" in passes:
            y = _matmul(quantize(x2), quantize(w, tiles=True))
        else:
            y = x2 @ w.to(x2.dtype).t()
        return y.to(x.dtype).view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if "dgrad" in ctx.passes:
                # dx = dy · W: W^T in 16 x 16 tiles holds W's values
                dyq = quantize(dy2, stochastic=True, seed=ctx.seed)
                wtq = quantize(w.t().contiguous(), tiles=True)
                dx = _matmul(dyq, wtq).to(x2.dtype).view(ctx.shape)
            else:
                dx = (dy2 @ w.to(dy2.dtype)).to(x2.dtype).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            if "wgrad" in ctx.passes:
                # dW = dy^T · x, contracted over tokens: both operands transformed along the tokens
                m = dy2.shape[0]
                pad = (-m) % BLOCK
                dyt, xt = dy2.t().float(), x2.t().float()
                if pad:
                    dyt = torch.nn.functional.pad(dyt, (0, pad))
                    xt = torch.nn.functional.pad(xt, (0, pad))
                dytq = quantize(dyt.contiguous(), stochastic=True, hadamard=True, seed=ctx.seed + 1)
                xtq = quantize(xt.contiguous(), hadamard=True)
                dw = _matmul(dytq, xtq).to(w.dtype)
            else:
                dw = (dy2.t() @ x2.to(dy2.dtype)).to(w.dtype)
        return dx, dw, None, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, seed: int = 0,
           passes=("fprop", "dgrad", "wgrad")) -> torch.Tensor:
    """x [..., in] · w [out, in]^T (+ bias) with NVFP4 operands in the products of `passes`
    (the others multiply in the compute dtype)."""
    y = _LinearNVFP4.apply(x, w, seed, tuple(passes))
    return y if bias is None else y + bias.to(y.dtype)


def pack(blocks: Blocks) -> tuple:
    """(uint8 [R, C/2] two E2M1 codes per byte, low nibble first; e4m3 scale bytes [R, C/16]):
    the storage an FP4 GEMM reads, and what the CUDA quantiser writes."""
    v = blocks.values
    grid = torch.tensor(_GRID, device=v.device)
    code = (v.abs().unsqueeze(-1) - grid).abs().argmin(-1).to(torch.uint8)
    code = code | ((v < 0) | ((v == 0) & (torch.signbit(v)))).to(torch.uint8) << 3
    r, c = v.shape
    pairs = code.view(r, c // 2, 2)
    packed = pairs[..., 0] | (pairs[..., 1] << 4)
    return packed, blocks.scales.to(torch.float8_e4m3fn).view(torch.uint8)
