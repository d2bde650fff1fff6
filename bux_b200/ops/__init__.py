"""Ops: sm_100a kernels on CUDA (`kernels`, `functional`, `fused`), plain PyTorch on CPU (`reference`)."""
from . import reference  # noqa: F401
from .functional import (attention, causal_conv, glu, kernels_on, linear, linear_f32, rmsnorm, rmsnorm_rope, rope,  # noqa: F401
                         set_kernels)
from .fused import cross_entropy_head, moe_experts, moe_reference, sort_picks  # noqa: F401
