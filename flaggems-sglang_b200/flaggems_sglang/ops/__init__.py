"""``flaggems_sglang.ops`` (reference: src/flaggems_sglang/ops/__init__.py:1-4, 14-21): the
fused-MoE operators.  The reference's other operators (gated-delta-rule decode, Gemma RMSNorm,
M-RoPE) are not part of this package."""
from flaggems_sglang_b200.ops import *  # noqa: F401,F403
from flaggems_sglang_b200.ops import __all__ as _b200_all

from . import fused_moe  # noqa: F401,E402
from .fused_moe import (  # noqa: F401,E402
    triton_kernel_fused_experts,
    triton_kernel_fused_experts_with_bias,
)

__all__ = list(_b200_all)
