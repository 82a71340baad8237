"""``flaggems_sglang.ops.fused_moe``: the module SGLang's plugin loader imports
``fused_moe_flagos`` from (reference: src/flaggems_sglang/ops/fused_moe.py:133, 219, 312) and
the reference's tests import the routing conversion from (tests/test_fused_moe.py:8-11)."""
from flaggems_sglang_b200.ops.fused_moe import (  # noqa: F401
    _standard_topk_to_triton_kernels,
    check_status,
    fused_experts,
    fused_moe,
    fused_moe_flagos,
    triton_kernel_fused_experts,
    triton_kernel_fused_experts_with_bias,
)

__all__ = [
    "triton_kernel_fused_experts",
    "triton_kernel_fused_experts_with_bias",
    "fused_moe_flagos",
    "_standard_topk_to_triton_kernels",
]
