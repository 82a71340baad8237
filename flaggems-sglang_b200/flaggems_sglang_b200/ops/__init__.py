from .fused_moe import (
    check_status,
    release_workspaces,
    fused_experts,
    fused_moe,
    fused_moe_flagos,
    triton_kernel_fused_experts,
    triton_kernel_fused_experts_with_bias,
)
from .router import grouped_topk, topk_softmax
from ..routing import moe_align_block_size, topk_to_routing

__all__ = [
    "check_status",
    "release_workspaces",
    "fused_experts",
    "fused_moe",
    "fused_moe_flagos",
    "grouped_topk",
    "topk_softmax",
    "triton_kernel_fused_experts",
    "triton_kernel_fused_experts_with_bias",
    "moe_align_block_size",
    "topk_to_routing",
]
