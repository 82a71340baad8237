"""B200-native fused Mixture-of-Experts, drop-in for ``flaggems_sglang``'s
fused-MoE entry points (src/flaggems_sglang/__init__.py:7-10 in the reference)."""
from .ops import (
    check_status,
    release_workspaces,
    fused_experts,
    fused_moe,
    fused_moe_flagos,
    grouped_topk,
    moe_align_block_size,
    topk_softmax,
    topk_to_routing,
    triton_kernel_fused_experts,
    triton_kernel_fused_experts_with_bias,
)
from .routing import ExptData, GatherIndx, RoutingData, ScatterIndx

__version__ = "0.1.0"
device = "cuda"
vendor_name = "nvidia"

__all__ = [
    "check_status",
    "release_workspaces",
    "fused_experts",
    "fused_moe",
    "fused_moe_flagos",
    "grouped_topk",
    "topk_softmax",
    "moe_align_block_size",
    "topk_to_routing",
    "triton_kernel_fused_experts",
    "triton_kernel_fused_experts_with_bias",
    "ExptData", "GatherIndx", "RoutingData", "ScatterIndx",
]
