"""Router front-end: gating logits -> (topk_weights, topk_ids) on the GPU.

The reference leaves this step to its caller (recipe in tests/test_fused_moe.py:21-27:
softmax, top-k, divide by the sum); grouped selection is the DeepSeek rule the serving
stack calls ``grouped_topk``.  One kernel, no host reads; ties go to the lower expert id.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from .. import _lib

_LOGIT_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16, torch.float32: _lib.DTYPE_FP32}
_SCORING = {"softmax": _lib.SCORE_SOFTMAX, "sigmoid": _lib.SCORE_SIGMOID}


def make_router(gating_output: torch.Tensor, topk: int, renormalize: bool, num_expert_group: int = 0,
                topk_group: int = 0, scoring_func: str = "softmax",
                correction_bias: Optional[torch.Tensor] = None, scale: float = 1.0):
    """Validated ``_lib.Router`` plus the tensors it points at (keep them alive for the call)."""
    assert gating_output.is_cuda, "the CUDA extension is the only implementation: tensors must be on a GPU"
    assert gating_output.dim() == 2, "gating_output must be [tokens, experts]"
    assert gating_output.dtype in _LOGIT_DTYPES, "gating_output must be bfloat16, float16 or float32"
    if scoring_func not in _SCORING:
        raise ValueError(f"Unsupported scoring function: {scoring_func}")
    e = gating_output.shape[1]
    assert 0 < topk <= min(e, _lib.ROUTER_MAX_TOPK), "topk out of range"
    assert e <= _lib.ROUTER_MAX_EXPERTS, "too many experts for the router kernel"
    if num_expert_group and num_expert_group > 1:
        assert num_expert_group <= 32 and e % num_expert_group == 0, "expert groups must divide the experts (<= 32)"
        assert 0 < topk_group <= num_expert_group, "topk_group out of range"
        assert topk <= topk_group * (e // num_expert_group), "topk exceeds the experts of the kept groups"
    bias = None
    if correction_bias is not None:
        bias = correction_bias.to(device=gating_output.device, dtype=torch.float32).contiguous()
        assert bias.shape == (e,), "correction_bias must be [experts]"
    logits = gating_output.contiguous()
    r = _lib.Router(C.sizeof(_lib.Router), _SCORING[scoring_func], int(bool(renormalize)),
                    int(num_expert_group or 0), int(topk_group or 0), _LOGIT_DTYPES[logits.dtype], float(scale), 0,
                    bias.data_ptr() if bias is not None else None)
    return r, logits, bias


def _route(gating_output, topk, renormalize, **kw) -> Tuple[torch.Tensor, torch.Tensor]:
    r, logits, bias = make_router(gating_output, topk, renormalize, **kw)
    m, e = logits.shape
    dev = logits.device
    tw = torch.empty((m, topk), dtype=torch.float32, device=dev)
    ids = torch.empty((m, topk), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.lib().b200moe_route_topk(C.byref(r), logits.data_ptr(), m, e, topk, tw.data_ptr(), ids.data_ptr(),
                                           torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "route_topk")
    return tw, ids


def topk_softmax(gating_output: torch.Tensor, topk: int, renormalize: bool = True):
    """softmax over the experts, the ``topk`` largest, optionally divided by their sum."""
    return _route(gating_output, topk, renormalize)


def grouped_topk(gating_output: torch.Tensor, topk: int, renormalize: bool, num_expert_group: int,
                 topk_group: int, scoring_func: str = "softmax", correction_bias: Optional[torch.Tensor] = None,
                 routed_scaling_factor: float = 1.0):
    """Group-limited top-k: experts form ``num_expert_group`` contiguous groups, the
    ``topk_group`` best groups stay eligible (group score: largest expert score, or with a
    ``correction_bias`` the sum of the two largest biased scores), then the ``topk``
    experts by (biased) score; weights are the unbiased scores."""
    return _route(gating_output, topk, renormalize, num_expert_group=num_expert_group, topk_group=topk_group,
                  scoring_func=scoring_func, correction_bias=correction_bias, scale=routed_scaling_factor)
