"""Routing containers and the device-side routing conversions.

The reference receives its routing as three objects defined by its dependency
(``RoutingData``, ``GatherIndx``, ``ScatterIndx``; built at
src/flaggems_sglang/ops/fused_moe.py:125-129).  That dependency is not needed
here: the containers below carry the same attribute names, and every entry point
reads its routing arguments by attribute only, so the dependency's own objects
are accepted as well.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib

BLOCK_MS = (16, 32, 64, 128)


@dataclass
class GatherIndx:
    src_indx: torch.Tensor
    dst_indx: torch.Tensor


@dataclass
class ScatterIndx:
    src_indx: torch.Tensor
    dst_indx: torch.Tensor


@dataclass
class ExptData:
    hist: torch.Tensor
    token_offs_raw: torch.Tensor
    token_offs_pad: dict
    block_pid_map: dict


@dataclass
class RoutingData:
    gate_scal: torch.Tensor = field()
    expt_hist: torch.Tensor = field()
    n_expts_tot: int = field()
    n_expts_act: int = field()
    expt_data: Optional[ExptData] = None
    expected_tokens_per_expt: Optional[int] = None


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: Optional[torch.Tensor] = None):
    """Group the flat slot ids ``token*topk + j`` by expert, each group padded
    to a multiple of ``block_size``.

    Returns ``(sorted_token_ids, expert_ids, num_tokens_post_padded)``, all int32
    on the device of ``topk_ids``.  Inside an expert the slots are in ascending
    order; padding entries of ``sorted_token_ids`` (and its unused tail) hold
    ``topk_ids.numel()``, the unused tail of ``expert_ids`` holds -1.
    ``expert_map`` (int32 [num_global_experts], negative = not local) drops the
    slots of experts held elsewhere; ``num_experts`` then counts local experts.
    """
    _require_cuda(topk_ids, "topk_ids")
    assert topk_ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64"
    ids = topk_ids.contiguous()
    n_slots = ids.numel()
    lib = _lib.lib()
    cap = lib.b200moe_align_capacity(n_slots, num_experts, block_size)
    _lib.check(min(cap, 0), "moe_align_block_size")
    dev = ids.device
    if cap == 0:
        z = torch.zeros(0, dtype=torch.int32, device=dev)
        return z, z.clone(), torch.zeros(1, dtype=torch.int32, device=dev)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty((cap + block_size - 1) // block_size, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    emap = None
    if expert_map is not None:
        emap = expert_map.to(device=dev, dtype=torch.int32).contiguous()
    with torch.cuda.device(dev):
        rc = lib.b200moe_align_block_size(
            ids.data_ptr(), int(ids.dtype == torch.int64), n_slots, num_experts, block_size,
            emap.data_ptr() if emap is not None else None, emap.numel() if emap is not None else 0,
            sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "moe_align_block_size")
    return sorted_ids, expert_ids, num_post


def topk_to_routing(topk_weights: torch.Tensor, topk_ids: torch.Tensor, n_expts_tot: int):
    """top-k output -> ``(RoutingData, GatherIndx, ScatterIndx)``.

    Same results as the reference's ``_standard_topk_to_triton_kernels``
    (src/flaggems_sglang/ops/fused_moe.py:103-130) in one kernel launch and with
    no host synchronisation.
    """
    _require_cuda(topk_ids, "topk_ids")
    assert topk_weights.shape == topk_ids.shape and topk_ids.ndim == 2
    assert topk_ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64"
    dev = topk_ids.device
    m, k = topk_ids.shape
    p = m * k
    ids = topk_ids.contiguous()
    w32 = topk_weights.to(torch.float32).contiguous()
    lib = _lib.lib()
    mt = lib.b200moe_routing_max_tiles(p, n_expts_tot)
    i32 = dict(dtype=torch.int32, device=dev)
    expt_indx = torch.empty(p, **i32)
    topk_indx = torch.empty(p, **i32)
    gate_indx = torch.empty(p, **i32)
    gate_scal = torch.empty(p, dtype=torch.float32, device=dev)
    hist = torch.empty(n_expts_tot, **i32)
    offs_raw = torch.empty(n_expts_tot + 1, **i32)
    offs_pad = torch.empty(4, n_expts_tot + 1, **i32)
    pid_map = torch.empty(4 * max(mt, 1), **i32)   # four block maps back to back, stride max_tiles
    with torch.cuda.device(dev):
        rc = lib.b200moe_routing_from_topk(
            w32.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64), m, k, n_expts_tot,
            expt_indx.data_ptr(), topk_indx.data_ptr(), gate_indx.data_ptr(), gate_scal.data_ptr(),
            hist.data_ptr(), offs_raw.data_ptr(), offs_pad.data_ptr(),
            pid_map.data_ptr(), _stream_ptr(dev))
    _lib.check(rc, "topk_to_routing")
    maps = pid_map[: 4 * mt].view(4, mt)
    expt_data = ExptData(
        hist=hist,
        token_offs_raw=offs_raw,
        token_offs_pad={bm: offs_pad[i] for i, bm in enumerate(BLOCK_MS)},
        block_pid_map={bm: maps[i] for i, bm in enumerate(BLOCK_MS)},
    )
    gs = gate_scal if topk_weights.dtype == torch.float32 else gate_scal.to(topk_weights.dtype)
    routing = RoutingData(gs, hist, n_expts_tot, k, expt_data)
    routing._expt_indx = expt_indx
    return routing, GatherIndx(src_indx=topk_indx, dst_indx=gate_indx), ScatterIndx(src_indx=gate_indx, dst_indx=topk_indx)
