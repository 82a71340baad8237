"""Expert parallelism: experts partitioned across ranks, tokens dispatched and
combined with all-to-all.

Rank r of R holds experts [r*E_loc, (r+1)*E_loc).  Every rank brings its own
tokens with routing over the *global* expert ids.  One call does

  dispatch   all_to_all: each peer receives this rank's token rows together with
             the top-k entries that point at the peer's experts (the other
             entries are masked to -1), in a fixed slot per (peer, token) so that
             no counts have to be exchanged and nothing on the host reads device
             data;
  local op   the single-GPU fused experts over the received rows (masked entries
             are dropped by the alignment kernel, so a token without a local
             expert costs no GEMM work and yields a zero row);
  combine    the per-(token, rank) partial sums travel back with the inverse
             all_to_all and the owner adds at most R of them in rank order.

With top-8 routing over at most 8 ranks nearly every token visits nearly every rank, and
the all-to-all above degenerates: every peer gets the same rows.  `mode="allgather"` (the
default when the ranks do not outnumber the experts per token) therefore dispatches with
an all-gather of the token rows and of the packed (ids, weights), lets each rank mask the
foreign experts through its `expert_map`, and combines with a reduce-scatter, which sums
the per-rank partial rows inside NCCL (in the NVSwitch where NVLS is active) instead of
moving all of them to the owner first.  `mode="alltoall"` keeps the slot-per-(peer, token)
exchange.

The reference has no counterpart: it rejects `expert_map`
(src/flaggems_sglang/ops/fused_moe.py:160-162) and contains no communication.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def dispatch_tables(topk_ids: torch.Tensor, topk_weights: torch.Tensor, n_local_experts: int, world: int):
    """Per-destination routing tables.

    Returns (ids [R, m, k] int32 with local expert ids or -1, weights [R, m, k]
    fp32 with 0 where masked)."""
    ids = topk_ids.to(torch.int64)
    dest = torch.div(ids, n_local_experts, rounding_mode="floor")
    ranks = torch.arange(world, device=ids.device).view(world, 1, 1)
    mine = dest.unsqueeze(0) == ranks
    local = (ids.unsqueeze(0) - ranks * n_local_experts)
    out_ids = torch.where(mine, local, torch.full_like(local, -1)).to(torch.int32)
    out_w = torch.where(mine, topk_weights.to(torch.float32).unsqueeze(0), torch.zeros((), device=ids.device))
    return out_ids.contiguous(), out_w.contiguous()


_expert_maps: dict = {}
_last_collective = "none"


def last_collective() -> str:
    """What the most recent ``ep_fused_experts`` call on this rank used to move rows (for reports)."""
    return _last_collective



def local_expert_map(n_global: int, n_local: int, rank: int, device) -> torch.Tensor:
    """int32 [n_global]: local index of the experts this rank holds, -1 elsewhere."""
    key = (n_global, n_local, rank, str(device))
    m = _expert_maps.get(key)
    if m is None:
        m = torch.full((n_global,), -1, dtype=torch.int32, device=device)
        m[rank * n_local:(rank + 1) * n_local] = torch.arange(n_local, dtype=torch.int32, device=device)
        _expert_maps[key] = m
    return m


def _reduce_scatter_rows(partial: torch.Tensor, m: int, group) -> torch.Tensor:
    out = torch.empty(m, partial.shape[1], dtype=partial.dtype, device=partial.device)
    try:
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=group)
    except (RuntimeError, NotImplementedError):     # back ends without reduce-scatter (gloo)
        full = partial.clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        out.copy_(full[r * m:(r + 1) * m])
    return out


def ep_fused_experts(
    hidden_states: torch.Tensor,
    w13_local: torch.Tensor,
    w2_local: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    group: Optional[dist.ProcessGroup] = None,
    local_fn: Optional[Callable] = None,
    mode: Optional[str] = None,
    **kwargs,
) -> torch.Tensor:
    """Expert-parallel fused MoE for this rank's tokens ``hidden_states [m, H]``.

    Every rank must call with the same ``m`` (pad the last batch if needed).
    ``local_fn(x, w13, w2, topk_weights, topk_ids, **kwargs)`` computes the local
    experts; it defaults to the CUDA operator of this package.
    """
    own_operator = local_fn is None
    if local_fn is None:
        from .ops.fused_moe import fused_experts as local_fn
    world = dist.get_world_size(group)
    m, h = hidden_states.shape
    k = topk_ids.shape[1]
    e_loc = w13_local.shape[0]
    global _last_collective
    if world == 1:
        _last_collective = "none (one rank)"
        return local_fn(hidden_states, w13_local, w2_local, topk_weights, topk_ids.to(torch.int32), **kwargs)
    if mode is None:
        mode = "allgather" if world <= max(k, 2) else "alltoall"
    if mode == "allgather":
        _last_collective = "all-gather of token rows and routing (dispatch) + reduce-scatter of partial rows (combine)"
        rank = dist.get_rank(group)
        x = hidden_states.contiguous()
        parts = [topk_ids.to(torch.int32), topk_weights.to(torch.float32).view(torch.int32)]
        fp8_rows = (own_operator and bool(kwargs.get("use_fp8_w8a8")) and x.is_cuda and h % 128 == 0
                    and x.dtype != torch.float8_e4m3fn)
        if fp8_rows:
            # FP8 weights: quantise this rank's rows before they travel (half the bytes on the wire, and
            # no rank quantises another rank's rows again); the 1x128 scales ride with ids and weights
            from .ops.quant import per_token_group_quant_fp8
            xq, xsc = per_token_group_quant_fp8(x)
            payload = xq.view(torch.uint8)
            parts.append(xsc.view(torch.int32))
        else:
            payload = x
        xg = torch.empty(world * m, h, dtype=payload.dtype, device=x.device)
        dist.all_gather_into_tensor(xg, payload, group=group)
        meta = torch.cat(parts, dim=1).contiguous()
        mg = torch.empty(world * m, meta.shape[1], dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(mg, meta, group=group)
        ids_all = mg[:, :k].contiguous()
        w_all = mg[:, k:2 * k].contiguous().view(torch.float32)
        emap = local_expert_map(e_loc * world, e_loc, rank, x.device)
        if fp8_rows:
            partial = local_fn(xg.view(torch.float8_e4m3fn), w13_local, w2_local, w_all, ids_all, expert_map=emap,
                               x_scale=mg[:, 2 * k:].contiguous().view(torch.float32), out_dtype=x.dtype, **kwargs)
        else:
            partial = local_fn(xg, w13_local, w2_local, w_all, ids_all, expert_map=emap, **kwargs)
        return _reduce_scatter_rows(partial.contiguous(), m, group)
    assert mode == "alltoall", f"unknown expert-parallel mode {mode!r}"
    _last_collective = "all-to-all of token rows and masked routing (dispatch) + all-to-all of partial rows (combine)"

    ids_t, w_t = dispatch_tables(topk_ids, topk_weights, e_loc, world)
    send_x = hidden_states.unsqueeze(0).expand(world, m, h).contiguous()
    recv_x = torch.empty_like(send_x)
    # ids and weights share one int32 payload: [R, m, 2k]
    meta = torch.cat([ids_t, w_t.view(torch.int32)], dim=2).contiguous()
    recv_meta = torch.empty_like(meta)
    dist.all_to_all_single(recv_x, send_x, group=group)
    dist.all_to_all_single(recv_meta, meta, group=group)

    r_ids = recv_meta[:, :, :k].reshape(world * m, k).contiguous()
    r_w = recv_meta[:, :, k:].contiguous().view(torch.float32).reshape(world * m, k)
    partial = local_fn(recv_x.view(world * m, h), w13_local, w2_local, r_w, r_ids, **kwargs)

    back = torch.empty(world, m, h, dtype=partial.dtype, device=partial.device)
    dist.all_to_all_single(back, partial.view(world, m, h).contiguous(), group=group)
    return back.float().sum(dim=0).to(hidden_states.dtype)
