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

`mode="peer"` (the default for FP8 weights on CUDA) uses no collective at all: every rank maps
the other ranks' heaps (CUDA IPC over NVLink) and one C call does everything -- tokens are
quantised once and stored straight into the heaps of the ranks that hold their experts (a row
travels only where it is needed), the local operator runs over the rows received, and the down
projection's epilogue stores each (token, choice) row into the heap of the rank that owns the
token, where the output conversion sums a token's rows in a fixed order.  Synchronisation is by
epoch flags with bounded waits.  Experts may sit anywhere (`plan_placement`): a load-balanced
placement keeps the hot experts of a skewed router on different ranks.  The result is
bit-identical to the single-GPU operator on the same tokens.

The reference has no counterpart: it rejects `expert_map`
(src/flaggems_sglang/ops/fused_moe.py:160-162) and contains no communication.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------- expert placement
def plan_placement(n_global_experts: int, world: int, load: Optional[Sequence[float]] = None) -> torch.Tensor:
    """Which rank holds which expert: int32 [n_global_experts], entry = (rank << 16) | local id.

    Every rank gets n_global_experts / world experts.  Without ``load`` the partition is
    contiguous (rank r holds experts [r * n_local, (r + 1) * n_local)).  With ``load`` (expected
    tokens per expert, e.g. counted over earlier batches) experts are dealt out heaviest first,
    each to the rank with the least load so far that still has a free place, so that the hot
    experts of a skewed router end up on different ranks."""
    assert n_global_experts % world == 0, "experts must divide evenly over the ranks"
    n_local = n_global_experts // world
    assert n_local <= 0xFFFF and world <= 0x7FFF
    place = torch.empty(n_global_experts, dtype=torch.int32)
    if load is None:
        e = torch.arange(n_global_experts, dtype=torch.int32)
        return ((e // n_local) << 16) | (e % n_local)
    load = [float(v) for v in load]
    assert len(load) == n_global_experts
    order = sorted(range(n_global_experts), key=lambda i: (-load[i], i))
    total = [0.0] * world
    used = [0] * world
    for e in order:
        r = min((r for r in range(world) if used[r] < n_local), key=lambda r: (total[r], r))
        place[e] = (r << 16) | used[r]
        used[r] += 1
        total[r] += load[e]
    return place


def validate_placement(placement: torch.Tensor, world: int, n_local: int) -> None:
    """A placement must send every expert it places to an existing rank and a free local index."""
    p = placement.detach().cpu().to(torch.int64)
    placed = p[p >= 0]
    ranks, locs = placed >> 16, placed & 0xFFFF
    if placed.numel() and (int(ranks.max()) >= world or int(locs.max()) >= n_local):
        raise ValueError("placement names a rank or a local expert index that does not exist")
    keys = ranks * n_local + locs
    if keys.unique().numel() != keys.numel():
        raise ValueError("placement puts two experts on the same (rank, local index)")


def local_experts(placement: torch.Tensor, rank: int) -> list:
    """Global ids of the experts ``rank`` holds, in local-index order."""
    p = placement.detach().cpu().to(torch.int64)
    mine = [(int(v & 0xFFFF), e) for e, v in enumerate(p.tolist()) if v >= 0 and (v >> 16) == rank]
    return [e for _, e in sorted(mine)]


def dispatch_tables_placed(topk_ids: torch.Tensor, topk_weights: torch.Tensor, placement: torch.Tensor, world: int):
    """What the dispatch kernel writes for each destination rank, in torch: ids [R, m, k] int32
    (local expert id on that rank, -1 where the expert lives elsewhere or nowhere) and weights
    [R, m, k] fp32 (0 where masked)."""
    ids = topk_ids.to(torch.int64)
    pl = placement.to(device=ids.device, dtype=torch.int64)
    ok = (ids >= 0) & (ids < pl.numel())
    v = torch.where(ok, pl[ids.clamp(0, pl.numel() - 1)], torch.full_like(ids, -1))
    dest = torch.where(v >= 0, v >> 16, torch.full_like(v, -1))
    loc = v & 0xFFFF
    ranks = torch.arange(world, device=ids.device).view(world, 1, 1)
    mine = dest.unsqueeze(0) == ranks
    out_ids = torch.where(mine, loc.unsqueeze(0), torch.full_like(loc, -1).unsqueeze(0)).to(torch.int32)
    out_w = torch.where(mine, topk_weights.to(torch.float32).unsqueeze(0), torch.zeros((), device=ids.device))
    return out_ids.contiguous(), out_w.contiguous()



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



# ---------------------------------------------------------------------------- peer-store mode (CUDA)
class EpContext:
    """One rank's side of the peer-store expert parallelism: its heap, the mappings of the other
    ranks' heaps, the scratch of the local operator.  Set-up allocates and synchronises; the
    forward call does neither.

    ``heaps`` lets a test drive several ranks from one process on one GPU: the contexts then share
    one list of heap addresses and call ``forward`` phase by phase."""

    def __init__(self, rank: int, world: int, m_cap: int, h: int, i: int, topk: int, n_local: int, n_global: int,
                 device, dtype=torch.bfloat16, group=None, heaps: Optional[list] = None, wait_limit_ns: int = 0,
                 flags: int = 0):
        from . import _lib
        self._lib, self.lib = _lib, _lib.lib()
        self.rank, self.world, self.m_cap, self.h, self.i, self.topk = rank, world, m_cap, h, i, topk
        self.n_local, self.n_global, self.device, self.group = n_local, n_global, torch.device(device), group
        self.flags = flags
        self.ep = _lib.EpCfg(C.sizeof(_lib.EpCfg), world, rank, m_cap, n_global, 0, wait_limit_ns)
        self._dt = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}[dtype]
        cfg = self._cfg(m_cap)
        with torch.cuda.device(self.device):
            self.heap_bytes = self.lib.b200moe_ep_heap_bytes(C.byref(cfg), C.byref(self.ep))
            if self.heap_bytes == 0:
                raise ValueError("expert-parallel configuration not supported (FP8 block-scaled weights, "
                                 f"1..{_lib.EP_MAX_RANKS} ranks)")
            self.own = heaps is None
            self._opened = []
            if heaps is not None:
                self.heaps = heaps
            else:
                p = C.c_void_p()
                _lib.check(self.lib.b200moe_ep_heap_alloc(self.heap_bytes, C.byref(p)), "ep heap alloc")
                self.heaps = [None] * world
                self.heaps[rank] = p.value
                if world > 1:
                    handle = (C.c_ubyte * 64)()
                    _lib.check(self.lib.b200moe_ep_ipc_export(p, handle), "ep ipc export")
                    gathered = [None] * world
                    dist.all_gather_object(gathered, bytes(handle), group=group)
                    for r, hb in enumerate(gathered):
                        if r == rank:
                            continue
                        q = C.c_void_p()
                        buf = (C.c_ubyte * 64).from_buffer_copy(hb)
                        _lib.check(self.lib.b200moe_ep_ipc_open(buf, C.byref(q)), f"ep ipc open (rank {r})")
                        self.heaps[r] = q.value
                        self._opened.append(q.value)
                    dist.barrier(group=group)
            ws_bytes = self.lib.b200moe_ep_workspace_bytes(C.byref(cfg), C.byref(self.ep))
            self.ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._placement = {}

    @classmethod
    def emulate(cls, world: int, m_cap: int, h: int, i: int, topk: int, n_local: int, n_global: int, device,
                dtype=torch.bfloat16, wait_limit_ns: int = 0) -> list:
        """``world`` ranks driven from this one process on ONE device: every rank gets its own
        heap on that device and the "peer" heaps are simply the other ranks' heaps.  The caller
        runs the phases in order over all ranks in one stream (all dispatches, then all computes,
        then all combines), so every flag is raised before anything waits on it.  For tests and
        for debugging where a single GPU is at hand; ``ctxs[0].close_emulated(ctxs)`` frees."""
        from . import _lib
        lib = _lib.lib()
        nbytes = cls.heap_bytes_for(world, m_cap, h, i, topk, n_local, n_global)
        if nbytes == 0:
            raise ValueError("expert-parallel configuration not supported")
        heaps = []
        with torch.cuda.device(torch.device(device)):
            for _ in range(world):
                p = C.c_void_p()
                _lib.check(lib.b200moe_ep_heap_alloc(nbytes, C.byref(p)), "ep heap alloc")
                heaps.append(p.value)
        return [cls(r, world, m_cap, h, i, topk, n_local, n_global, device, dtype=dtype, heaps=heaps,
                    wait_limit_ns=wait_limit_ns) for r in range(world)]

    @staticmethod
    def close_emulated(ctxs: list) -> None:
        torch.cuda.synchronize(ctxs[0].device)
        with torch.cuda.device(ctxs[0].device):
            for hp in ctxs[0].heaps:
                if hp is not None:
                    ctxs[0].lib.b200moe_ep_heap_free(C.c_void_p(hp))
        for c in ctxs:
            c.heaps = [None] * c.world

    @staticmethod
    def heap_bytes_for(world, m_cap, h, i, topk, n_local, n_global) -> int:
        from . import _lib
        cfg = _lib.Cfg(C.sizeof(_lib.Cfg), m_cap, h, i, n_local, topk, _lib.DTYPE_BF16, _lib.W_FP8_BLOCK,
                       _lib.LAYOUT_LAYER, _lib.ACT_SILU, 0, 0, 1.0, 0, 0)
        ep = _lib.EpCfg(C.sizeof(_lib.EpCfg), world, 0, m_cap, n_global, 0, 0)
        return _lib.lib().b200moe_ep_heap_bytes(C.byref(cfg), C.byref(ep))

    def _cfg(self, m, activation=0, flags=0, routed_scaling=1.0):
        L = self._lib
        return L.Cfg(C.sizeof(L.Cfg), m, self.h, self.i, self.n_local, self.topk, self._dt, L.W_FP8_BLOCK,
                     L.LAYOUT_LAYER, activation, flags | self.flags, 0, routed_scaling, 0, 0)

    def placement_on_device(self, placement: torch.Tensor) -> torch.Tensor:
        key = id(placement)
        ent = self._placement.get(key)
        if ent is None or ent[0] is not placement:
            validate_placement(placement, self.world, self.n_local)
            ent = (placement, placement.to(device=self.device, dtype=torch.int32).contiguous())
            self._placement = {key: ent}
        return ent[1]

    def forward(self, x, w13q, w2q, w13_scale, w2_scale, topk_weights, topk_ids, placement, *, phases: int = 7,
                activation: str = "silu", apply_router_weight_on_input: bool = False,
                routed_scaling_factor: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        L = self._lib
        m = x.shape[0]
        assert x.is_cuda and x.shape[1] == self.h and m <= self.m_cap, "token batch exceeds the context's capacity"
        assert w13q.dtype == torch.float8_e4m3fn and w13q.shape == (self.n_local, 2 * self.i, self.h)
        assert w2q.dtype == torch.float8_e4m3fn and w2q.shape == (self.n_local, self.h, self.i)
        acts = {"silu": L.ACT_SILU, "gelu": L.ACT_GELU}
        if activation not in acts:
            raise ValueError(f"Unsupported FusedMoe activation: {activation}")
        flags = L.FLAG_WEIGHT_ON_INPUT if apply_router_weight_on_input else 0
        ids = topk_ids.contiguous()
        if ids.dtype == torch.int64:
            flags |= L.FLAG_IDS_I64
        else:
            assert ids.dtype == torch.int32
        tw = topk_weights.to(torch.float32).contiguous()
        xs = x.contiguous()
        s1, s2 = w13_scale.to(torch.float32).contiguous(), w2_scale.to(torch.float32).contiguous()
        quant = L.Quant(s1.data_ptr(), s2.data_ptr(), None, None)
        cfg = self._cfg(m, acts[activation], flags, float(routed_scaling_factor))
        if out is None:
            out = torch.empty(m, self.h, dtype=x.dtype, device=self.device)
        pl = self.placement_on_device(placement)
        heaps = (C.c_void_p * self.world)(*self.heaps)
        base = (self.ws.data_ptr() + 255) & ~255
        with torch.cuda.device(self.device):
            rc = self.lib.b200moe_ep_forward(
                C.byref(cfg), C.byref(self.ep), heaps, phases, xs.data_ptr(), w13q.data_ptr(), w2q.data_ptr(),
                C.byref(quant), tw.data_ptr(), ids.data_ptr(), pl.data_ptr(), base,
                self.ws.numel() - (base - self.ws.data_ptr()), out.data_ptr(), self.status.data_ptr(),
                torch.cuda.current_stream(self.device).cuda_stream)
        L.check(rc, "ep_forward")
        return out

    def check_status(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"b200moe: device-side wait timed out (code {code}) on rank {self.rank}")

    def close(self) -> None:
        """Unmap the peers' heaps and free this rank's (after a barrier, so that no peer still
        stores into it)."""
        if not self.own:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for q in self._opened:
                self.lib.b200moe_ep_ipc_close(C.c_void_p(q))
            self._opened = []
            if self.heaps[self.rank] is not None:
                self.lib.b200moe_ep_heap_free(C.c_void_p(self.heaps[self.rank]))
                self.heaps[self.rank] = None
        self.own = False


_contexts: dict = {}


def peer_context(group, m_cap, h, i, topk, n_local, n_global, device, dtype) -> EpContext:
    """The cached context of (group, shape): the heaps are allocated and mapped once."""
    key = (id(group), m_cap, h, i, topk, n_local, n_global, str(device), dtype)
    ctx = _contexts.get(key)
    if ctx is None:
        import os
        from . import _lib
        flags = _lib.FLAG_EP_DIAG_LOCAL_COMBINE if os.environ.get("B200MOE_EP_DIAG_LOCAL_COMBINE") == "1" else 0
        ctx = EpContext(dist.get_rank(group), dist.get_world_size(group), m_cap, h, i, topk, n_local, n_global,
                        device, dtype=dtype, group=group, flags=flags)
        _contexts[key] = ctx
    return ctx


def close_contexts() -> None:
    for ctx in list(_contexts.values()):
        ctx.close()
    _contexts.clear()

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


def _peer_protocol_over_collectives(hidden_states, w13_local, w2_local, topk_weights, topk_ids, placement, group,
                                    local_fn, **kwargs):
    """The data movement of ``mode="peer"`` written with collectives, for back ends without peer
    memory (the CPU tests of the index arithmetic run it over gloo): a fixed row per
    (source rank, token) on every destination, routing entries translated through the placement
    and masked per destination, rows sent only where an expert of the token lives (zeros
    elsewhere, which nothing may read), one output row per (token, choice) pair travelling back
    to the token's owner, who sums a token's rows in column order."""
    world = dist.get_world_size(group)
    m, h = hidden_states.shape
    k = topk_ids.shape[1]
    ids_t, w_t = dispatch_tables_placed(topk_ids, topk_weights, placement, world)          # [R, m, k]
    needed = (ids_t >= 0).any(dim=2)                                                       # [R, m]
    send_x = torch.where(needed[:, :, None], hidden_states.unsqueeze(0), torch.zeros((), dtype=hidden_states.dtype,
                                                                                     device=hidden_states.device))
    send_x = send_x.contiguous()
    recv_x = torch.empty_like(send_x)
    meta = torch.cat([ids_t, w_t.view(torch.int32)], dim=2).contiguous()
    recv_meta = torch.empty_like(meta)
    dist.all_to_all_single(recv_x, send_x, group=group)
    dist.all_to_all_single(recv_meta, meta, group=group)
    r_ids = recv_meta[:, :, :k].reshape(world * m, k).contiguous()
    r_w = recv_meta[:, :, k:].contiguous().view(torch.float32).reshape(world * m, k)
    pairs = local_fn(recv_x.view(world * m, h), w13_local, w2_local, r_w, r_ids, no_combine=True, **kwargs)
    back = torch.empty(world, m, k, h, dtype=pairs.dtype, device=pairs.device)
    dist.all_to_all_single(back, pairs.reshape(world, m, k, h).contiguous(), group=group)
    rows = back.float().sum(dim=0)            # a pair is computed on exactly one rank: the others sent zeros
    out = torch.zeros(m, h, dtype=torch.float32, device=rows.device)
    for j in range(k):
        out += rows[:, j]
    return out.to(hidden_states.dtype)


_contig: dict = {}


def _contiguous_placement(n_global: int, world: int) -> torch.Tensor:
    key = (n_global, world)
    if key not in _contig:
        _contig[key] = plan_placement(n_global, world)
    return _contig[key]


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
    placement: Optional[torch.Tensor] = None,
    **kwargs,
) -> torch.Tensor:
    """Expert-parallel fused MoE for this rank's tokens ``hidden_states [m, H]``.

    Every rank must call with the same ``m`` (pad the last batch if needed).
    ``local_fn(x, w13, w2, topk_weights, topk_ids, **kwargs)`` computes the local
    experts; it defaults to the CUDA operator of this package.
    ``placement`` (``plan_placement``): which rank holds which expert; ``w13_local`` / ``w2_local``
    then hold ``local_experts(placement, rank)`` in that order.  Default: contiguous.  The NCCL
    modes need a contiguous placement; ``mode="peer"`` takes any.
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
    peer_ok = (own_operator and hidden_states.is_cuda and bool(kwargs.get("use_fp8_w8a8")) and world <= 8
               and hidden_states.dtype in (torch.bfloat16, torch.float16))
    if mode is None:
        mode = "peer" if peer_ok else ("allgather" if world <= max(k, 2) else "alltoall")
    if mode == "peer" and not peer_ok:
        _last_collective = "peer protocol emulated with all-to-all (no peer memory on this back end)"
        if placement is None:
            placement = _contiguous_placement(e_loc * world, world)
        validate_placement(placement, world, e_loc)
        return _peer_protocol_over_collectives(hidden_states, w13_local, w2_local, topk_weights, topk_ids, placement,
                                               group, local_fn, **kwargs)
    if mode == "peer":
        _last_collective = ("none: rows stored into the peers' heaps over NVLink (dispatch), down-projection rows "
                            "stored into the owners' heaps from the GEMM epilogue (combine), epoch flags")
        i_dim = w2_local.shape[2]
        n_global = e_loc * world
        if placement is None:
            placement = _contiguous_placement(n_global, world)
        ctx = peer_context(group, m, h, i_dim, k, e_loc, n_global, hidden_states.device, hidden_states.dtype)
        extra = {kk: kwargs[kk] for kk in ("activation", "apply_router_weight_on_input", "routed_scaling_factor")
                 if kk in kwargs}
        return ctx.forward(hidden_states, w13_local, w2_local, kwargs["w13_scale"], kwargs["w2_scale"], topk_weights,
                           topk_ids, placement, **extra)
    assert placement is None or torch.equal(placement.cpu(), _contiguous_placement(e_loc * world, world)), \
        "the collective modes need the contiguous expert partition"
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
