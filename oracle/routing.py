"""Integer routing / alignment oracle (numpy, CPU).  Test infrastructure only.

Two formats are produced from the same ``topk_ids``:

* the *routing triple* the reference builds in
  ``_standard_topk_to_triton_kernels`` (src/flaggems_sglang/ops/fused_moe.py:103-130)
  together with the expert-data tables of the dependency it calls
  (``compute_expt_data_torch``: histogram, raw offsets, per-block-size padded
  offsets and block maps);
* the *block-aligned* format (``sorted_token_ids``, ``expert_ids``,
  ``num_tokens_post_padded``) that MoE GEMMs in the serving ecosystem consume.

Everything here is written with explicit loops or a stable argsort so that it
can be checked by eye; speed does not matter.
"""
from __future__ import annotations

import numpy as np

BLOCK_MS = (16, 32, 64, 128)


def _as_np(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu()
        if a.dtype.is_floating_point:
            a = a.float()
        a = a.numpy()
    return np.asarray(a)


def max_tiles(n_gates: int, n_experts: int, min_block: int = 16) -> int:
    """Upper bound on the number of row blocks over every supported block size.

    Follows the dependency's bound: if there are no more slots than experts,
    every slot can be its own block; otherwise the worst case puts one slot in
    each of E-1 experts and the rest in the last one.
    """
    if n_gates <= n_experts:
        return n_gates
    # python floor division on a negative numerator, as upstream writes it
    return n_experts - 1 - ((n_experts - n_gates - 1) // min_block)


def topk_to_routing(topk_weights, topk_ids, n_experts: int) -> dict:
    """Restates fused_moe.py:112-130.

    Returns a dict of numpy arrays:
      expt_indx   [P] int32  per-token-sorted expert ids, flattened
      topk_indx   [P] int32  stable argsort of expt_indx (sorted row -> slot)
      gate_indx   [P] int32  inverse permutation (slot -> sorted row)
      gate_scal   [P]        routing weights in sorted-row order
      hist        [E] int32
      token_offs_raw [E+1] int32
      token_offs_pad {bm: [E+1] int32}
      block_pid_map  {bm: [max_tiles] int32}   (block << 16) | expert, -1 padded
    """
    w = _as_np(topk_weights)
    ids = _as_np(topk_ids).astype(np.int64)
    n_tokens, k = ids.shape
    n_gates = n_tokens * k

    # line 114-115: ascending sort of each token's experts, weights follow
    order = np.argsort(ids, axis=1, kind="stable")
    ids_sorted = np.take_along_axis(ids, order, axis=1)
    w_sorted = np.take_along_axis(w, order, axis=1)
    expt_indx = ids_sorted.reshape(-1).astype(np.int32)
    expt_scal = w_sorted.reshape(-1)

    # line 118-120
    topk_indx = np.argsort(expt_indx, kind="stable").astype(np.int32)
    gate_indx = np.argsort(topk_indx, kind="stable").astype(np.int32)
    gate_scal = expt_scal[topk_indx]

    # line 121-123 (histc over integer-valued floats == bincount)
    hist = np.bincount(expt_indx, minlength=n_experts)[:n_experts].astype(np.int32)

    token_offs_raw = np.zeros(n_experts + 1, dtype=np.int32)
    token_offs_raw[1:] = np.cumsum(hist)

    mt = max_tiles(n_gates, n_experts, min(BLOCK_MS))
    token_offs_pad = {}
    block_pid_map = {}
    for bm in BLOCK_MS:
        tiles = (hist + bm - 1) // bm
        offs = np.zeros(n_experts + 1, dtype=np.int32)
        offs[1:] = np.cumsum(tiles)
        token_offs_pad[bm] = offs
        bmap = np.full(mt, -1, dtype=np.int32)
        for e in range(n_experts):
            for b in range(int(tiles[e])):
                bmap[offs[e] + b] = (b << 16) + e
        block_pid_map[bm] = bmap

    return dict(
        expt_indx=expt_indx,
        topk_indx=topk_indx,
        gate_indx=gate_indx,
        gate_scal=gate_scal,
        hist=hist,
        token_offs_raw=token_offs_raw,
        token_offs_pad=token_offs_pad,
        block_pid_map=block_pid_map,
        n_expts_tot=n_experts,
        n_expts_act=k,
    )


def align_capacity(n_slots: int, n_experts: int, block: int) -> int:
    """Length of ``sorted_token_ids``: every non-empty expert wastes at most
    block-1 rows, and there cannot be more non-empty experts than slots."""
    cap = n_slots + n_experts * (block - 1)
    if n_slots < n_experts:
        cap = min(n_slots * block, cap)
    return cap


def moe_align_block_size(topk_ids, block: int, n_experts: int):
    """Block-aligned grouping of the raw slot ids ``i = token*k + j``.

    For expert 0..E-1 in turn: that expert's slot ids in ascending order, then
    the sentinel ``P`` (= number of slots) up to the next multiple of
    ``block``.  Slots whose expert id is outside [0, E) (masked for expert
    parallelism) are dropped.  Tail fill is part of this repo's contract:
    ``sorted_token_ids`` tail = P, ``expert_ids`` tail = -1.
    """
    ids = _as_np(topk_ids).astype(np.int64).reshape(-1)
    n_slots = ids.shape[0]
    cap = align_capacity(n_slots, n_experts, block)
    n_blocks_cap = (cap + block - 1) // block
    sorted_ids = np.full(cap, n_slots, dtype=np.int32)
    expert_ids = np.full(n_blocks_cap, -1, dtype=np.int32)
    pos = 0
    for e in range(n_experts):
        members = [i for i in range(n_slots) if ids[i] == e]
        if not members:
            continue
        sorted_ids[pos:pos + len(members)] = members
        padded = (len(members) + block - 1) // block * block
        expert_ids[pos // block:(pos + padded) // block] = e
        pos += padded
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)


def moe_align_block_size_fast(topk_ids, block: int, n_experts: int):
    """Same contract as :func:`moe_align_block_size`, vectorised with a stable
    argsort so that the full-size configurations finish in milliseconds."""
    ids = _as_np(topk_ids).astype(np.int64).reshape(-1)
    n_slots = ids.shape[0]
    cap = align_capacity(n_slots, n_experts, block)
    n_blocks_cap = (cap + block - 1) // block
    sorted_ids = np.full(cap, n_slots, dtype=np.int32)
    expert_ids = np.full(n_blocks_cap, -1, dtype=np.int32)
    valid = (ids >= 0) & (ids < n_experts)
    slots = np.nonzero(valid)[0]
    order = slots[np.argsort(ids[slots], kind="stable")]
    hist = np.bincount(ids[slots], minlength=n_experts)
    padded = (hist + block - 1) // block * block
    starts = np.concatenate([[0], np.cumsum(padded)])
    raw = np.concatenate([[0], np.cumsum(hist)])
    for e in range(n_experts):
        if hist[e]:
            sorted_ids[starts[e]:starts[e] + hist[e]] = order[raw[e]:raw[e + 1]]
            expert_ids[starts[e] // block:starts[e + 1] // block] = e
    return sorted_ids, expert_ids, np.array([starts[-1]], dtype=np.int32)
