"""GPU: expert parallelism by peer stores (`b200moe_ep_forward`).

On ONE device: several ranks driven from one process, each with its own heap on that device,
phase by phase in one stream (all dispatches, all computes, all combines), so that every flag
is raised before anything waits on it -- the whole data path (placement, masked routing rows,
fixed row per (source, token), the down projection storing each pair's row on the owner's heap,
the owner's fixed-order sum) runs exactly as it does across GPUs, only the stores stay on one
device.  The result must be bit-identical to the single-GPU operator wherever that one, too,
stores one row per pair (no fp32 atomics), and within tolerance of the oracle everywhere.

On two devices: the same through CUDA IPC mappings, one process per GPU.

A flag that is never raised: the bounded wait runs out, the status word says so, nothing hangs,
and the heaps work again afterwards."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as OM
from parity import assert_parity

pytestmark = pytest.mark.gpu


def _case(h, i, e, k, m, seed, skew=True):
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(h, i, e, seed=seed)
    x, tw, ids = make_tokens(m, h, e, k, seed=seed, skew=skew)
    w13q, s13 = quantize_fp8_block(w13)
    w2q, s2 = quantize_fp8_block(w2)
    return x, tw, ids, w13q, s13, w2q, s2


def _run_emulated(d, world, placement, x, tw, ids, w13q, s13, w2q, s2, m_cap=None, held=None, **kw):
    """`held`: the placement that says which experts each rank's weight shard holds (default: `placement`)."""
    from flaggems_sglang_b200 import ep
    m_all, h = x.shape
    e, i = w13q.shape[0], w2q.shape[2]
    k = ids.shape[1]
    m = m_all // world
    n_local = e // world
    ctxs = ep.EpContext.emulate(world, m_cap or m, h, i, k, n_local, e, d)
    try:
        shards, toks = [], []
        for r in range(world):
            mine = ep.local_experts(placement if held is None else held, r)
            shards.append(tuple(t[mine].contiguous().to(d) for t in (w13q, s13, w2q, s2)))
            toks.append(tuple(t[r * m:(r + 1) * m].contiguous().to(d) for t in (x, tw, ids)))
        outs = [torch.empty(m, h, dtype=x.dtype, device=d) for _ in range(world)]
        for phase in (1, 2, 4):
            for r in range(world):
                (a13, as13, a2, as2), (xr, twr, idr) = shards[r], toks[r]
                ctxs[r].forward(xr, a13, a2, as13, as2, twr, idr, placement, phases=phase, out=outs[r], **kw)
        torch.cuda.synchronize()
        for c in ctxs:
            c.check_status()
        return torch.cat(outs)
    finally:
        ep.EpContext.close_emulated(ctxs)


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("shape", [(512, 256, 16, 4, 48), (2048, 256, 16, 8, 640)],
                         ids=["decode-sized (fp32 rows added on the owner)", "prefill-sized (pair rows stored on the owner)"])
@pytest.mark.parametrize("balanced", [False, True], ids=["contiguous", "load-balanced"])
def test_emulated_ranks_match_single_gpu(cuda_device, world, shape, balanced):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import ep
    h, i, e, k, m = shape
    x, tw, ids, w13q, s13, w2q, s2 = _case(h, i, e, k, m, seed=77)
    d = cuda_device
    load = torch.bincount(ids.flatten().long(), minlength=e).tolist() if balanced else None
    placement = ep.plan_placement(e, world, load)
    out = _run_emulated(d, world, placement, x, tw, ids, w13q, s13, w2q, s2, routed_scaling_factor=1.25)
    single = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), use_fp8_w8a8=True,
                             w13_scale=s13.to(d), w2_scale=s2.to(d), routed_scaling_factor=1.25)
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(out, (ref.float() * 1.25).to(ref.dtype), what=f"ep emulated world={world} {shape}")
    if m * k >= 4096:
        assert torch.equal(out, single), "pair rows: expert parallelism must reproduce the single-GPU bits"
    else:
        torch.testing.assert_close(out.float(), single.float(), rtol=2e-2, atol=2e-3)


def test_emulated_partial_batch_and_dropped_expert(cuda_device):
    """A rank with fewer tokens than the capacity, and an expert the placement holds nowhere."""
    from flaggems_sglang_b200 import ep
    h, i, e, k, m = 512, 256, 8, 2, 40
    x, tw, ids, w13q, s13, w2q, s2 = _case(h, i, e, k, m, seed=3)
    held = ep.plan_placement(e, 2)
    placement = held.clone()
    placement[5] = -1
    out = _run_emulated(cuda_device, 2, placement, x, tw, ids, w13q, s13, w2q, s2, m_cap=32, held=held)
    tw_ref = torch.where(ids == 5, torch.zeros_like(tw), tw)
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw_ref, ids)
    assert_parity(out, ref, what="ep emulated, capacity 32 > 20 tokens per rank, expert 5 nowhere")


def test_flag_never_raised_times_out_and_recovers(cuda_device):
    from flaggems_sglang_b200 import ep
    h, i, e, k, m = 512, 256, 8, 2, 32
    x, tw, ids, w13q, s13, w2q, s2 = _case(h, i, e, k, m, seed=9)
    d = cuda_device
    world, mr = 2, m // 2
    placement = ep.plan_placement(e, world)
    ctxs = ep.EpContext.emulate(world, mr, h, i, k, e // world, e, d, wait_limit_ns=1_000_000)      # 1 ms
    try:
        shards = [tuple(t[ep.local_experts(placement, r)].contiguous().to(d) for t in (w13q, s13, w2q, s2))
                  for r in range(world)]
        toks = [tuple(t[r * mr:(r + 1) * mr].contiguous().to(d) for t in (x, tw, ids)) for r in range(world)]
        outs = [torch.empty(mr, h, dtype=x.dtype, device=d) for _ in range(world)]

        def run(r, phase):
            (a13, as13, a2, as2), (xr, twr, idr) = shards[r], toks[r]
            ctxs[r].forward(xr, a13, a2, as13, as2, twr, idr, placement, phases=phase, out=outs[r])

        # rank 1 never dispatches: rank 0's wait for its "ready" flag must run out after ~1 ms
        run(0, 1)
        run(0, 2)
        torch.cuda.synchronize()                       # returned by itself
        assert int(ctxs[0].status.item()) == 104
        with pytest.raises(RuntimeError, match="timed out"):
            ctxs[0].check_status()
        run(0, 4)                                      # "done" from rank 1 never comes either
        torch.cuda.synchronize()
        assert int(ctxs[0].status.item()) == 104
        ctxs[0].status.zero_()
        # rank 1 catches up with the call it missed (its epoch), then a complete call works
        for phase in (1, 2, 4):
            run(1, phase)
        torch.cuda.synchronize()
        ctxs[1].status.zero_()
        for phase in (1, 2, 4):
            for r in range(world):
                run(r, phase)
        torch.cuda.synchronize()
        for c in ctxs:
            c.check_status()
        ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
        assert_parity(torch.cat(outs), ref, what="ep after a provoked peer time-out")
    finally:
        ep.EpContext.close_emulated(ctxs)


# ------------------------------------------------------------------ two real GPUs, one process each
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, shape, balanced, ret):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "flaggems-sglang_b200", root / "tests"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flaggems_sglang_b200 as F
        from flaggems_sglang_b200 import ep
        h, i, e, k, m = shape
        x, tw, ids, w13q, s13, w2q, s2 = _case(h, i, e, k, m, seed=h)
        load = torch.bincount(ids.flatten().long(), minlength=e).tolist() if balanced else None
        placement = ep.plan_placement(e, world, load)
        mine = ep.local_experts(placement, rank)
        mr = m // world
        sl = slice(rank * mr, (rank + 1) * mr)
        kw = dict(use_fp8_w8a8=True, w13_scale=s13[mine].contiguous().to(dev), w2_scale=s2[mine].contiguous().to(dev))
        for _ in range(3):           # several calls in a row: the epochs advance, the heaps are reused
            out = ep.ep_fused_experts(x[sl].to(dev), w13q[mine].contiguous().to(dev), w2q[mine].contiguous().to(dev),
                                      tw[sl].to(dev), ids[sl].to(dev), mode="peer", placement=placement, **kw)
        torch.cuda.synchronize()
        for c in ep._contexts.values():
            c.check_status()
        single = F.fused_experts(x.to(dev), w13q.to(dev), w2q.to(dev), tw.to(dev), ids.to(dev), use_fp8_w8a8=True,
                                 w13_scale=s13.to(dev), w2_scale=s2.to(dev))
        F.check_status()
        ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids).float()[sl]
        err = (out.float().cpu() - ref).abs()
        ret[rank] = (float(err.max()), float(ref.abs().max()), float((err <= 1e-2 + 1e-2 * ref.abs()).float().mean()),
                     bool(torch.equal(out, single[sl])))
        ep.close_contexts()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(512, 256, 16, 4, 48), (2048, 256, 16, 8, 640)], ids=["decode-sized", "prefill-sized"])
@pytest.mark.parametrize("balanced", [False, True], ids=["contiguous", "load-balanced"])
def test_peer_mode_two_gpus(shape, balanced):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, shape, balanced, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            max_err, scale, frac, same_bits = ret[r]
            assert frac >= 0.99 and max_err <= 1e-2 * max(1.0, scale) + 1e-2 * scale, (r, ret[r])
            if shape[4] * shape[3] >= 4096:
                assert same_bits, f"rank {r}: pair rows must reproduce the single-GPU bits"


def test_emulated_call_replays_from_a_cuda_graph(cuda_device):
    """Nothing in the expert-parallel call reads device data on the host and the epoch lives in
    device memory, so the whole call -- all phases of all (emulated) ranks -- can be captured once
    and replayed; every replay opens a new epoch and gives the same bits."""
    from flaggems_sglang_b200 import ep
    h, i, e, k, m = 512, 256, 8, 2, 64
    x, tw, ids, w13q, s13, w2q, s2 = _case(h, i, e, k, m, seed=21)
    d = cuda_device
    world, mr = 2, m // 2
    placement = ep.plan_placement(e, world)
    ctxs = ep.EpContext.emulate(world, mr, h, i, k, e // world, e, d)
    try:
        shards = [tuple(t[ep.local_experts(placement, r)].contiguous().to(d) for t in (w13q, s13, w2q, s2))
                  for r in range(world)]
        toks = [tuple(t[r * mr:(r + 1) * mr].contiguous().to(d) for t in (x, tw, ids)) for r in range(world)]
        outs = [torch.empty(mr, h, dtype=x.dtype, device=d) for _ in range(world)]

        def call():
            for phase in (1, 2, 4):
                for r in range(world):
                    (a13, as13, a2, as2), (xr, twr, idr) = shards[r], toks[r]
                    ctxs[r].forward(xr, a13, a2, as13, as2, twr, idr, placement, phases=phase, out=outs[r])

        call()                                        # outside capture first (placement upload, lazy set-up)
        torch.cuda.synchronize()
        eager = torch.cat(outs).clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call()
        for _ in range(3):
            for o in outs:
                o.zero_()
            g.replay()
            torch.cuda.synchronize()
            for c in ctxs:
                c.check_status()
            assert torch.equal(torch.cat(outs), eager)
        assert_parity(eager, OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids), what="ep graph replay")
    finally:
        ep.EpContext.close_emulated(ctxs)
