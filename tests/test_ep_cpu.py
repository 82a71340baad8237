"""CPU, two gloo ranks: the dispatch / combine plumbing of expert parallelism.
The local experts are computed by the oracle here (the product has no CPU path);
what is checked is the index math: masked top-k tables, fixed-slot all-to-all,
per-rank partial sums and their combination."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_local(x, w13, w2, tw, ids, expert_map=None, **kw):
    from oracle import moe as OM
    ids = ids.to(torch.int64)
    if expert_map is not None:
        ids = expert_map.to(torch.int64)[ids]
    return OM.fused_experts(x, w13, w2, tw, ids, mimic_rounding=False)


def _oracle_pairs(x, w13, w2, tw, ids, no_combine=False, **kw):
    from oracle import moe as OM
    return OM.fused_experts(x, w13, w2, tw, ids.to(torch.int64), mimic_rounding=False, no_combine=no_combine)


def _worker_peer(rank, world, port, balanced, ret):
    """The peer-store protocol's index arithmetic over gloo: placement -> masked routing rows ->
    fixed row per (source, token) -> pair rows back to the owner."""
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "flaggems-sglang_b200"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flaggems_sglang_b200 import ep
        from flaggems_sglang_b200.testing import make_tokens, make_weights
        from oracle import moe as OM
        h, i, e, k, m = 64, 32, 8, 3, 10
        w13, w2 = make_weights(h, i, e, dtype=torch.float32, seed=0, scale=0.1)
        xs, tws, idss = zip(*[make_tokens(m, h, e, k, dtype=torch.float32, seed=20 + r, skew=True) for r in range(world)])
        load = torch.bincount(torch.cat(idss).flatten().long(), minlength=e).tolist() if balanced else None
        placement = ep.plan_placement(e, world, load)
        mine = ep.local_experts(placement, rank)
        ref = OM.fused_experts(xs[rank], w13, w2, tws[rank], idss[rank], mimic_rounding=False)
        out = ep.ep_fused_experts(xs[rank], w13[mine].contiguous(), w2[mine].contiguous(), tws[rank], idss[rank],
                                  local_fn=_oracle_pairs, mode="peer", placement=placement)
        err = float((out - ref).abs().max())
        # an expert that the placement leaves out (negative entry) is dropped on every rank alike
        holes = placement.clone()
        holes[3] = -1
        tw_ref = torch.where(idss[rank] == 3, torch.zeros_like(tws[rank]), tws[rank])
        ref2 = OM.fused_experts(xs[rank], w13, w2, tw_ref, idss[rank], mimic_rounding=False)
        out2 = ep.ep_fused_experts(xs[rank], w13[mine].contiguous(), w2[mine].contiguous(), tws[rank], idss[rank],
                                   local_fn=_oracle_pairs, mode="peer", placement=holes)
        err = max(err, float((out2 - ref2).abs().max()))
        # a corrupted table (two experts on one place; a rank that does not exist) is refused on the host
        bad = placement.clone()
        bad[0] = bad[1]
        refused = 0
        for table in (bad, torch.where(torch.arange(e) == 2, torch.tensor((world + 3) << 16), placement)):
            try:
                ep.ep_fused_experts(xs[rank], w13[mine].contiguous(), w2[mine].contiguous(), tws[rank], idss[rank],
                                    local_fn=_oracle_pairs, mode="peer", placement=table.to(torch.int32))
            except ValueError:
                refused += 1
        ret[rank] = (err, refused)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
@pytest.mark.parametrize("balanced", [False, True], ids=["contiguous", "load-balanced"])
def test_peer_protocol_two_cpu_ranks(balanced):
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker_peer, args=(world, port, balanced, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            err, refused = ret[r]
            assert err < 1e-5, f"rank {r}: max abs err {err}"
            assert refused == 2, f"rank {r}: corrupted placements accepted"


def test_placement_planning():
    from flaggems_sglang_b200 import ep
    p = ep.plan_placement(16, 4)
    assert (p >> 16).tolist() == [e // 4 for e in range(16)] and (p & 0xFFFF).tolist() == [e % 4 for e in range(16)]
    load = [100, 90, 80, 70] + [1] * 12
    b = ep.plan_placement(16, 4, load)
    ep.validate_placement(b, 4, 4)
    assert sorted((b[:4] >> 16).tolist()) == [0, 1, 2, 3]            # the four hot experts sit on four different ranks
    per_rank = [sum(load[e] for e in ep.local_experts(b, r)) for r in range(4)]
    assert max(per_rank) - min(per_rank) <= 30 and all(len(ep.local_experts(b, r)) == 4 for r in range(4))
    # the dispatch tables against a plain loop
    ids = torch.tensor([[0, 5, 9], [3, 15, 1], [7, 7, 2]])
    w = torch.rand(3, 3)
    t_ids, t_w = ep.dispatch_tables_placed(ids, w, b, 4)
    for t in range(3):
        for j in range(3):
            v = int(b[ids[t, j]])
            for r in range(4):
                want = (v & 0xFFFF) if (v >> 16) == r else -1
                assert int(t_ids[r, t, j]) == want
                assert float(t_w[r, t, j]) == (float(w[t, j]) if want >= 0 else 0.0)
    with pytest.raises(ValueError):
        ep.validate_placement(torch.tensor([0, 0, 1 << 16, (1 << 16) | 1], dtype=torch.int32), 2, 2)
    with pytest.raises(ValueError):
        ep.validate_placement(torch.tensor([0, 1, 5 << 16, (1 << 16) | 1], dtype=torch.int32), 2, 2)


def _worker(rank, world, port, ret):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    for p in (root, root / "flaggems-sglang_b200"):
        sys.path.insert(0, str(p))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flaggems_sglang_b200.ep import ep_fused_experts
        from flaggems_sglang_b200.testing import make_tokens, make_weights
        from oracle import moe as OM
        h, i, e, k, m = 64, 32, 8, 3, 10
        e_loc = e // world
        w13, w2 = make_weights(h, i, e, dtype=torch.float32, seed=0, scale=0.1)
        xs, tws, idss = zip(*[make_tokens(m, h, e, k, dtype=torch.float32, seed=10 + r) for r in range(world)])
        ref = OM.fused_experts(xs[rank], w13, w2, tws[rank], idss[rank], mimic_rounding=False)
        err = 0.0
        for mode in ("alltoall", "allgather"):
            out = ep_fused_experts(xs[rank], w13[rank * e_loc:(rank + 1) * e_loc].contiguous(),
                                   w2[rank * e_loc:(rank + 1) * e_loc].contiguous(), tws[rank], idss[rank],
                                   local_fn=_oracle_local, mode=mode)
            err = max(err, float((out - ref).abs().max()))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_ep_dispatch_combine_two_cpu_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            assert ret[r] < 1e-5, f"rank {r}: max abs err {ret[r]}"


def test_dispatch_tables_mask():
    import sys
    from flaggems_sglang_b200.ep import dispatch_tables
    ids = torch.tensor([[0, 5], [7, 2], [3, 4]])
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5], [0.1, 0.9]])
    t_ids, t_w = dispatch_tables(ids, w, 4, 2)
    assert t_ids.tolist() == [[[0, -1], [-1, 2], [3, -1]], [[-1, 1], [3, -1], [-1, 0]]]
    assert torch.allclose(t_w[0], torch.tensor([[0.25, 0.0], [0.0, 0.5], [0.1, 0.0]]))
    assert torch.allclose(t_w.sum(0), w)
