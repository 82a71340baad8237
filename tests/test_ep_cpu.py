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
