"""GPU: alignment / routing kernels through the C ABI, bit-exact against the
oracle and against the reference's golden routing vectors."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import routing as R

pytestmark = pytest.mark.gpu

GOLD = np.load(GOLDEN / "routing_golden.npz")
CASES = sorted({k.split("/")[0] for k in GOLD.files})


def _rand_ids(m, k, e, seed, dtype=torch.int32):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(m)]) if m else torch.zeros(0, k)
    return ids.to(dtype)


@pytest.mark.parametrize("m,k,e,bs", [
    (1, 2, 8, 16), (7, 2, 8, 4), (33, 4, 16, 16), (64, 2, 8, 64), (17, 8, 64, 16), (1024, 8, 64, 128),
    (4096, 2, 8, 256), (256, 8, 128, 16), (4096, 8, 256, 128), (5, 1, 3, 128), (3, 2, 1000, 16),
    (2, 8, 128, 64), (0, 2, 8, 16),
])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_align_block_size_bit_exact(cuda_device, m, k, e, bs, dtype):
    import flaggems_sglang_b200 as F
    ids = _rand_ids(m, k, e, m * 7 + e, dtype)
    s, eid, n = F.moe_align_block_size(ids.to(cuda_device), bs, e)
    rs, re_, rn = R.moe_align_block_size_fast(ids.numpy(), bs, e)
    np.testing.assert_array_equal(n.cpu().numpy(), rn)
    np.testing.assert_array_equal(s.cpu().numpy(), rs)
    np.testing.assert_array_equal(eid.cpu().numpy(), re_)


def test_align_skewed_and_masked(cuda_device):
    import flaggems_sglang_b200 as F
    # all tokens pick the same two experts; then an expert map that keeps only experts 4..7
    ids = torch.tensor([[5, 1]] * 300, dtype=torch.int32)
    s, eid, n = F.moe_align_block_size(ids.to(cuda_device), 64, 8)
    rs, re_, rn = R.moe_align_block_size_fast(ids.numpy(), 64, 8)
    np.testing.assert_array_equal(s.cpu().numpy(), rs)
    np.testing.assert_array_equal(eid.cpu().numpy(), re_)
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3], dtype=torch.int32)
    ids2 = _rand_ids(50, 2, 8, 3)
    s, eid, n = F.moe_align_block_size(ids2.to(cuda_device), 16, 4, expert_map=emap.to(cuda_device))
    local = emap[ids2.long()].numpy()
    rs, re_, rn = R.moe_align_block_size_fast(local, 16, 4)
    k = int(rn[0])
    np.testing.assert_array_equal(n.cpu().numpy(), rn)
    np.testing.assert_array_equal(s.cpu().numpy()[:k], rs[:k])
    np.testing.assert_array_equal(eid.cpu().numpy()[:k // 16], re_[:k // 16])


def test_align_is_deterministic(cuda_device):
    import flaggems_sglang_b200 as F
    ids = _rand_ids(4096, 8, 256, 11).to(cuda_device)
    a = F.moe_align_block_size(ids, 128, 256)
    b = F.moe_align_block_size(ids, 128, 256)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("name", CASES)
def test_routing_from_topk_matches_reference_golden(cuda_device, name):
    import flaggems_sglang_b200 as F
    g = {k.split("/")[1]: GOLD[k] for k in GOLD.files if k.startswith(name + "/")}
    e = int(name.split("_")[1][1:])
    w = torch.from_numpy(g["topk_weights"]).to(cuda_device)
    ids = torch.from_numpy(g["topk_ids"]).to(cuda_device)
    rd, gi, si = F.topk_to_routing(w, ids, e)
    np.testing.assert_array_equal(rd.expt_hist.cpu().numpy(), g["hist"])
    np.testing.assert_array_equal(gi.src_indx.cpu().numpy(), g["topk_indx"])
    np.testing.assert_array_equal(gi.dst_indx.cpu().numpy(), g["gate_indx"])
    np.testing.assert_array_equal(si.src_indx.cpu().numpy(), g["gate_indx"])
    np.testing.assert_array_equal(rd.gate_scal.cpu().numpy(), g["gate_scal"])
    np.testing.assert_array_equal(rd.expt_data.token_offs_raw.cpu().numpy(), g["token_offs_raw"])
    for bm in R.BLOCK_MS:
        np.testing.assert_array_equal(rd.expt_data.token_offs_pad[bm].cpu().numpy(), g[f"token_offs_pad_{bm}"])
        np.testing.assert_array_equal(rd.expt_data.block_pid_map[bm].cpu().numpy(), g[f"block_pid_map_{bm}"])


@pytest.mark.parametrize("m,k,e", [(4096, 8, 256), (2048, 8, 64), (4096, 2, 8), (3, 8, 128)])
def test_routing_from_topk_full_size(cuda_device, m, k, e):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import route
    g = torch.Generator().manual_seed(m + e)
    w, ids = route(torch.randn(m, e, generator=g), k)
    rd, gi, si = F.topk_to_routing(w.to(cuda_device), ids.to(cuda_device), e)
    r = R.topk_to_routing(w.numpy(), ids.numpy(), e)
    np.testing.assert_array_equal(rd.expt_hist.cpu().numpy(), r["hist"])
    np.testing.assert_array_equal(gi.src_indx.cpu().numpy(), r["topk_indx"])
    np.testing.assert_array_equal(gi.dst_indx.cpu().numpy(), r["gate_indx"])
    np.testing.assert_array_equal(rd.gate_scal.cpu().numpy(), r["gate_scal"])
    for bm in R.BLOCK_MS:
        np.testing.assert_array_equal(rd.expt_data.token_offs_pad[bm].cpu().numpy(), r["token_offs_pad"][bm])
        np.testing.assert_array_equal(rd.expt_data.block_pid_map[bm].cpu().numpy(), r["block_pid_map"][bm])
    # size-independent property: gate_indx is the inverse permutation of topk_indx
    ti, gi_ = gi.src_indx.long(), gi.dst_indx.long()
    assert torch.equal(gi_[ti], torch.arange(m * k, device=cuda_device))
