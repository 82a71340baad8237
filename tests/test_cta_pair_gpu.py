"""GPU: the 16-bit prefill GEMMs on CTA pairs (tcgen05.mma.cta_group::2, B200MOE_CTA_PAIR=1)
against the oracle and against the one-CTA-per-tile kernels.  Shapes with odd numbers of
128-token blocks per expert (the second half of a pair tile is then empty), several n-tiles,
ragged K, and the pair-row and fp32-atomic epilogues."""
import pytest
import torch

from oracle import moe as OM
from parity import assert_parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("h,i,e,k,m,dtype", [(512, 384, 8, 2, 300, torch.bfloat16), (1024, 512, 4, 2, 1100, torch.bfloat16),
                                              (2048, 1024, 8, 2, 4800, torch.bfloat16), (520, 264, 3, 1, 700, torch.float16)])
def test_cta_pairs_match_oracle_and_single_cta(cuda_device, monkeypatch, h, i, e, k, m, dtype):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(h, i, e, dtype=dtype, seed=h + m, scale=0.05)
    x, tw, ids = make_tokens(m, h, e, k, dtype=dtype, seed=h + m)
    d = cuda_device
    args = (x.to(d), w13.to(d), w2.to(d), tw.to(d), ids.to(d))
    single = F.fused_experts(*args, block_tokens=128)
    F.check_status()
    monkeypatch.setenv("B200MOE_CTA_PAIR", "1")
    pair = F.fused_experts(*args, block_tokens=128)
    again = F.fused_experts(*args, block_tokens=128)
    torch.cuda.synchronize()
    F.check_status()
    assert any("tc2" in n for n in _lib.launch_stats()[1]), _lib.launch_stats()[1]
    ref = OM.fused_experts(x, w13, w2, tw, ids)
    assert_parity(pair, ref, what=f"cta pairs {(h, i, e, k, m)}")
    # same MMAs in the same order: wherever nothing is summed by atomics the bits agree
    if "finalize_pairs_kernel" in _lib.launch_stats()[1]:
        assert torch.equal(pair, single) and torch.equal(pair, again)
    else:
        torch.testing.assert_close(pair.float(), single.float(), rtol=2e-2, atol=2e-2)
