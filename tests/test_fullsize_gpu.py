"""GPU: parity at the full sizes the benchmark numbers are quoted on.

Mixtral-8x7B-shaped bf16 at M = 1024 / 4096, the Qwen3-30B-A3B-shaped layer at its decode
sizes, the DeepSeek-V3-shaped FP8 layer with all 256 experts and the zipf-skewed routing at
M = 1 / 64 / 512 / 4096, and the Mixtral-shaped int4 AWQ layer with I = 14336 at
M = 1 / 32 / 256 / 2048 -- each against the CPU oracle on the same seeded inputs.

Weights are drawn (and quantised, with the product's offline quantisers, which CPU tests show
bit-equal to the oracle's) once per module on the GPU and copied to the host for the oracle;
the oracle's per-expert loop over a few thousand tokens takes seconds on the host cores.
FP8 and int4 have no reference implementation: "parity unpinned", the oracle is the guard.
"""
import gc

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import moe as OM
from oracle import quant as OQ
from parity import assert_parity

pytestmark = pytest.mark.gpu


def _free():
    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------ bf16
@pytest.fixture(scope="module")
def mixtral(cuda_device):
    from flaggems_sglang_b200.testing import CONFIGS, make_weights
    h, i, e, k = CONFIGS["mixtral"]
    w13, w2 = make_weights(h, i, e, device=cuda_device, seed=0)
    host = (w13.cpu().float(), w2.cpu().float())        # fp32 once: the oracle converts per expert otherwise
    yield (h, i, e, k, w13, w2, host)
    del w13, w2, host
    _free()


@pytest.mark.parametrize("M", [1024, 4096])
def test_mixtral_bf16_prefill_sizes(cuda_device, mixtral, M):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, k, w13, w2, (w13f, w2f) = mixtral
    x, tw, ids = make_tokens(M, h, e, k, seed=0)
    d = cuda_device
    out = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    again = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    F.check_status()
    ref = OM.fused_experts(x, w13f, w2f, tw, ids)
    assert_parity(out, ref, what=f"mixtral bf16 M={M}")
    if M >= 4096:
        # with this many pairs the combine sums a token's stored rows in a fixed order: a rerun gives the same bits
        assert torch.equal(out, again), "rerun differs"


@pytest.fixture(scope="module")
def qwen3(cuda_device):
    from flaggems_sglang_b200.testing import CONFIGS, make_weights
    h, i, e, k = CONFIGS["qwen3-30b-a3b"]
    w13, w2 = make_weights(h, i, e, device=cuda_device, seed=0)
    host = (w13.cpu().float(), w2.cpu().float())
    yield (h, i, e, k, w13, w2, host)
    del w13, w2, host
    _free()


@pytest.mark.parametrize("M", [8, 64, 128])
def test_qwen3_bf16_decode_sizes(cuda_device, qwen3, M):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, k, w13, w2, (w13f, w2f) = qwen3
    x, tw, ids = make_tokens(M, h, e, k, seed=0)
    d = cuda_device
    out = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    F.check_status()
    ref = OM.fused_experts(x, w13f, w2f, tw, ids)
    assert_parity(out, ref, what=f"qwen3 bf16 M={M}")


# ------------------------------------------------------------------ reference shapes at M = 2048 / 4096
@pytest.mark.parametrize("M", [2048, 4096])
def test_reference_large_shapes(cuda_device, M):
    """The two largest shapes of the reference's own test list (tests/accuracy_utils.py:107-118)."""
    import flaggems_sglang
    from test_fused_moe_gpu import _ref_inputs, _run_reference_api
    shape = (M, 1280, 3072, 64, 8)
    x, w1, w2, tw, ids = _ref_inputs(*shape, cuda_device)
    out = _run_reference_api(x, w1, w2, tw, ids, 64, cuda_device)
    assert out.shape == (M, 1280) and out.dtype == torch.bfloat16
    ref = OM.fused_experts(x, w1.transpose(1, 2).float(), w2.transpose(1, 2).float(), tw, ids)
    assert_parity(out, ref, what=f"reference shape {shape}")
    # the oracle itself against the reference's recorded output (every 16th row), at this size
    gold = np.load(GOLDEN / "fused_moe_ref_golden.npz")
    key = "M%d_K%d_N%d_E%d_topk%d/out_rows16" % shape
    if key in gold.files:
        g = torch.from_numpy(gold[key]).view(torch.bfloat16)
        st = assert_parity(ref[::16], g, what=f"oracle vs recorded reference output, {key}")
        assert st["bit_equal"] >= 0.9, f"oracle pin at {key}: {st['bit_equal']:.4f} bit-identical"


# ------------------------------------------------------------------ FP8, DeepSeek-V3 shape, all 256 experts
@pytest.fixture(scope="module")
def dsv3(cuda_device):
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import CONFIGS, make_weights
    h, i, e, k = CONFIGS["deepseek-v3"]
    parts = [[], [], [], []]
    for ei in range(e):                      # expert by expert keeps the bf16 temporaries small
        a, b = make_weights(h, i, e, device=cuda_device, seed=0, expert_ids=[ei])
        for lst, t in zip(parts, (*quantize_fp8_block(a), *quantize_fp8_block(b))):
            lst.append(t)
    w13q, s13, w2q, s2 = (torch.cat(p, dim=0).contiguous() for p in parts)
    del parts
    host = tuple(t.cpu() for t in (w13q, s13, w2q, s2))
    yield (h, i, e, k, w13q, s13, w2q, s2, host)
    del w13q, s13, w2q, s2, host
    _free()


@pytest.mark.parametrize("M", [1, 64, 512, 4096])
def test_deepseek_v3_fp8_full_layer(cuda_device, dsv3, M):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, k, w13q, s13, w2q, s2, (hw13, hs13, hw2, hs2) = dsv3
    x, tw, ids = make_tokens(M, h, e, k, seed=0, skew=True)      # zipf-skewed routing over the 256 experts
    d = cuda_device
    out = F.fused_experts(x.to(d), w13q, w2q, tw.to(d), ids.to(d), use_fp8_w8a8=True, w13_scale=s13, w2_scale=s2)
    F.check_status()
    ref = OM.fused_experts_fp8(x, hw13, hw2, hs13, hs2, tw, ids)
    assert_parity(out, ref, what=f"deepseek-v3 fp8 E=256 zipf M={M}")


# ------------------------------------------------------------------ int4 AWQ, Mixtral shape, I = 14336
@pytest.fixture(scope="module")
def mixtral_awq(cuda_device):
    from flaggems_sglang_b200.quant import quantize_awq, repack_awq_for_kernel
    from flaggems_sglang_b200.testing import CONFIGS, make_weights
    h, i, e, k = CONFIGS["mixtral"]
    parts = [[], [], [], []]
    w13f = torch.empty(e, 2 * i, h, dtype=torch.float32)        # the oracle's dequantised weights, once
    w2f = torch.empty(e, h, i, dtype=torch.float32)
    for ei in range(e):
        a, b = make_weights(h, i, e, dtype=torch.float16, device=cuda_device, seed=0, expert_ids=[ei])
        q1 = quantize_awq(a.transpose(1, 2).contiguous())       # AWQ layout [1, K, N]
        q2 = quantize_awq(b.transpose(1, 2).contiguous())
        for lst, t in zip(parts, (*repack_awq_for_kernel(*q1), *repack_awq_for_kernel(*q2))):
            lst.append(t)
        w13f[ei] = OQ.dequant_weight_awq(*[t[0].cpu() for t in q1]).t()
        w2f[ei] = OQ.dequant_weight_awq(*[t[0].cpu() for t in q2]).t()
        del a, b, q1, q2
    p1, z1, p2, z2 = (torch.cat(p, dim=0).contiguous() for p in parts)
    yield (h, i, e, k, p1, z1, p2, z2, w13f, w2f)
    del p1, z1, p2, z2, w13f, w2f
    _free()


@pytest.mark.parametrize("M", [1, 32, 256, 2048])
def test_mixtral_int4_awq_full_layer(cuda_device, mixtral_awq, M):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, k, p1, z1, p2, z2, w13f, w2f = mixtral_awq
    x, tw, ids = make_tokens(M, h, e, k, dtype=torch.float16, seed=0)
    d = cuda_device
    out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), use_int4_w4a16=True, w13_sz=z1, w2_sz=z2)
    F.check_status()
    # same arithmetic as oracle.moe.fused_experts_awq, with the weights dequantised once for all M
    ref = OM.fused_experts(x, w13f, w2f, tw, ids)
    assert out.dtype == torch.float16
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what=f"mixtral int4 awq I=14336 M={M}")
