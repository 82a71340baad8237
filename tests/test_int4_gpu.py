"""GPU: int4 AWQ w4a16 (group 128, zero points, fp16 activations) against the CPU
oracle.  The reference has no int4 path at all (its signature carries no zero
points, src/flaggems_sglang/ops/fused_moe.py:133-152): "parity unpinned".
Tolerance for this mode: rtol = atol = 2e-2."""
import pytest
import torch

from oracle import moe as OM
from parity import assert_parity

pytestmark = pytest.mark.gpu


def _case(h, i, e, k, m, seed):
    from flaggems_sglang_b200.quant import quantize_awq
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(h, i, e, dtype=torch.float16, seed=seed)
    x, tw, ids = make_tokens(m, h, e, k, dtype=torch.float16, seed=seed)
    # AWQ layout: [E, K, N] with K the reduction dim
    q1 = quantize_awq(w13.transpose(1, 2).contiguous())
    q2 = quantize_awq(w2.transpose(1, 2).contiguous())
    return x, tw, ids, q1, q2


@pytest.mark.parametrize("h,i,e,k,m", [(256, 256, 4, 2, 20), (512, 384, 8, 2, 100), (1024, 512, 8, 2, 1),
                                        (4096, 1024, 8, 2, 32), (1024, 512, 8, 2, 600)])
def test_int4_fused_experts(cuda_device, h, i, e, k, m):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.quant import repack_awq_for_kernel
    x, tw, ids, q1, q2 = _case(h, i, e, k, m, seed=h + m)
    d = cuda_device
    p1, z1 = repack_awq_for_kernel(*[t.to(d) for t in q1])
    p2, z2 = repack_awq_for_kernel(*[t.to(d) for t in q2])
    assert p1.shape == (e, 2 * i, h // 8) and z1.shape == (e, h // 128, 2 * i)
    out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), use_int4_w4a16=True, w13_sz=z1, w2_sz=z2)
    F.check_status()
    ref = OM.fused_experts_awq(x, *q1, *q2, tw, ids)
    assert out.dtype == torch.float16
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what=f"int4 {(h, i, e, k, m)}")


@pytest.mark.parametrize("bt", [16, 32, 64, 128, 256])
def test_int4_every_token_block(cuda_device, bt):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.quant import repack_awq_for_kernel
    x, tw, ids, q1, q2 = _case(512, 256, 4, 2, 300, seed=bt)
    d = cuda_device
    p1, z1 = repack_awq_for_kernel(*[t.to(d) for t in q1])
    p2, z2 = repack_awq_for_kernel(*[t.to(d) for t in q2])
    out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), use_int4_w4a16=True, w13_sz=z1, w2_sz=z2,
                          block_tokens=bt)
    F.check_status()
    ref = OM.fused_experts_awq(x, *q1, *q2, tw, ids)
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what=f"int4 BT={bt}")


def test_int4_through_reference_signature(cuda_device):
    """AWQ checkpoint tensors straight into the op-level entry point (keyword-only extension)."""
    import flaggems_sglang
    x, tw, ids, q1, q2 = _case(512, 256, 8, 2, 40, seed=4)
    d = cuda_device
    rd, gi, si = flaggems_sglang.topk_to_routing(tw.to(d), ids.to(d), 8)
    out = flaggems_sglang.triton_kernel_fused_experts(
        x.to(d), q1[0].to(d), q2[0].to(d), rd, gi, si, w1_scale=q1[1].to(d), w2_scale=q2[1].to(d),
        use_int4_w4a16=True, w1_zp=q1[2].to(d), w2_zp=q2[2].to(d))
    flaggems_sglang.check_status()
    ref = OM.fused_experts_awq(x, *q1, *q2, tw, ids)
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what="int4 reference signature")


@pytest.mark.parametrize("m,bt", [(20, 16), (60, 32), (300, 64), (300, 128)])
def test_int4_bias_and_clamped_swiglu(cuda_device, m, bt):
    """Per-expert biases and the bias variant's activation on both int4 kernels (integer MMAs for
    blocks of 16 / 32 tokens, fp16 operands above)."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.quant import repack_awq_for_kernel
    h, i, e, k = 512, 256, 4, 2
    x, tw, ids, q1, q2 = _case(h, i, e, k, m, seed=m + bt)
    g = torch.Generator().manual_seed(m)
    b13 = (torch.randn(e, 2 * i, generator=g) * 0.5).to(torch.float16)
    b2 = (torch.randn(e, h, generator=g) * 0.5).to(torch.float16)
    d = cuda_device
    p1, z1 = repack_awq_for_kernel(*[t.to(d) for t in q1])
    p2, z2 = repack_awq_for_kernel(*[t.to(d) for t in q2])
    out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), use_int4_w4a16=True, w13_sz=z1, w2_sz=z2,
                          activation="swiglu_oai", b13=b13.to(d), b2=b2.to(d), swiglu_alpha=1.702, swiglu_limit=7.0,
                          block_tokens=bt)
    F.check_status()
    ref = OM.fused_experts_awq(x, *q1, *q2, tw, ids, activation="swiglu_oai", b1=b13, b2=b2, swiglu_alpha=1.702,
                               swiglu_limit=7.0)
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what=f"int4 bias M={m} BT={bt}")
