"""GPU: FP8 (e4m3, 128x128 weight block scales, dynamic 1x128 activation groups)
path against the CPU oracle.  The reference rejects these arguments
(src/flaggems_sglang/ops/fused_moe.py:154-169), so parity here is against this
repository's restatement of the ecosystem's conventions only ("parity unpinned")."""
import numpy as np
import pytest
import torch

from oracle import moe as OM
from oracle import quant as Q
from parity import assert_parity

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,k", [(7, 512), (83, 4096), (300, 7168), (1, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_per_token_group_quant_bit_exact(cuda_device, rows, k, dtype):
    from flaggems_sglang_b200.ops.quant import per_token_group_quant_fp8
    g = torch.Generator().manual_seed(rows + k)
    x = (torch.randn(rows, k, generator=g) * 3).to(dtype)
    x[0, :128] = 0                                     # an all-zero group
    q, s = per_token_group_quant_fp8(x.to(cuda_device))
    rq, rs = Q.quant_act_fp8_group(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (rows, k // 128)
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))


def _fp8_case(h, i, e, k, m, seed, skew=False):
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(h, i, e, seed=seed)
    x, tw, ids = make_tokens(m, h, e, k, seed=seed, skew=skew)
    w13q, s13 = quantize_fp8_block(w13)
    w2q, s2 = quantize_fp8_block(w2)
    return x, tw, ids, w13q, s13, w2q, s2


@pytest.mark.parametrize("h,i,e,k,m", [(256, 256, 4, 2, 20), (512, 384, 8, 2, 100), (1024, 512, 8, 2, 64),
                                        (7168, 2048, 8, 4, 1), (7168, 2048, 16, 8, 64), (2048, 768, 32, 8, 300)])
def test_fp8_fused_experts(cuda_device, h, i, e, k, m):
    import flaggems_sglang_b200 as F
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(h, i, e, k, m, seed=h + m, skew=(e >= 16))
    d = cuda_device
    out = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), use_fp8_w8a8=True,
                          w13_scale=s13.to(d), w2_scale=s2.to(d))
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(out, ref, what=f"fp8 {(h, i, e, k, m)}")


@pytest.mark.parametrize("bt", [16, 32, 64, 128])
def test_fp8_every_token_block(cuda_device, bt):
    import flaggems_sglang_b200 as F
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(512, 256, 4, 2, 150, seed=bt)
    d = cuda_device
    out = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), use_fp8_w8a8=True,
                          w13_scale=s13.to(d), w2_scale=s2.to(d), block_tokens=bt)
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(out, ref, what=f"fp8 BT={bt}")


def test_fp8_through_reference_signature(cuda_device):
    """The reference's signature already carries use_fp8_w8a8 / w1_scale / w2_scale /
    block_shape (fused_moe.py:143-151) and asserts them away; here they work."""
    import flaggems_sglang
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(512, 256, 8, 2, 40, seed=9)
    d = cuda_device
    rd, gi, si = flaggems_sglang.topk_to_routing(tw.to(d), ids.to(d), 8)
    out = flaggems_sglang.triton_kernel_fused_experts(x.to(d), w13q.to(d), w2q.to(d), rd, gi, si, use_fp8_w8a8=True,
                                                      w1_scale=s13.to(d), w2_scale=s2.to(d), block_shape=[128, 128])
    flaggems_sglang.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(out, ref, what="fp8 reference signature")
    with pytest.raises(AssertionError):
        flaggems_sglang.triton_kernel_fused_experts(x.to(d), w13q.to(d), w2q.to(d), rd, gi, si, use_fp8_w8a8=True,
                                                    w1_scale=s13.to(d), w2_scale=s2.to(d), block_shape=[64, 64])


@pytest.mark.parametrize("masked", [False, True])
def test_fp8_many_pairs_stored_per_pair(cuda_device, masked):
    """Enough (token, choice) pairs that the down projection stores 16-bit rows per pair and the
    output conversion sums them (instead of fp32 atomics); with an expert map, masked pairs must
    contribute nothing."""
    import flaggems_sglang_b200 as F
    h, i, e, k, m = 2048, 256, 16, 8, 640           # 5120 pairs / 128 * 8 column tiles >= 2 * SMs
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(h, i, e, k, m, seed=77)
    d = cuda_device
    kw = dict(use_fp8_w8a8=True, w13_scale=s13.to(d), w2_scale=s2.to(d), routed_scaling_factor=1.5)
    if masked:
        emap = torch.arange(e, dtype=torch.int32)
        emap[1::3] = -1                              # every third expert lives elsewhere
        out = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), expert_map=emap.to(d), **kw)
        tw_ref = torch.where(emap[ids.long()] >= 0, tw, torch.zeros_like(tw))
    else:
        out = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), **kw)
        tw_ref = tw
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw_ref, ids)
    assert_parity(out, (ref.float() * 1.5).to(ref.dtype), what=f"fp8 pair rows masked={masked}")


def test_alignment_on_many_ctas_matches_single_cta(cuda_device, monkeypatch):
    """From 8192 slots on, the alignment runs on 32 CTAs in three launches; it must order the rows
    exactly like the single-CTA kernel.  The FP8 path with pair rows has no atomics, so the two
    outputs must be bit-equal."""
    import flaggems_sglang_b200 as F
    h, i, e, k, m = 2048, 256, 64, 8, 1100          # 8800 slots, skewed routing, some experts empty
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(h, i, e, k, m, seed=5, skew=True)
    d = cuda_device
    args = (x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d))
    kw = dict(use_fp8_w8a8=True, w13_scale=s13.to(d), w2_scale=s2.to(d))
    multi = F.fused_experts(*args, **kw)
    F.check_status()
    monkeypatch.setenv("B200MOE_ALIGN_ONE_CTA", "1")
    single = F.fused_experts(*args, **kw)
    F.check_status()
    assert torch.equal(multi, single)
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(multi, ref, what="fp8 after multi-CTA alignment")


@pytest.mark.parametrize("h,i,e,k,m", [(512, 384, 8, 2, 100), (2048, 256, 16, 8, 640)])
def test_fp8_prequantised_activations(cuda_device, h, i, e, k, m):
    """Rows that arrive already quantised (expert-parallel dispatch sends bytes) give what the
    in-call quantisation gives."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.ops.quant import per_token_group_quant_fp8
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(h, i, e, k, m, seed=h + 1)
    d = cuda_device
    kw = dict(use_fp8_w8a8=True, w13_scale=s13.to(d), w2_scale=s2.to(d))
    plain = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), **kw)
    xq, xs = per_token_group_quant_fp8(x.to(d))
    pre = F.fused_experts(xq, w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), x_scale=xs, out_dtype=x.dtype, **kw)
    F.check_status()
    assert pre.dtype == plain.dtype
    torch.testing.assert_close(pre.float(), plain.float(), rtol=1e-2, atol=1e-3)
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids)
    assert_parity(pre, ref, what=f"fp8 prequantised {(h, i, e, k, m)}")


@pytest.mark.parametrize("h,i,e,k,m,bt", [(512, 384, 8, 2, 100, 0), (512, 256, 4, 2, 150, 16), (512, 256, 4, 2, 150, 64),
                                           (2048, 256, 16, 8, 640, 0), (1024, 512, 8, 2, 300, 128)])
@pytest.mark.parametrize("alpha,limit", [(1.702, 7.0), (None, None)])
def test_fp8_bias_and_clamped_swiglu(cuda_device, h, i, e, k, m, bt, alpha, limit):
    """Per-expert biases and the bias variant's activation (reference: fused_moe.py:219-309, bf16 only
    there) on the FP8 kernels: weights-on-M blocks, 128-token blocks with atomics and with pair rows."""
    import flaggems_sglang_b200 as F
    x, tw, ids, w13q, s13, w2q, s2 = _fp8_case(h, i, e, k, m, seed=h + m + bt)
    g = torch.Generator().manual_seed(bt + m)
    b13 = (torch.randn(e, 2 * i, generator=g) * 0.5).to(torch.bfloat16)
    b2 = (torch.randn(e, h, generator=g) * 0.5).to(torch.bfloat16)
    d = cuda_device
    out = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), use_fp8_w8a8=True, w13_scale=s13.to(d),
                          w2_scale=s2.to(d), activation="swiglu_oai", b13=b13.to(d), b2=b2.to(d),
                          swiglu_alpha=1.0 if alpha is None else alpha, swiglu_limit=limit, block_tokens=bt)
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids, activation="swiglu_oai", b1=b13, b2=b2,
                               swiglu_alpha=1.0 if alpha is None else alpha, swiglu_limit=limit)
    assert_parity(out, ref, what=f"fp8 bias {(h, i, e, k, m, bt)}")
    # biases with the plain activation
    out2 = F.fused_experts(x.to(d), w13q.to(d), w2q.to(d), tw.to(d), ids.to(d), use_fp8_w8a8=True, w13_scale=s13.to(d),
                           w2_scale=s2.to(d), b13=b13.to(d), b2=b2.to(d), block_tokens=bt)
    F.check_status()
    ref2 = OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids, b1=b13, b2=b2)
    assert_parity(out2, ref2, what=f"fp8 bias + silu {(h, i, e, k, m, bt)}")
