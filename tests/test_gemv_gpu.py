"""GPU: the matrix-vector path for a handful of (token, choice) pairs (csrc/gemv.cu).

Calls with 16-bit or int4 weights and M * topk <= 16 skip alignment, gather, grouped GEMMs and output
conversion: two launches read the routing input directly.  Every case here is checked against the
CPU oracle and against the grouped-GEMM path on the same inputs (forced by fixing the token
block), and the launch log must show which path ran.
"""
import pytest
import torch

from oracle import moe as OM
from parity import assert_parity

pytestmark = pytest.mark.gpu


def _names():
    from flaggems_sglang_b200 import _lib
    return _lib.launch_stats()[1]


def _is_gemv():
    return any("gemv" in n for n in _names())


def _layer(h, i, e, device, dtype=torch.bfloat16, seed=3):
    from flaggems_sglang_b200.testing import make_weights
    return make_weights(h, i, e, dtype=dtype, device=device, seed=seed)


@pytest.mark.parametrize("M,topk", [(1, 2), (1, 8), (2, 8), (3, 4), (16, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemv_16bit_matches_oracle_and_grouped_path(cuda_device, M, topk, dtype):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e = 1024, 768, 64
    d = cuda_device
    w13, w2 = _layer(h, i, e, d, dtype)
    x, tw, ids = make_tokens(M, h, e, topk, dtype=dtype, seed=M * 10 + topk)
    out = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    assert _is_gemv(), _names()
    grouped = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d), block_tokens=16)
    assert not _is_gemv(), _names()
    F.check_status()
    ref = OM.fused_experts(x, w13.cpu().float(), w2.cpu().float(), tw, ids)
    assert_parity(out, ref, what=f"gemv {dtype} M={M} topk={topk} vs oracle")
    assert_parity(out, grouped.float(), what=f"gemv {dtype} M={M} topk={topk} vs grouped path")
    again = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    assert torch.equal(out, again), "fixed summation order: a rerun gives the same bits"


@pytest.mark.parametrize("h,i", [(264, 136), (1280, 384), (1536, 520)])
def test_gemv_ragged_hidden_sizes(cuda_device, h, i):
    """H and I that are multiples of 8 but not of the 256-element warp stride, and rows of five and
    six chunks (kernel variants that keep the whole row in flight)."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    e, topk = 16, 2
    d = cuda_device
    w13, w2 = _layer(h, i, e, d)
    x, tw, ids = make_tokens(2, h, e, topk, seed=5)
    out = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    assert _is_gemv(), _names()
    F.check_status()
    ref = OM.fused_experts(x, w13.cpu().float(), w2.cpu().float(), tw, ids)
    assert_parity(out, ref, what=f"gemv ragged H={h} I={i}")


def test_gemv_options(cuda_device):
    """Router weight on the input side, scaling factor, per-pair output, gelu, int64 ids."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, topk = 512, 256, 32, 4
    d = cuda_device
    w13, w2 = _layer(h, i, e, d)
    x, tw, ids = make_tokens(2, h, e, topk, seed=9)
    xd, twd, idd = x.to(d), tw.to(d), ids.to(d)
    for kw in (dict(apply_router_weight_on_input=True), dict(routed_scaling_factor=2.5), dict(no_combine=True),
               dict(activation="gelu"), dict(mimic_reference_rounding=False)):
        out = F.fused_experts(xd, w13, w2, twd, idd, **kw)
        assert _is_gemv(), (kw, _names())
        grouped = F.fused_experts(xd, w13, w2, twd, idd, block_tokens=16, **kw)
        F.check_status()
        assert out.shape == grouped.shape
        assert_parity(out, grouped.float(), what=f"gemv {kw} vs grouped path")
    out64 = F.fused_experts(xd, w13, w2, twd, idd.long())
    assert _is_gemv(), _names()
    assert torch.equal(out64, F.fused_experts(xd, w13, w2, twd, idd))


def test_gemv_expert_map_drops_foreign_experts(cuda_device):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e_global, topk = 512, 256, 64, 4
    d = cuda_device
    w13, w2 = _layer(h, i, e_global, d)
    x, tw, ids = make_tokens(2, h, e_global, topk, seed=11)
    # this rank holds the even experts only
    held = torch.arange(0, e_global, 2)
    emap = torch.full((e_global,), -1, dtype=torch.int32)
    emap[held] = torch.arange(held.numel(), dtype=torch.int32)
    out = F.fused_experts(x.to(d), w13[held.to(d)].contiguous(), w2[held.to(d)].contiguous(), tw.to(d), ids.to(d),
                          expert_map=emap.to(d))
    assert _is_gemv(), _names()
    F.check_status()
    keep = (ids % 2 == 0)
    ref = OM.fused_experts(x, w13.cpu().float(), w2.cpu().float(), tw * keep, ids)
    assert_parity(out, ref, what="gemv with expert_map")


def test_gemv_bias_and_clamped_swiglu(cuda_device):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, topk = 512, 256, 8, 4
    d = cuda_device
    w13, w2 = _layer(h, i, e, d)
    g = torch.Generator().manual_seed(4)
    b13 = torch.randn(e, 2 * i, generator=g) * 0.1
    b2 = torch.randn(e, h, generator=g) * 0.1
    x, tw, ids = make_tokens(1, h, e, topk, seed=13)
    kw = dict(b13=b13.to(d), b2=b2.to(d), activation="swiglu_oai", swiglu_alpha=1.702, swiglu_limit=7.0)
    out = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d), **kw)
    assert _is_gemv(), _names()
    grouped = F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d), block_tokens=16, **kw)
    F.check_status()
    assert_parity(out, grouped.float(), what="gemv bias + clamped swiglu vs grouped path")


def test_gemv_through_the_operator_entry_point(cuda_device):
    """The reference-compatible call (routing triple) takes the same path."""
    import flaggems_sglang
    from test_fused_moe_gpu import _ref_inputs, _run_reference_api
    shape = (1, 1280, 3072, 64, 8)
    x, w1, w2, tw, ids = _ref_inputs(*shape, cuda_device)
    out = _run_reference_api(x, w1, w2, tw, ids, 64, cuda_device)
    assert _is_gemv(), _names()
    ref = OM.fused_experts(x, w1.transpose(1, 2).float(), w2.transpose(1, 2).float(), tw, ids)
    assert_parity(out, ref, what="gemv through triton_kernel_fused_experts")


def _awq_case(h, i, e, k, m, seed, device):
    from flaggems_sglang_b200.quant import quantize_awq, repack_awq_for_kernel
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(h, i, e, dtype=torch.float16, seed=seed)
    x, tw, ids = make_tokens(m, h, e, k, dtype=torch.float16, seed=seed)
    q1 = quantize_awq(w13.transpose(1, 2).contiguous())      # AWQ layout [E, K, N]
    q2 = quantize_awq(w2.transpose(1, 2).contiguous())
    p1, z1 = repack_awq_for_kernel(*[t.to(device) for t in q1])
    p2, z2 = repack_awq_for_kernel(*[t.to(device) for t in q2])
    return x, tw, ids, q1, q2, dict(use_int4_w4a16=True, w13_sz=z1, w2_sz=z2), p1, p2


@pytest.mark.parametrize("h,i,e,k,m", [(1024, 512, 8, 2, 1), (4096, 1024, 8, 2, 1), (512, 384, 64, 8, 2),
                                        (256, 128, 16, 4, 1), (2048, 1152, 64, 4, 3)])
def test_gemv_int4_integer_dot_products(cuda_device, h, i, e, k, m):
    """int4 (AWQ) weights: dp4a on raw nibbles and three int8 activation planes, the arithmetic of the
    integer tensor-core kernels, so the two paths agree far inside the tolerance."""
    import flaggems_sglang_b200 as F
    d = cuda_device
    x, tw, ids, q1, q2, kw, p1, p2 = _awq_case(h, i, e, k, m, seed=h + m, device=d)
    out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), **kw)
    assert any("gemv_w4" in n for n in _names()), _names()
    grouped = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), block_tokens=16, **kw)
    assert not _is_gemv(), _names()
    F.check_status()
    ref = OM.fused_experts_awq(x, *q1, *q2, tw, ids)
    assert out.dtype == torch.float16
    assert_parity(out, ref, rtol=2e-2, atol=2e-2, what=f"gemv int4 {(h, i, e, k, m)} vs oracle")
    assert_parity(out, grouped.float(), rtol=2e-3, atol=2e-3, what=f"gemv int4 {(h, i, e, k, m)} vs grouped path")
    assert torch.equal(out, F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), **kw)), "rerun differs"


def test_gemv_int4_options(cuda_device):
    import flaggems_sglang_b200 as F
    d = cuda_device
    h, i, e, k = 512, 256, 32, 4
    x, tw, ids, q1, q2, kw, p1, p2 = _awq_case(h, i, e, k, 2, seed=31, device=d)
    g = torch.Generator().manual_seed(6)
    b13 = (torch.randn(e, 2 * i, generator=g) * 0.1).to(d)
    b2 = (torch.randn(e, h, generator=g) * 0.1).to(d)
    for extra in (dict(apply_router_weight_on_input=True), dict(no_combine=True), dict(routed_scaling_factor=0.5),
                  dict(b13=b13, b2=b2, activation="swiglu_oai", swiglu_alpha=1.702, swiglu_limit=7.0)):
        out = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), **kw, **extra)
        assert any("gemv_w4" in n for n in _names()), (extra.keys(), _names())
        grouped = F.fused_experts(x.to(d), p1, p2, tw.to(d), ids.to(d), block_tokens=16, **kw, **extra)
        F.check_status()
        assert_parity(out, grouped.float(), rtol=2e-3, atol=2e-3, what=f"gemv int4 {list(extra)} vs grouped path")


def test_fp8_weights_take_the_grouped_path(cuda_device):
    """FP8 rows would be converted element by element on the CUDA cores: slower than the
    tensor-core path even at one token, so they stay on it."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import make_tokens
    h, i, e, topk = 1024, 512, 16, 8
    d = cuda_device
    w13, w2 = _layer(h, i, e, d)
    w13q, s13 = quantize_fp8_block(w13)
    w2q, s2 = quantize_fp8_block(w2)
    x, tw, ids = make_tokens(1, h, e, topk, seed=22)
    out = F.fused_experts(x.to(d), w13q, w2q, tw.to(d), ids.to(d), use_fp8_w8a8=True, w13_scale=s13, w2_scale=s2)
    assert not _is_gemv(), _names()
    F.check_status()
    ref = OM.fused_experts_fp8(x, w13q.cpu(), w2q.cpu(), s13.cpu(), s2.cpu(), tw, ids)
    assert_parity(out, ref, what="fp8 M=1 on the grouped path")


def test_more_pairs_than_the_limit_take_the_grouped_path(cuda_device):
    """More than 16 pairs, or several tokens whose pairs would often meet in one expert (pairs >
    experts / 4: each pair streams its expert's weights by itself)."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200.testing import make_tokens
    h, i, topk = 512, 256, 2
    d = cuda_device
    for m, e in ((9, 128), (4, 8)):                        # 18 pairs; 8 pairs over 8 experts
        w13, w2 = _layer(h, i, e, d)
        x, tw, ids = make_tokens(m, h, e, topk, seed=2)
        F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
        assert not _is_gemv(), (m, e, _names())
    w13, w2 = _layer(h, i, 8, d)
    x, tw, ids = make_tokens(1, h, 8, topk, seed=2)        # one token: its experts are distinct
    F.fused_experts(x.to(d), w13, w2, tw.to(d), ids.to(d))
    assert _is_gemv(), _names()
