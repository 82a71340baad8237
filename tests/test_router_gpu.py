"""GPU: the router kernel against its CPU restatement (expert ids bit-exact, weights to
fp32 rounding), and the whole layer started from gating logits."""
import numpy as np
import pytest
import torch

from oracle import moe as OM
from oracle.router import route_topk
from parity import assert_parity

pytestmark = pytest.mark.gpu

W_RTOL = 1e-5     # exp() on the GPU and in numpy differ by a few ulp; sums run in another order


def _check(logits, k, cuda_device, **kw):
    import flaggems_sglang_b200 as F
    names = dict(scoring="scoring_func", n_group="num_expert_group", bias="correction_bias", scale="routed_scaling_factor")
    okw = dict(kw)
    gkw = {names.get(a, a): v for a, v in kw.items() if a != "renormalize"}
    renorm = kw.get("renormalize", True)
    okw.pop("renormalize", None)
    bias = okw.get("bias")
    w_ref, i_ref = route_topk(logits.float().numpy(), k, renorm, bias=None if bias is None else bias.numpy(),
                              **{a: v for a, v in okw.items() if a != "bias"})
    if gkw.get("num_expert_group") or gkw.get("correction_bias") is not None or gkw.get("scoring_func", "softmax") != "softmax":
        if "correction_bias" in gkw and gkw["correction_bias"] is not None:
            gkw["correction_bias"] = gkw["correction_bias"].to(cuda_device)
        gkw.setdefault("num_expert_group", 0)
        gkw.setdefault("topk_group", 0)
        w, i = F.grouped_topk(logits.to(cuda_device), k, renorm, **gkw)
    else:
        w, i = F.topk_softmax(logits.to(cuda_device), k, renorm)
    assert w.dtype == torch.float32 and i.dtype == torch.int32
    assert np.array_equal(i.cpu().numpy(), i_ref), "expert ids differ"
    np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=W_RTOL, atol=1e-9)


@pytest.mark.parametrize("m,e,k", [(1, 8, 2), (7, 8, 2), (33, 16, 4), (64, 64, 8), (1024, 64, 8), (4096, 8, 2),
                                   (256, 128, 8), (100, 60, 6), (5, 1024, 32), (4096, 256, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_softmax(cuda_device, m, e, k, dtype):
    torch.manual_seed(m + e + k)
    logits = torch.randn(m, e, dtype=torch.float32).to(dtype)
    _check(logits, k, cuda_device)
    if m <= 64:
        _check(logits, k, cuda_device, renormalize=False)


def test_ties_and_half_logits(cuda_device):
    logits = torch.zeros(3, 16, dtype=torch.float16)
    logits[1, 5] = logits[1, 9] = 2.0
    _check(logits, 3, cuda_device)


@pytest.mark.parametrize("m", [1, 64, 512])
def test_grouped_topk_deepseek_shapes(cuda_device, m):
    """E = 256 in 8 groups, 4 groups kept, top-8: sigmoid scores with a selection bias (sum of
    the two best per group) and softmax scores without one (best per group)."""
    torch.manual_seed(m)
    logits = torch.randn(m, 256, dtype=torch.float32)
    bias = torch.randn(256) * 0.1
    _check(logits, 8, cuda_device, scoring="sigmoid", n_group=8, topk_group=4, bias=bias, scale=2.5)
    _check(logits, 8, cuda_device, scoring="softmax", n_group=8, topk_group=4)
    _check(logits, 6, cuda_device, scoring="softmax", n_group=4, topk_group=2, renormalize=False)
    _check(logits, 8, cuda_device, scoring="sigmoid")


@pytest.mark.parametrize("shape", [(7, 128, 256, 8, 2), (300, 256, 384, 64, 8)], ids=str)
def test_layer_from_logits(cuda_device, shape):
    """fused_moe(x, w13, w2, logits, k) == the experts applied to the oracle's routing."""
    import flaggems_sglang_b200 as F
    M, H, I, E, k = shape
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    logits = torch.randn(M, E, generator=g)
    d = cuda_device
    out = F.fused_moe(x.to(d), w13.to(d), w2.to(d), logits.to(d), k, renormalize=True)
    F.check_status()
    w, i = route_topk(logits.numpy(), k, True)
    ref = OM.fused_experts(x, w13, w2, torch.from_numpy(w), torch.from_numpy(i).long())
    assert_parity(out, ref, rtol=1e-2, atol=1e-2, what=f"layer from logits {shape}")
    # same as the two-step path on the GPU's own routing (the fp32 combine uses atomics, so the
    # last bf16 bit may differ between runs)
    tw, ids = F.topk_softmax(logits.to(d), k, True)
    two = F.fused_experts(x.to(d), w13.to(d), w2.to(d), tw, ids)
    torch.testing.assert_close(out.float(), two.float(), rtol=1e-2, atol=1e-3)


def test_layer_from_logits_grouped_fp8_graph(cuda_device):
    """DeepSeek-style gate in front of the FP8 experts, captured in a CUDA graph."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import quant as Q
    M, H, I, E, k = 48, 512, 256, 64, 4
    g = torch.Generator().manual_seed(9)
    x = torch.randn(M, H, generator=g).to(torch.bfloat16)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    logits = torch.randn(M, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1
    d = cuda_device
    q13, s13 = Q.quantize_fp8_block(w13)
    q2, s2 = Q.quantize_fp8_block(w2)
    args = (x.to(d), q13.to(d), q2.to(d), logits.to(d), k)
    kw = dict(renormalize=True, num_expert_group=8, topk_group=4, scoring_func="sigmoid", correction_bias=bias.to(d),
              use_fp8_w8a8=True, w13_scale=s13.to(d), w2_scale=s2.to(d))
    eager = F.fused_moe(*args, **kw)
    F.check_status()
    w, i = route_topk(logits.numpy(), k, True, "sigmoid", 8, 4, bias.numpy())
    ref = OM.fused_experts_fp8(x, q13, q2, s13, s2, torch.from_numpy(w), torch.from_numpy(i).long())
    assert_parity(eager, ref, rtol=1e-2, atol=1e-2, what="grouped fp8 layer")
    torch.cuda.synchronize(d)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        captured = F.fused_moe(*args, **kw)
    gr.replay()
    torch.cuda.synchronize(d)
    F.check_status()
    torch.testing.assert_close(captured.float(), eager.float(), rtol=1e-2, atol=1e-3)
