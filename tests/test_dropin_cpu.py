"""CPU: the package answers at the reference's module paths with the reference's
signatures, and the per-weight layout caches survive a second look-up with the same tensor."""
import importlib
import inspect

import torch

# parameter names and defaults of the reference's entry points, restated from
# src/flaggems_sglang/ops/fused_moe.py:133-152, 219-236 and 312-316
REF_FUSED_EXPERTS = [
    ("hidden_states", inspect.Parameter.empty), ("w1", inspect.Parameter.empty), ("w2", inspect.Parameter.empty),
    ("routing_data", inspect.Parameter.empty), ("gather_indx", inspect.Parameter.empty),
    ("scatter_indx", inspect.Parameter.empty), ("inplace", False), ("activation", "silu"),
    ("apply_router_weight_on_input", False), ("use_fp8_w8a8", False), ("per_channel_quant", False),
    ("global_num_experts", -1), ("expert_map", None), ("w1_scale", None), ("w2_scale", None),
    ("a1_scale", None), ("a2_scale", None), ("block_shape", None),
]
REF_WITH_BIAS = [
    ("hidden_states", inspect.Parameter.empty), ("w1", inspect.Parameter.empty), ("w1_pcg", inspect.Parameter.empty),
    ("b1", inspect.Parameter.empty), ("w2", inspect.Parameter.empty), ("w2_pcg", inspect.Parameter.empty),
    ("b2", inspect.Parameter.empty), ("routing_data", inspect.Parameter.empty),
    ("gather_indx", inspect.Parameter.empty), ("scatter_indx", inspect.Parameter.empty), ("inplace", False),
    ("activation", "silu"), ("apply_router_weight_on_input", False), ("global_num_experts", -1),
    ("gemm1_alpha", None), ("gemm1_clamp_limit", None),
]
REF_FLAGOS = [("obj", inspect.Parameter.empty), ("layer", inspect.Parameter.empty),
              ("dispatch_output", inspect.Parameter.empty)]


def _positional(fn):
    return [(p.name, p.default) for p in inspect.signature(fn).parameters.values()
            if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]


def test_reference_module_paths_and_signatures():
    import flaggems_sglang
    import flaggems_sglang.ops
    import flaggems_sglang.ops.fused_moe as fm
    from flaggems_sglang.ops.fused_moe import (_standard_topk_to_triton_kernels, fused_moe_flagos,
                                               triton_kernel_fused_experts, triton_kernel_fused_experts_with_bias)
    assert flaggems_sglang.triton_kernel_fused_experts is triton_kernel_fused_experts
    assert flaggems_sglang.ops.triton_kernel_fused_experts is triton_kernel_fused_experts
    assert flaggems_sglang.ops.triton_kernel_fused_experts_with_bias is triton_kernel_fused_experts_with_bias
    assert fm.fused_moe_flagos is fused_moe_flagos and callable(_standard_topk_to_triton_kernels)
    assert _positional(triton_kernel_fused_experts) == REF_FUSED_EXPERTS
    assert _positional(triton_kernel_fused_experts_with_bias) == REF_WITH_BIAS
    assert _positional(fused_moe_flagos) == REF_FLAGOS
    assert [p.name for p in inspect.signature(_standard_topk_to_triton_kernels).parameters.values()][:3] == \
        ["topk_weights", "topk_ids", "n_expts_tot"]
    # the build's extensions are keyword-only, so the reference's positional calls keep their meaning
    extra = [p for p in inspect.signature(triton_kernel_fused_experts).parameters.values() if p.kind == p.KEYWORD_ONLY]
    assert {p.name for p in extra} == {"use_int4_w4a16", "w1_zp", "w2_zp", "group_size"}
    assert flaggems_sglang.device == "cuda" and flaggems_sglang.vendor_name == "nvidia"
    import flaggems_sglang.testing as T
    T.assert_equal(torch.ones(3), torch.ones(3))
    T.assert_close(torch.ones(3, dtype=torch.bfloat16), torch.ones(3) * 1.01, torch.bfloat16)


def test_layout_caches_hit_on_the_second_call():
    """A serving step passes the same weight objects every time: the second look-up must return
    the cached re-layout, not compare tensors by value."""
    fm = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")   # (the package also exports a function of that name)
    w = torch.randn(3, 8, 16).to(torch.bfloat16)            # op layout [E, K, N]
    a = fm._layer_layout(w)
    b = fm._layer_layout(w)
    assert a.data_ptr() == b.data_ptr() and a.shape == (3, 16, 8) and a.is_contiguous()
    assert torch.equal(a, w.transpose(1, 2))
    view = a.transpose(1, 2)                                 # a transposed view of layer-layout storage: used as is
    assert fm._layer_layout(view).data_ptr() == a.data_ptr()
    w.mul_(2)                                                # written in place -> rebuilt
    c = fm._layer_layout(w)
    assert torch.equal(c, w.transpose(1, 2))

    b1 = torch.randn(3, 16)
    s1 = fm._deinterleaved(w, b1)
    s2 = fm._deinterleaved(w, b1)
    assert s1[0].data_ptr() == s2[0].data_ptr() and s1[1].data_ptr() == s2[1].data_ptr()
    assert torch.equal(s1[0][:, :8], w.transpose(1, 2)[:, 0::2]) and torch.equal(s1[1][:, 8:], b1[:, 1::2])
    # the two kinds of derived layout of one tensor do not evict each other
    assert fm._layer_layout(w).data_ptr() == c.data_ptr()
    ll = fm._deinterleaved(a, b1, layer_layout=True)
    assert ll[0].shape == a.shape and torch.equal(ll[0][:, :8], a[:, 0::2])


def test_workspace_cache_is_bounded():
    fm = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")   # (the package also exports a function of that name)
    assert fm.MAX_CACHED_WORKSPACES >= 2
    fm.release_workspaces()
    assert len(fm._workspaces) == 0
