"""CPU: the per-expert-loop oracle against a dense restatement on tiny cases,
and the quantiser oracle's round trips."""
import numpy as np
import pytest
import torch

from oracle import moe as OM
from oracle import quant as Q


def _dense(x, w13, w2, tw, ids):
    m, h = x.shape
    out = torch.zeros(m, h)
    for t in range(m):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            y1 = w13[e].float() @ x[t].float()
            i = y1.shape[0] // 2
            a = torch.nn.functional.silu(y1[:i]) * y1[i:]
            out[t] += tw[t, j] * (w2[e].float() @ a)
    return out


def test_oracle_matches_dense_without_rounding():
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(64, 48, 4, dtype=torch.float32, seed=0, scale=0.1)
    x, tw, ids = make_tokens(9, 64, 4, 2, dtype=torch.float32, seed=0)
    got = OM.fused_experts(x, w13, w2, tw, ids, mimic_rounding=False)
    torch.testing.assert_close(got, _dense(x, w13, w2, tw, ids), rtol=1e-5, atol=1e-5)
    got_in = OM.fused_experts(x, w13, w2, tw, ids, mimic_rounding=False, apply_router_weight_on_input=False)
    torch.testing.assert_close(got_in, got)


def test_oracle_config1_tiny_bf16():
    """BASELINE config 1: M=64, H=1024, I=512, E=8, top-2, seed 0."""
    from flaggems_sglang_b200.testing import CONFIGS, make_tokens, make_weights
    h, i, e, k = CONFIGS["tiny"]
    w13, w2 = make_weights(h, i, e, seed=0)
    x, tw, ids = make_tokens(64, h, e, k, seed=0)
    out = OM.fused_experts(x, w13, w2, tw, ids)
    assert out.shape == (64, h) and out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    dense = _dense(x, w13, w2, tw, ids)
    torch.testing.assert_close(out.float(), dense, rtol=2e-2, atol=2e-3)


def test_oracle_matches_reference_outputs():
    """Pins the floating-point oracle: outputs of the reference's Triton op recorded
    on a B200 for its own test shapes and input recipe (tests/test_fused_moe.py:50-58)."""
    from conftest import GOLDEN
    from flaggems_sglang_b200.testing import route
    from parity import assert_parity, bit_equal_fraction
    gold = np.load(GOLDEN / "fused_moe_ref_golden.npz")
    for key in sorted(gold.files):
        name, which = key.split("/")
        M, K, N, E, topk = (int(p.lstrip("MKNEtopk")) for p in name.split("_"))
        if M * K * N > 17 * 1280 * 3072:
            continue                      # keep the CPU suite short
        torch.manual_seed(M + K + N + E + topk)
        x = torch.randn(M, K, dtype=torch.bfloat16)
        w1 = torch.randn(E, K, N * 2, dtype=torch.bfloat16) * 0.1
        w2 = torch.randn(E, N, K, dtype=torch.bfloat16) * 0.1
        tw, ids = route(torch.randn(M, E, dtype=torch.float32), topk)
        ref = OM.fused_experts(x, w1.transpose(1, 2), w2.transpose(1, 2), tw, ids,
                               apply_router_weight_on_input=(which == "gate_in"))
        g = torch.from_numpy(gold[key]).view(torch.bfloat16)
        assert_parity(ref, g, what=key)
        assert bit_equal_fraction(ref, g) >= 0.9, key


def test_reference_split_rule_on_recorded_shapes():
    # (M, K, N, E, topk, rounds GEMM-2 rows): which recorded outputs carry rounding point 3
    for M, K, N, E, k, rounds in [(1, 128, 256, 8, 2, True), (7, 128, 256, 8, 2, True), (33, 256, 512, 16, 4, False),
                                  (1, 1280, 3072, 64, 8, False), (4, 1280, 3072, 64, 8, False),
                                  (17, 1280, 3072, 64, 8, True), (64, 1280, 3072, 64, 8, True)]:
        assert OM.reference_rounds_pairs(M * k, E, K, N) is rounds


def test_expert_lo_partition_sums_to_whole():
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    w13, w2 = make_weights(64, 32, 8, dtype=torch.float32, seed=1, scale=0.1)
    x, tw, ids = make_tokens(20, 64, 8, 2, dtype=torch.float32, seed=1)
    whole = OM.fused_experts(x, w13, w2, tw, ids, mimic_rounding=False)
    parts = sum(OM.fused_experts(x, w13[lo:lo + 4], w2[lo:lo + 4], tw, ids, mimic_rounding=False, expert_lo=lo)
                for lo in (0, 4))
    torch.testing.assert_close(parts, whole, rtol=1e-5, atol=1e-6)


def test_awq_pack_unpack_identity():
    g = torch.Generator().manual_seed(0)
    v = torch.randint(0, 16, (3, 40, 64), generator=g, dtype=torch.uint8)
    p = Q.awq_pack(v)
    assert p.dtype == torch.int32 and p.shape == (3, 40, 8)
    assert torch.equal(Q.awq_unpack(p), v)
    # nibble order: logical column 1 lands in nibble 4
    one = torch.zeros(1, 1, 8, dtype=torch.uint8)
    one[0, 0, 1] = 0xF
    assert int(Q.awq_pack(one)[0, 0, 0]) == 0xF << 16


def test_awq_quant_error_bound():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(2, 256, 64, generator=g) * 0.02
    q, s, z = Q.quant_weight_awq(w)
    deq = Q.dequant_weight_awq(Q.awq_pack(q), s, Q.awq_pack(z))
    assert (deq - w).abs().max() <= s.float().max() * 0.51 + 1e-6


def test_fp8_block_quant_round_trip():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(2, 256, 384, generator=g) * 0.02
    q, s = Q.quant_weight_fp8_block(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (2, 2, 3)
    deq = Q.dequant_weight_fp8_block(q, s)
    assert ((deq - w).abs() <= w.abs() * 0.0625 + s.max() * 2 ** -9 + 1e-9).all()
    x = torch.randn(5, 256, generator=g)
    xq, xs = Q.quant_act_fp8_group(x)
    assert xs.shape == (5, 2) and torch.isfinite(xq.float()).all()
    assert (xq.float().abs().amax(dim=1) <= 448).all()
    zq, zs = Q.quant_act_fp8_group(torch.zeros(1, 128))
    assert (zq.float() == 0).all() and torch.isfinite(zs).all()


def test_product_quantisers_agree_with_oracle():
    from flaggems_sglang_b200 import quant as PQ
    g = torch.Generator().manual_seed(3)
    w = torch.randn(2, 256, 256, generator=g) * 0.02
    q, s = PQ.quantize_fp8_block(w)
    oq, os_ = Q.quant_weight_fp8_block(w)
    assert torch.equal(q.view(torch.uint8), oq.view(torch.uint8)) and torch.equal(s, os_)
    wk = torch.randn(2, 256, 64, generator=g) * 0.02
    pq, ps, pz = PQ.quantize_awq(wk)
    oq, os_, oz = Q.quant_weight_awq(wk)
    assert torch.equal(pq, Q.awq_pack(oq)) and torch.equal(ps, os_) and torch.equal(pz, Q.awq_pack(oz))


def test_bias_variant_against_a_direct_loop():
    """The oracle's bias / clamped-swiglu branch (order: bias, activation, routing weight, as the
    dependency's grouped matmul applies them) against a token-by-token loop in fp32."""
    import torch
    from flaggems_sglang_b200.testing import route
    from oracle import moe as OM
    g = torch.Generator().manual_seed(0)
    M, H, I, E, k = 5, 32, 16, 4, 2
    x = torch.randn(M, H, generator=g)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.1
    w2 = torch.randn(E, H, I, generator=g) * 0.1
    b1 = torch.randn(E, 2 * I, generator=g)
    b2 = torch.randn(E, H, generator=g)
    tw, ids = route(torch.randn(M, E, generator=g), k)
    out = OM.fused_experts(x, w13, w2, tw, ids, activation="swiglu_oai", b1=b1, b2=b2, swiglu_alpha=1.7,
                           swiglu_limit=2.0, mimic_rounding=False)
    ref = torch.zeros(M, H)
    for t in range(M):
        for j in range(k):
            e = int(ids[t, j])
            y = w13[e] @ x[t] + b1[e]
            gate, lin = y[:I].clamp(max=2.0), y[I:].clamp(-2.0, 2.0)
            s = gate * torch.sigmoid(1.7 * gate)
            ref[t] += tw[t, j] * (w2[e] @ (s * (lin + 1)) + b2[e])
    assert float((out - ref).abs().max()) < 1e-5


def test_no_combine_rows_follow_topk_columns():
    """no_combine returns pair j of token t in the column order of topk_ids, whatever order the
    routing tables sort a token's experts in."""
    import torch
    from flaggems_sglang_b200.testing import route
    from oracle import moe as OM
    g = torch.Generator().manual_seed(1)
    M, H, I, E, k = 6, 32, 16, 5, 3
    x = torch.randn(M, H, generator=g)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.1
    w2 = torch.randn(E, H, I, generator=g) * 0.1
    tw, ids = route(torch.randn(M, E, generator=g), k)
    pairs = OM.fused_experts(x, w13, w2, tw, ids, no_combine=True, mimic_rounding=False)
    assert pairs.shape == (M, k, H)
    for t in range(M):
        for j in range(k):
            e = int(ids[t, j])
            y = w13[e] @ x[t]
            a = torch.nn.functional.silu(y[:I]) * y[I:]
            assert float((pairs[t, j] - tw[t, j] * (w2[e] @ a)).abs().max()) < 1e-5
    whole = OM.fused_experts(x, w13, w2, tw, ids, mimic_rounding=False)
    assert float((pairs.sum(1) - whole).abs().max()) < 1e-5
