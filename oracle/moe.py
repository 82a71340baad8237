"""Per-expert-loop MoE forward (torch on CPU, fp32 math).  Test infrastructure only.

Restates what the reference's ``triton_kernel_fused_experts`` computes
(src/flaggems_sglang/ops/fused_moe.py:181-216) through its dependency's
grouped matmul:

  GEMM-1 (189-196)   y1[r] = x[token(r)] @ W1[e(r)]   (* gamma_r if the router
                     weight is applied on the input), fp32 accumulate, rounded
                     to the activation dtype                       (point 1)
  activation (198-202, kernels 28-69)
                     a[r] = y1[r, :I] / (1 + exp(-y1[r, :I])) * y1[r, I:],
                     fp32 math, rounded to the activation dtype    (point 2)
  GEMM-2 (208-215)   y2[r] = a[r] @ W2[e(r)] (* gamma_r otherwise), rounded to
                     the activation dtype when the dependency does not split K
                                                                   (point 3)
  combine            out[t] = round( sum_j fp32(y2[row of (t, j)]) ), experts of
                     a token visited in ascending order.

Weights are taken in the *layer* layout ``w1 [E, 2I, H]``, ``w2 [E, H, I]``
(the reduction dimension last); the op-level layout is its transpose.
"""
from __future__ import annotations

import numpy as np
import torch

from . import quant as Q
from .routing import topk_to_routing


def _next_pow2(v: int) -> int:
    p = 1
    while p < v:
        p <<= 1
    return p


def reference_rounds_pairs(n_slots: int, n_experts: int, n: int, k: int, n_sms: int = 148) -> bool:
    """Does the reference round each (token, expert) row of GEMM-2 to the 16-bit
    type before the top-k sum (rounding point 3)?

    Only when its dependency does not split the reduction.  Restated from
    triton_kernels/matmul_ogs_details/opt_flags.py (make_default_opt_flags_nvidia:
    block_m, persistence, split_k) and opt_flags_details/opt_flags_nvidia.py
    (compute_block_n, compute_grid_size, compute_split_k); n = output columns (H),
    k = reduction length (I), n_sms = 148 on a B200.  Checked against outputs of
    the reference recorded on a B200 (tests/golden/fused_moe_ref_golden.npz)."""
    cdiv = lambda a, b: -(-a // b)
    block_m = max(16, min(_next_pow2(max(1, n_slots // n_experts)), 128))
    block_n = 256 if n > 128 else max(16, min(128, _next_pow2(n)))
    grid_n = cdiv(n, block_n)
    if n_slots <= n_experts:
        grid_m_routed = n_slots
    else:
        grid_m_routed = cdiv(max(n_slots - n_experts + 1, 0), block_m) + n_experts - 1
    if grid_m_routed * grid_n / n_sms >= 2.0:       # persistent kernel: never splits
        return True
    grid = cdiv(n_slots, block_m) * grid_n
    split = max(1, min(n_sms // grid, cdiv(k, 64) // 4))
    return split == 1


def silu_mul(y1: torch.Tensor) -> torch.Tensor:
    i = y1.shape[-1] // 2
    g, u = y1[..., :i].float(), y1[..., i:].float()
    return g / (1.0 + torch.exp(-g)) * u


def gelu_mul(y1: torch.Tensor) -> torch.Tensor:
    i = y1.shape[-1] // 2
    g, u = y1[..., :i].float(), y1[..., i:].float()
    return torch.nn.functional.gelu(g) * u


def swiglu_oai(y1: torch.Tensor, alpha: float = 1.0, limit=None) -> torch.Tensor:
    """Activation the reference's bias variant fuses into GEMM-1 (its dependency's swiglu:
    triton_kernels/swiglu_details/_swiglu.py, compute_swiglu): on [gate | linear] halves,
    gate clamped from above, linear to [-limit, limit], s = g / (1 + exp(-alpha g)),
    result s * linear + s."""
    i = y1.shape[-1] // 2
    g, u = y1[..., :i].float(), y1[..., i:].float()
    if limit is not None and limit > 0:
        g = torch.minimum(g, torch.tensor(float(limit)))
        u = u.clamp(-float(limit), float(limit))
    s = g / (1.0 + torch.exp(-alpha * g))
    return s * u + s


def _n_local(w1) -> int:
    return w1.shape[0] if hasattr(w1, "shape") else w1.n_experts


def _round(t: torch.Tensor, dtype, on: bool) -> torch.Tensor:
    return t.to(dtype).float() if on else t


def fused_experts(
    x: torch.Tensor,
    w1,
    w2,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    *,
    apply_router_weight_on_input: bool = False,
    activation: str = "silu",
    mimic_rounding: bool = True,
    round_y2: bool | None = None,
    out_dtype=None,
    act_quant=None,
    expert_lo: int = 0,
    no_combine: bool = False,
    b1=None,
    b2=None,
    swiglu_alpha: float = 1.0,
    swiglu_limit=None,
) -> torch.Tensor:
    """x [M, H]; w1 [E, 2I, H] / w2 [E, H, I] tensors (any float dtype), or
    callables ``e -> fp32 matrix`` for lazily dequantised weights.

    ``act_quant``: optional ``fn(rows fp32) -> rows fp32`` applied to the input
    of each GEMM (quantise-dequantise); used by the FP8 path.
    ``expert_lo``: global id of local expert 0 (expert-parallel shards); ids
    outside the local range contribute nothing.
    """
    m, h = x.shape
    k = topk_ids.shape[1]
    out_dtype = out_dtype or x.dtype
    if round_y2 is None:
        i_dim = (w2.shape[2] if hasattr(w2, "shape") else getattr(w2, "i_dim", None))
        round_y2 = mimic_rounding and (i_dim is None or reference_rounds_pairs(m * k, _n_local(w1), h, i_dim))
    n_local = w1.shape[0] if hasattr(w1, "shape") else w1.n_experts
    get1 = (lambda e: w1[e].float()) if hasattr(w1, "shape") else w1
    get2 = (lambda e: w2[e].float()) if hasattr(w2, "shape") else w2
    act = {"silu": silu_mul, "gelu": gelu_mul,
           "swiglu_oai": lambda y: swiglu_oai(y, swiglu_alpha, swiglu_limit)}
    if activation not in act:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")

    ids = topk_ids.to(torch.int64) - expert_lo
    ids = torch.where((ids >= 0) & (ids < n_local), ids, torch.full_like(ids, n_local))
    r = topk_to_routing(topk_weights.float(), ids, n_local + 1)
    raw, topk_indx = r["token_offs_raw"], r["topk_indx"]
    gate_scal = torch.from_numpy(np.ascontiguousarray(r["gate_scal"])).float()

    xf = x.float()
    if act_quant is not None:
        xf = act_quant(xf)
    out = torch.zeros(m, h, dtype=torch.float32)
    pairs = torch.zeros(m * k, h, dtype=torch.float32) if no_combine else None
    for e in range(n_local):
        lo, hi = int(raw[e]), int(raw[e + 1])
        if lo == hi:
            continue
        slots = torch.from_numpy(topk_indx[lo:hi].astype(np.int64))
        tok = slots // k
        gam = gate_scal[lo:hi, None]
        y1 = xf[tok] @ get1(e).t()
        if b1 is not None:
            y1 = y1 + b1[e].float()
        if activation == "swiglu_oai":
            # bias variant (fused_moe.py:285-298): activation fused into GEMM-1, routing weight after it,
            # a single rounding of the activated rows
            a = act[activation](y1)
            if apply_router_weight_on_input:
                a = a * gam
            a = a.to(out_dtype).float()
        else:
            if apply_router_weight_on_input:
                y1 = y1 * gam
            y1 = _round(y1, out_dtype, mimic_rounding)
            a = act[activation](y1).to(out_dtype).float()      # point 2 is inherent
        if act_quant is not None:
            a = act_quant(a)
        y2 = a @ get2(e).t()
        if b2 is not None:
            y2 = y2 + b2[e].float()
        if not apply_router_weight_on_input:
            y2 = y2 * gam
        y2 = _round(y2, out_dtype, round_y2)
        if no_combine:
            pairs[slots] = y2
        else:
            out.index_add_(0, tok, y2)
    if no_combine:
        # The routing tables number a token's pairs in ascending expert order (the converter sorts
        # each row first); hand them back in the order of the caller's topk_ids columns.
        order = torch.from_numpy(np.argsort(ids.numpy(), axis=1, kind="stable"))
        by_sorted = pairs.to(out_dtype).view(m, k, h)
        res = torch.empty_like(by_sorted)
        res.scatter_(1, order[:, :, None].expand(m, k, h), by_sorted)
        return res
    return out.to(out_dtype)


# ------------------------------------------------------------------ quantised variants
class _LazyWeights:
    def __init__(self, n_experts, fn, i_dim=None):
        self.n_experts = n_experts
        self.i_dim = i_dim
        self._fn = fn

    def __call__(self, e):
        return self._fn(e)


def fused_experts_fp8(x, w1_q, w2_q, w1_scale, w2_scale, topk_weights, topk_ids, **kw):
    """FP8 e4m3 weights with 128x128 block scales, activations quantised per
    1x128 group before each GEMM.  No bf16 rounding of y1 / y2 (the accumulator
    is promoted in fp32); the activation is rounded to bf16 before its quantisation."""
    e = w1_q.shape[0]
    w1 = _LazyWeights(e, lambda i: Q.dequant_weight_fp8_block(w1_q[i], w1_scale[i]))
    w2 = _LazyWeights(e, lambda i: Q.dequant_weight_fp8_block(w2_q[i], w2_scale[i]))

    def qdq(rows):
        q, s = Q.quant_act_fp8_group(rows)
        return Q.dequant_act_fp8_group(q, s)

    kw.setdefault("mimic_rounding", False)
    return fused_experts(x, w1, w2, topk_weights, topk_ids, act_quant=qdq, **kw)


def fused_experts_awq(x, w1_qweight, w1_scales, w1_qzeros, w2_qweight, w2_scales, w2_qzeros,
                      topk_weights, topk_ids, group: int = 128, **kw):
    """int4 AWQ w4a16: qweight [E, K, N/8] int32 (K = reduction dim), scales
    [E, K/g, N] fp16, qzeros [E, K/g, N/8] int32; fp16 activations."""
    e = w1_qweight.shape[0]
    w1 = _LazyWeights(e, lambda i: Q.dequant_weight_awq(w1_qweight[i], w1_scales[i], w1_qzeros[i], group).t())
    w2 = _LazyWeights(e, lambda i: Q.dequant_weight_awq(w2_qweight[i], w2_scales[i], w2_qzeros[i], group).t(),
                      i_dim=w2_qweight.shape[1])
    return fused_experts(x, w1, w2, topk_weights, topk_ids, **kw)
