"""Quantiser / packer oracle (torch on CPU).  Test infrastructure only.

The reference implements none of these (fused_moe.py:154-169 rejects every
quantised argument), so the conventions below are the serving ecosystem's:

* FP8: float8_e4m3fn, scale = amax / 448 per 128x128 weight block and per
  1x128 activation group, value = q * scale.
* int4 AWQ: asymmetric uint4 per (output column, group of 128 along K),
  w ~= (q - z) * s, eight output columns per int32 with logical column j in
  nibble [0, 4, 1, 5, 2, 6, 3, 7][j].
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
FP8_EPS = 1e-10
AWQ_NIBBLE_OF_COLUMN = (0, 4, 1, 5, 2, 6, 3, 7)


# ----------------------------------------------------------------------------- FP8
def fp8_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto e4m3fn with saturation, returned as fp8."""
    return x.float().clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def quant_weight_fp8_block(w: torch.Tensor, block=(128, 128)):
    """w [..., N, K] -> (q fp8 [..., N, K], scale fp32 [..., ceil(N/bn), ceil(K/bk)])."""
    bn, bk = block
    *lead, n, k = w.shape
    nb, kb = -(-n // bn), -(-k // bk)
    wp = torch.zeros(*lead, nb * bn, kb * bk, dtype=torch.float32)
    wp[..., :n, :k] = w.float()
    blocks = wp.reshape(*lead, nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(FP8_EPS)          # [..., nb, kb]
    scale = amax / FP8_MAX
    q = blocks / scale[..., :, None, :, None]
    q = fp8_round(q).reshape(*lead, nb * bn, kb * bk)[..., :n, :k].contiguous()
    return q, scale.contiguous()


def dequant_weight_fp8_block(q: torch.Tensor, scale: torch.Tensor, block=(128, 128)):
    bn, bk = block
    *lead, n, k = q.shape
    s = scale.repeat_interleave(bn, dim=-2).repeat_interleave(bk, dim=-1)[..., :n, :k]
    return q.float() * s


def quant_act_fp8_group(x: torch.Tensor, group: int = 128):
    """x [R, K] (any float dtype) -> (q fp8 [R, K], scale fp32 [R, K/group]).

    scale = max(amax, eps) / 448 ; q = rne_sat(x / scale) with a true fp32 divide.
    """
    r, k = x.shape
    assert k % group == 0
    xg = x.float().reshape(r, k // group, group)
    amax = xg.abs().amax(dim=-1).clamp_min(FP8_EPS)
    scale = amax / FP8_MAX
    q = fp8_round(xg / scale[..., None]).reshape(r, k)
    return q, scale


def dequant_act_fp8_group(q: torch.Tensor, scale: torch.Tensor, group: int = 128):
    r, k = q.shape
    return (q.float().reshape(r, k // group, group) * scale[..., None]).reshape(r, k)


# ----------------------------------------------------------------------------- AWQ
def quant_weight_awq(w: torch.Tensor, group: int = 128):
    """w [..., K, N] (K = reduction dim) -> (q uint8 [..., K, N], scales fp16
    [..., K/group, N], zeros uint8 [..., K/group, N])."""
    *lead, k, n = w.shape
    assert k % group == 0
    wg = w.float().reshape(*lead, k // group, group, n)
    wmax = wg.amax(dim=-2)
    wmin = wg.amin(dim=-2)
    scale = ((wmax - wmin).clamp_min(1e-5) / 15.0).to(torch.float16)
    sf = scale.float()
    zero = torch.round(-wmin / sf).clamp(0, 15)
    q = (torch.round(wg / sf[..., None, :]) + zero[..., None, :]).clamp(0, 15)
    return (
        q.reshape(*lead, k, n).to(torch.uint8),
        scale,
        zero.to(torch.uint8),
    )


def awq_pack(v: torch.Tensor) -> torch.Tensor:
    """uint4 values [..., R, N] -> int32 [..., R, N/8]; logical column j of each
    group of eight goes to nibble AWQ_NIBBLE_OF_COLUMN[j]."""
    *lead, r, n = v.shape
    assert n % 8 == 0
    g = v.to(torch.int64).reshape(*lead, r, n // 8, 8)
    out = torch.zeros(*lead, r, n // 8, dtype=torch.int64)
    for j in range(8):
        out |= (g[..., j] & 0xF) << (4 * AWQ_NIBBLE_OF_COLUMN[j])
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def awq_unpack(p: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`awq_pack`: int32 [..., R, N/8] -> uint8 [..., R, N]."""
    *lead, r, n8 = p.shape
    u = p.to(torch.int64) & 0xFFFFFFFF
    cols = [((u >> (4 * AWQ_NIBBLE_OF_COLUMN[j])) & 0xF) for j in range(8)]
    return torch.stack(cols, dim=-1).reshape(*lead, r, n8 * 8).to(torch.uint8)


def dequant_weight_awq(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor,
                       group: int = 128) -> torch.Tensor:
    """(packed int32 [..., K, N/8], fp16 [..., K/g, N], packed int32 [..., K/g, N/8])
    -> fp32 [..., K, N] with w = (q - z) * s."""
    q = awq_unpack(qweight).float()
    z = awq_unpack(qzeros).float().repeat_interleave(group, dim=-2)
    s = scales.float().repeat_interleave(group, dim=-2)
    return (q - z) * s
