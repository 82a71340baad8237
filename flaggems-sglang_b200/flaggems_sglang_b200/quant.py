"""Offline weight quantisers / packers (torch, any device).  One-time set-up
work: nothing here runs inside a forward call.

FP8: float8_e4m3fn with one fp32 scale per 128x128 block (amax / 448).
int4 AWQ: asymmetric uint4 per output column and group of 128 along the
reduction dim, eight output columns per int32 in the AWQ nibble order.
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
_AWQ_SHIFTS = (0, 16, 4, 20, 8, 24, 12, 28)   # bit offset of logical column j inside its int32


def quantize_fp8_block(w: torch.Tensor, block: int = 128):
    """w [E, N, K] -> (float8_e4m3fn [E, N, K], fp32 scales [E, ceil(N/b), ceil(K/b)])."""
    e, n, k = w.shape
    nb, kb = -(-n // block), -(-k // block)
    q = torch.empty(e, n, k, dtype=torch.float8_e4m3fn, device=w.device)
    scales = torch.empty(e, nb, kb, dtype=torch.float32, device=w.device)
    for ei in range(e):                      # per expert keeps the fp32 temporaries small
        wf = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
        wf[:n, :k] = w[ei]
        t = wf.view(nb, block, kb, block)
        s = t.abs().amax(dim=(1, 3)).clamp_min(1e-10) / FP8_MAX
        scales[ei] = s
        qq = (t / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        q[ei] = qq.view(nb * block, kb * block)[:n, :k]
    return q, scales


def quantize_awq(w: torch.Tensor, group: int = 128):
    """w [E, K, N] (K = reduction dim) -> (qweight int32 [E, K, N/8], scales fp16
    [E, K/g, N], qzeros int32 [E, K/g, N/8])."""
    e, k, n = w.shape
    assert k % group == 0 and n % 8 == 0
    wg = w.float().view(e, k // group, group, n)
    wmax, wmin = wg.amax(dim=2), wg.amin(dim=2)
    scales = ((wmax - wmin).clamp_min(1e-5) / 15.0).to(torch.float16)
    sf = scales.float()
    zeros = torch.round(-wmin / sf).clamp_(0, 15)
    q = (torch.round(wg / sf[:, :, None, :]) + zeros[:, :, None, :]).clamp_(0, 15)
    return pack_awq(q.view(e, k, n).to(torch.int32)), scales, pack_awq(zeros.to(torch.int32))


def pack_awq(v: torch.Tensor) -> torch.Tensor:
    """uint4 values (int32 tensor) [..., R, N] -> int32 [..., R, N/8]."""
    g = v.view(*v.shape[:-1], v.shape[-1] // 8, 8).to(torch.int64)
    out = torch.zeros(g.shape[:-1], dtype=torch.int64, device=v.device)
    for j, sh in enumerate(_AWQ_SHIFTS):
        out += (g[..., j] & 0xF) << sh
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def unpack_awq(p: torch.Tensor) -> torch.Tensor:
    """int32 [..., R, N/8] in the AWQ nibble order -> int32 values 0..15 [..., R, N]."""
    u = p.to(torch.int64) & 0xFFFFFFFF
    cols = [((u >> sh) & 0xF) for sh in _AWQ_SHIFTS]
    return torch.stack(cols, dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 8).to(torch.int32)


def repack_awq_for_kernel(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor, group: int = 128):
    """AWQ checkpoint tensors -> the layout the int4 kernels stream (one-time set-up).

    qweight [E, K, N/8] int32, scales [E, K/g, N] fp16, qzeros [E, K/g, N/8] int32
    (K = reduction dim, N = output dim) become

      wp [E, N, K/8] int32   one output row per line, reduction dim contiguous; a word
                             holds eight consecutive k: element 2i in nibble i, element
                             2i+1 in nibble 4+i, so that (w >> 4i) & 0x000F000F is the
                             adjacent pair (2i, 2i+1) as two 16-bit lanes;
      sz [E, K/g, N] int32   per (group, output row): fp16 scale in the low half,
                             fp16(1024 + zero) in the high half.
    """
    assert group == 128
    e, k, n8 = qweight.shape
    n = n8 * 8
    q = unpack_awq(qweight).transpose(1, 2).contiguous()          # [E, N, K]
    g8 = q.view(e, n, k // 8, 8).to(torch.int64)
    wp = torch.zeros(e, n, k // 8, dtype=torch.int64, device=q.device)
    for i in range(4):
        wp += (g8[..., 2 * i] & 0xF) << (4 * i)
        wp += (g8[..., 2 * i + 1] & 0xF) << (16 + 4 * i)
    wp = torch.where(wp >= 2 ** 31, wp - 2 ** 32, wp).to(torch.int32)
    z = unpack_awq(qzeros).to(torch.float16) + 1024.0              # [E, K/g, N], exact in fp16
    s_bits = scales.to(torch.float16).contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    z_bits = z.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
    sz = s_bits | (z_bits << 16)
    sz = torch.where(sz >= 2 ** 31, sz - 2 ** 32, sz).to(torch.int32)
    return wp.contiguous(), sz.contiguous()
