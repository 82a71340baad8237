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
