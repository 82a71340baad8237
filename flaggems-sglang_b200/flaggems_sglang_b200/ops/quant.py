"""Stand-alone dynamic FP8 quantisation of activations (1 x 128 groups)."""
from __future__ import annotations

import torch

from .. import _lib

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128):
    """x [rows, K] (bf16 / fp16, CUDA) -> (q float8_e4m3fn [rows, K], scale fp32 [rows, K/128]).

    scale = max(amax, 1e-10) / 448 per group, q = round-to-nearest-even, saturating.
    The step listed in the reference's shape tables (benchmark/core_shapes.yaml:311-317)
    for which it ships no operator."""
    if not x.is_cuda:
        raise RuntimeError("x must be a CUDA tensor: this package has no CPU path")
    assert group_size == 128, "only 1x128 groups are implemented"
    assert x.ndim == 2 and x.shape[1] % 128 == 0, "x must be [rows, K] with K a multiple of 128"
    x = x.contiguous()
    rows, k = x.shape
    q = torch.empty(rows, k, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(rows, k // 128, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().b200moe_per_token_group_quant_fp8(
            x.data_ptr(), _DTYPES[x.dtype], rows, k, q.data_ptr(), s.data_ptr(),
            torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "per_token_group_quant_fp8")
    return q, s
