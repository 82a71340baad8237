"""Generates tests/golden/fused_moe_ref_golden.npz: outputs of the REFERENCE's own
`triton_kernel_fused_experts` (src/flaggems_sglang/ops/fused_moe.py:133-216) on a
CUDA device, for the reference's test shapes (tests/accuracy_utils.py:100-118)
with the reference's input recipe (tests/test_fused_moe.py:50-58; tensors are
drawn on the CPU generator and then moved, so that the inputs can be rebuilt
anywhere).

Needs a GPU, the unmodified reference installed under baseline/_ref
(`pip install --no-deps --target baseline/_ref <reference tree>`) and the
`triton_kernels` package bundled in the installed vllm wheel (baseline/ref_shim.py).
From M = 1024 on the file keeps every 16th token row of the output.

    python tests/golden/make_fused_moe_golden.py [out.npz]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT / "baseline"))
from ref_shim import load_reference  # noqa: E402

flaggems_sglang, _standard_topk_to_triton_kernels = load_reference()   # the reference, from baseline/_ref

import torch  # noqa: E402

# from M = 1024 on only every 16th token row is kept (the whole outputs would add tens of MB)
ROW_STRIDE_FROM = 1024
ROW_STRIDE = 16

SHAPES = [(1, 128, 256, 8, 2), (7, 128, 256, 8, 2), (33, 256, 512, 16, 4),
          (1, 1280, 3072, 64, 8), (4, 1280, 3072, 64, 8), (17, 1280, 3072, 64, 8), (64, 1280, 3072, 64, 8),
          (1024, 1280, 3072, 64, 8), (2048, 1280, 3072, 64, 8), (4096, 1280, 3072, 64, 8)]

dev = torch.device("cuda:0")
out = {}
for shape in SHAPES:
    M, K, N, E, topk = shape
    torch.manual_seed(M + K + N + E + topk)
    x = torch.randn(M, K, dtype=torch.bfloat16)
    w1 = torch.randn(E, K, N * 2, dtype=torch.bfloat16) * 0.1
    w2 = torch.randn(E, N, K, dtype=torch.bfloat16) * 0.1
    logits = torch.randn(M, E, dtype=torch.float32)
    tw = torch.softmax(logits, dim=-1)
    tw, ids = torch.topk(tw, k=topk, dim=-1)
    tw = tw / tw.sum(dim=-1, keepdim=True)
    rd, gi, si = _standard_topk_to_triton_kernels(tw.to(dev), ids.to(dev), E)
    key = "M%d_K%d_N%d_E%d_topk%d" % shape
    for gate_in in (False, True):
        if gate_in and M * K * N > 33 * 256 * 512:
            continue
        res = flaggems_sglang.triton_kernel_fused_experts(x.to(dev), w1.to(dev), w2.to(dev), rd, gi, si,
                                                          apply_router_weight_on_input=gate_in)
        torch.cuda.synchronize()
        if M >= ROW_STRIDE_FROM:
            out[key + f"/out_rows{ROW_STRIDE}"] = res[::ROW_STRIDE].contiguous().cpu().view(torch.int16).numpy()
        else:
            out[key + ("/gate_in" if gate_in else "/out")] = res.cpu().view(torch.int16).numpy()
    print(key, "ok", float(res.float().abs().max()))

dst = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parent / "fused_moe_ref_golden.npz"
np.savez_compressed(dst, **out)
print("wrote", dst, dst.stat().st_size, "bytes")
