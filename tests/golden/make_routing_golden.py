"""Generates tests/golden/routing_golden.npz by running the REFERENCE's own
routing conversion (src/flaggems_sglang/ops/fused_moe.py:103-130,
`_standard_topk_to_triton_kernels`) on CPU.

Runs only where the reference tree is available (pass its path as the first
argument, or set REFERENCE_ROOT) and where the dependency it imports (`triton_kernels`) can be
found inside the installed vllm wheel.  The inputs follow the recipe of the
reference's test (tests/test_fused_moe.py:15-27, 50-58): seed M+K+N+E+topk,
logits randn(M, E), softmax, top-k, renormalise.

    python tests/golden/make_routing_golden.py /path/to/reference
"""
import importlib
import os
import sys
import types
from pathlib import Path

import numpy as np

ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ["REFERENCE_ROOT"]
os.environ["DNN_VENDOR"] = "nvidia"
sys.path.insert(0, os.path.join(ref_root, "src"))
import vllm.third_party.triton_kernels as tk  # noqa: E402

sys.modules["triton_kernels"] = tk
for sub in ("matmul_ogs", "routing", "numerics", "swiglu"):
    sys.modules["triton_kernels." + sub] = importlib.import_module("vllm.third_party.triton_kernels." + sub)
stub = types.ModuleType("sgl_kernel")
stub.gelu_and_mul = lambda x, out: None
sys.modules["sgl_kernel"] = stub

import torch  # noqa: E402
from flaggems_sglang.ops.fused_moe import _standard_topk_to_triton_kernels  # noqa: E402

# (M, K, N, E, topk): the reference's own test shapes (tests/accuracy_utils.py:100-118)
# plus the BASELINE configurations' routing shapes at small M.
SHAPES = [
    (1, 128, 256, 8, 2), (7, 128, 256, 8, 2), (33, 256, 512, 16, 4),
    (1, 1280, 3072, 64, 8), (4, 1280, 3072, 64, 8), (17, 1280, 3072, 64, 8), (64, 1280, 3072, 64, 8),
    (1024, 1280, 3072, 64, 8),
    (64, 1024, 512, 8, 2), (16, 4096, 14336, 8, 2), (32, 2048, 768, 128, 8), (64, 7168, 2048, 256, 8),
]

out = {}
for (M, K, N, E, topk) in SHAPES:
    # the routing only depends on the logits: draw them from a dedicated generator
    # seeded like the reference test, without materialising the weights
    gen = torch.Generator().manual_seed(M + K + N + E + topk)
    logits = torch.randn(M, E, generator=gen, dtype=torch.float32)
    w = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(w, k=topk, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    rd, g, s = _standard_topk_to_triton_kernels(w, ids, E)
    key = f"M{M}_E{E}_k{topk}"
    out[key + "/topk_weights"] = w.numpy()
    out[key + "/topk_ids"] = ids.numpy().astype(np.int32)
    out[key + "/gate_scal"] = rd.gate_scal.numpy()
    out[key + "/hist"] = rd.expt_hist.numpy()
    out[key + "/topk_indx"] = g.src_indx.numpy()
    out[key + "/gate_indx"] = g.dst_indx.numpy()
    assert torch.equal(s.src_indx, g.dst_indx) and torch.equal(s.dst_indx, g.src_indx)
    out[key + "/token_offs_raw"] = rd.expt_data.token_offs_raw.numpy()
    for bm in (16, 32, 64, 128):
        out[key + f"/token_offs_pad_{bm}"] = rd.expt_data.token_offs_pad[bm].numpy()
        out[key + f"/block_pid_map_{bm}"] = rd.expt_data.block_pid_map[bm].numpy()

dst = Path(__file__).resolve().parent / "routing_golden.npz"
np.savez_compressed(dst, **out)
print("wrote", dst, dst.stat().st_size, "bytes,", len(SHAPES), "cases")
