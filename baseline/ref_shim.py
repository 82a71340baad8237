"""Imports the UNMODIFIED reference package (installed under baseline/_ref with
`pip install --no-deps --target baseline/_ref <reference tree>`) on a machine where its
dependencies `triton_kernels` and `sgl_kernel` are not installed under those names.

`triton_kernels` is taken from the copy bundled in the installed vllm wheel (same API as the
reference's call sites: src/flaggems_sglang/ops/fused_moe.py:16, 105-110); `sgl_kernel` is
stubbed (the reference only needs the name `gelu_and_mul` to import,
src/flaggems_sglang/ops/fused_moe.py:18-21).  Used by the golden-vector generator and by
`bench.py --impl reference-gpu`; never by the product package.
"""
import importlib
import os
import sys
import types
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


def load_reference():
    """Returns (flaggems_sglang module of the reference, its _standard_topk_to_triton_kernels)."""
    if not (REF_DIR / "flaggems_sglang").is_dir():
        raise RuntimeError(f"{REF_DIR} holds no reference install")
    os.environ["DNN_VENDOR"] = "nvidia"       # skips the reference's nvidia-smi probe
    for name in [m for m in sys.modules if m == "flaggems_sglang" or m.startswith("flaggems_sglang.")]:
        del sys.modules[name]                  # the B200 alias package must not answer to this name here
    sys.path.insert(0, str(REF_DIR))
    import vllm.third_party.triton_kernels as tk
    sys.modules["triton_kernels"] = tk
    for sub in ("matmul_ogs", "routing", "numerics", "swiglu"):
        sys.modules["triton_kernels." + sub] = importlib.import_module("vllm.third_party.triton_kernels." + sub)
    stub = types.ModuleType("sgl_kernel")
    stub.gelu_and_mul = lambda x, out: None
    sys.modules["sgl_kernel"] = stub
    import flaggems_sglang
    from flaggems_sglang.ops.fused_moe import _standard_topk_to_triton_kernels
    assert "_ref" in flaggems_sglang.__file__, flaggems_sglang.__file__
    return flaggems_sglang, _standard_topk_to_triton_kernels
