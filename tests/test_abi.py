"""CPU: the shared object loads, exports every symbol the header declares, and
its host-only entry points agree with the oracle.  No kernel is launched."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import routing as R

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (ROOT / "include" / "b200moe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_lib):
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(built_lib, n), f"{n} declared in include/b200moe.h but not exported"


def test_binding_covers_header(built_lib):
    from flaggems_sglang_b200 import _lib
    assert sorted(_lib.SYMBOLS) == _declared_symbols()
    assert built_lib.b200moe_version() == _lib.VERSION
    assert C.sizeof(_lib.Cfg) == 15 * 4


@pytest.mark.parametrize("p,e,b", [(0, 8, 16), (2, 8, 16), (128, 8, 64), (8192, 8, 256), (2048, 128, 16),
                                   (32768, 256, 128), (5, 3, 128)])
def test_capacity_matches_oracle(built_lib, p, e, b):
    assert built_lib.b200moe_align_capacity(p, e, b) == R.align_capacity(p, e, b)
    assert built_lib.b200moe_routing_max_tiles(p, e) == R.max_tiles(p, e)


def test_argument_errors(built_lib):
    from flaggems_sglang_b200 import _lib
    assert built_lib.b200moe_align_capacity(-1, 8, 16) == _lib.ERR_BAD_ARG
    bad = _lib.Cfg(4, 1, 128, 128, 8, 2, 0, 0, 0, 0, 0, 0, 1.0, 0)
    assert built_lib.b200moe_workspace_bytes(C.byref(bad)) == 0
    assert built_lib.b200moe_pick_block_tokens(C.byref(bad)) == _lib.ERR_BAD_ARG
    ok = _lib.Cfg(C.sizeof(_lib.Cfg), 64, 1024, 512, 8, 2, 0, 0, 0, 0, 0, 0, 1.0, 148)
    assert built_lib.b200moe_pick_block_tokens(C.byref(ok)) in (16, 32, 64, 128, 256)
    assert built_lib.b200moe_workspace_bytes(C.byref(ok)) > 64 * 1024 * 4
    odd = _lib.Cfg(C.sizeof(_lib.Cfg), 64, 1023, 512, 8, 2, 0, 0, 0, 0, 0, 0, 1.0, 148)
    assert built_lib.b200moe_pick_block_tokens(C.byref(odd)) == _lib.ERR_UNSUPPORTED
    assert built_lib.b200moe_status_string(_lib.ERR_WORKSPACE).decode().startswith("workspace")


def test_matrix_vector_path_selection(built_lib):
    """Which problems the forward calls run on the two matrix-vector kernels (host arithmetic only)."""
    from flaggems_sglang_b200 import _lib

    def uses(m, h, i, e, k, wmode=_lib.W_16BIT, dtype=0, block_tokens=0, flags=0):
        cfg = _lib.Cfg(C.sizeof(_lib.Cfg), m, h, i, e, k, dtype, wmode, 0, 0, flags, block_tokens, 1.0, 148)
        return built_lib.b200moe_uses_matrix_vector_path(C.byref(cfg))

    assert uses(1, 4096, 14336, 8, 2) == 1                     # one token: always, its experts are distinct
    assert uses(1, 2048, 768, 128, 8) == 1
    assert uses(2, 2048, 768, 128, 8) == 1                     # 16 pairs over 128 experts
    assert uses(2, 4096, 14336, 8, 2) == 0                     # 4 pairs over 8 experts: they would meet
    assert uses(3, 2048, 768, 128, 8) == 0                     # 24 pairs
    assert uses(1, 2048, 768, 128, 8, block_tokens=16) == 0    # the caller asked for the grouped GEMMs
    assert uses(1, 7168, 2048, 256, 8, wmode=_lib.W_FP8_BLOCK) == 0
    assert uses(1, 4096, 14336, 8, 2, wmode=_lib.W_INT4_AWQ, dtype=1) == 1
    assert uses(1, 4096, 14336, 8, 2, flags=_lib.FLAG_SIMT) == 0
    assert uses(1, 4096, 32768, 8, 4) == 0                     # 4 x 32768 fp32 activations do not fit in shared memory
    bad = _lib.Cfg(4, 1, 128, 128, 8, 2, 0, 0, 0, 0, 0, 0, 1.0, 0)
    assert built_lib.b200moe_uses_matrix_vector_path(C.byref(bad)) == _lib.ERR_BAD_ARG


def test_product_fails_loudly_without_gpu():
    import torch
    import flaggems_sglang_b200 as F
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    w13 = torch.zeros(2, 256, 128, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        F.fused_experts(x, w13, w2, torch.ones(2, 1), torch.zeros(2, 1, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        F.moe_align_block_size(torch.zeros(2, 1, dtype=torch.int32), 16, 2)


def test_reference_error_conventions():
    import torch
    import flaggems_sglang
    from flaggems_sglang_b200 import RoutingData, GatherIndx, ScatterIndx
    z = torch.zeros(1, dtype=torch.int32)
    rd = RoutingData(torch.ones(2), z, 2, 1, None)
    gi, si = GatherIndx(z, z), ScatterIndx(z, z)
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    w1 = torch.zeros(2, 128, 256, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        flaggems_sglang.triton_kernel_fused_experts(x, w1, w2, rd, gi, si, inplace=True)
    with pytest.raises(AssertionError):
        flaggems_sglang.triton_kernel_fused_experts(x.float(), w1, w2, rd, gi, si)
    with pytest.raises(AssertionError):
        flaggems_sglang.triton_kernel_fused_experts(x, w1, w2, rd, gi, si, per_channel_quant=True)
    with pytest.raises(ValueError):
        flaggems_sglang.triton_kernel_fused_experts(x, w1, w2, rd, gi, si, activation="relu")


def test_bias_variant_error_conventions():
    """Same exception types as the reference's bias variant (fused_moe.py:247-261): asserts for
    inplace / dtype, ValueError for any activation but silu."""
    import torch
    import flaggems_sglang
    from flaggems_sglang_b200 import RoutingData, GatherIndx, ScatterIndx
    z = torch.zeros(1, dtype=torch.int32)
    rd = RoutingData(torch.ones(2), z, 2, 1, None)
    gi, si = GatherIndx(z, z), ScatterIndx(z, z)
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    w1 = torch.zeros(2, 128, 256, dtype=torch.bfloat16)
    w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16)
    b1 = torch.zeros(2, 256, dtype=torch.bfloat16)
    b2 = torch.zeros(2, 128, dtype=torch.bfloat16)
    f = flaggems_sglang.triton_kernel_fused_experts_with_bias
    with pytest.raises(AssertionError):
        f(x, w1, None, b1, w2, None, b2, rd, gi, si, inplace=True)
    with pytest.raises(AssertionError):
        f(x.float(), w1, None, b1, w2, None, b2, rd, gi, si)
    with pytest.raises(ValueError):
        f(x, w1, None, b1, w2, None, b2, rd, gi, si, activation="gelu")


def test_router_python_validation():
    """The router's Python layer refuses CPU tensors (no CPU path) and unknown scoring names."""
    import torch
    from flaggems_sglang_b200.ops.router import make_router
    with pytest.raises(AssertionError):
        make_router(torch.zeros(4, 8), 2, True)
    if torch.cuda.is_available():
        with pytest.raises(ValueError):
            make_router(torch.zeros(4, 8, device="cuda"), 2, True, scoring_func="tanh")


def test_workspace_grows_with_the_optional_paths(built_lib):
    """Workspace queries run without a GPU and account for the path-specific buffers."""
    import ctypes as C
    from flaggems_sglang_b200 import _lib
    lib = _lib.lib()

    def ws(m, h, i, e, k, wmode, dtype=_lib.DTYPE_BF16, flags=0):
        cfg = _lib.Cfg(C.sizeof(_lib.Cfg), m, h, i, e, k, dtype, wmode, _lib.LAYOUT_LAYER, 0, flags, 0, 1.0, 0)
        return lib.b200moe_workspace_bytes(C.byref(cfg))

    small = ws(64, 1024, 512, 8, 2, _lib.W_16BIT)
    assert 0 < small < ws(64, 1024, 512, 8, 2, _lib.W_16BIT, flags=_lib.FLAG_NO_COMBINE)      # [P, H] instead of [M, H]
    big_fp8 = ws(4096, 7168, 2048, 256, 8, _lib.W_FP8_BLOCK)
    assert big_fp8 > 4096 * 8 * 7168 * 2                        # 16-bit pair rows are part of it
    assert ws(4096, 7168, 2048, 256, 8, _lib.W_FP8_BLOCK, flags=_lib.FLAG_X_FP8) < big_fp8     # no quantise-once buffers
    assert ws(32, 4096, 14336, 8, 2, _lib.W_INT4_AWQ, dtype=_lib.DTYPE_FP16) > 0
    assert ws(32, 4096, 14336, 8, 2, _lib.W_INT4_AWQ) == 0      # int4 needs fp16 activations
    assert ws(64, 1024, 512, 8, 2, _lib.W_16BIT, flags=_lib.FLAG_X_FP8) == 0                   # FP8 rows need FP8 weights
