"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h)."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from ._build import LIB_PATH

VERSION = 2

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_TOO_LARGE = -1, -2, -3, -4, -5, -6

DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
ROUTER_MAX_EXPERTS, ROUTER_MAX_TOPK = 1024, 32
W_16BIT, W_FP8_BLOCK, W_INT4_AWQ = 0, 1, 2
LAYOUT_LAYER, LAYOUT_OP = 0, 1
ACT_SILU, ACT_GELU, ACT_SWIGLU_OAI = 0, 1, 2
NOALLOC_SCRATCH_BYTES = 16 * 1024 * 1024
FLAG_WEIGHT_ON_INPUT, FLAG_MIMIC_ROUNDING, FLAG_SIMT, FLAG_IDS_I64, FLAG_NO_SPLIT_K, \
    FLAG_NO_GRID_BALANCE, FLAG_NO_PDL, FLAG_W4_SMEM_OPERANDS, FLAG_NO_COMBINE, FLAG_ALIGN_ONE_CTA, FLAG_X_FP8 = \
    1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024
FLAG_EP_DIAG_LOCAL_COMBINE = 2048
FLAG_CTA_PAIR = 4096


class Cfg(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_int32), ("M", C.c_int32), ("H", C.c_int32), ("I", C.c_int32),
        ("E", C.c_int32), ("topk", C.c_int32), ("dtype", C.c_int32), ("wmode", C.c_int32),
        ("w_layout", C.c_int32), ("activation", C.c_int32), ("flags", C.c_int32),
        ("block_tokens", C.c_int32), ("routed_scaling", C.c_float), ("num_sms", C.c_int32),
        ("n_global_experts", C.c_int32),
    ]


class Quant(C.Structure):
    _fields_ = [("w1_scale", C.c_void_p), ("w2_scale", C.c_void_p), ("w1_sz", C.c_void_p), ("w2_sz", C.c_void_p),
                ("b1", C.c_void_p), ("b2", C.c_void_p), ("swiglu_alpha", C.c_float), ("swiglu_limit", C.c_float),
                ("x_scale", C.c_void_p)]


class EpCfg(C.Structure):
    _fields_ = [("struct_bytes", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32), ("m_cap", C.c_int32),
                ("n_global_experts", C.c_int32), ("reserved", C.c_int32), ("wait_limit_ns", C.c_uint64)]


EP_MAX_RANKS = 8
EP_PHASE_DISPATCH, EP_PHASE_COMPUTE, EP_PHASE_COMBINE, EP_PHASE_ALL = 1, 2, 4, 7


class Router(C.Structure):
    _fields_ = [("struct_bytes", C.c_int32), ("scoring", C.c_int32), ("renormalize", C.c_int32),
                ("n_group", C.c_int32), ("topk_group", C.c_int32), ("logits_dtype", C.c_int32),
                ("scale", C.c_float), ("reserved", C.c_int32), ("bias", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/b200moe.h declares
SYMBOLS = {
    "b200moe_version": (C.c_int, []),
    "b200moe_status_string": (C.c_char_p, [C.c_int]),
    "b200moe_pick_block_tokens": (C.c_int, [C.POINTER(Cfg)]),
    "b200moe_uses_matrix_vector_path": (C.c_int, [C.POINTER(Cfg)]),
    "b200moe_workspace_bytes": (C.c_size_t, [C.POINTER(Cfg)]),
    "b200moe_align_capacity": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "b200moe_align_block_size": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_routing_max_tiles": (C.c_int, [C.c_int, C.c_int]),
    "b200moe_routing_from_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_forward_topk": (C.c_int, [C.POINTER(Cfg), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Quant),
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                       C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_forward_topk_noalloc": (C.c_int, [C.POINTER(Cfg), C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.POINTER(Quant), C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_forward_routed": (C.c_int, [C.POINTER(Cfg), C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Quant),
                                         C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_route_topk": (C.c_int, [C.POINTER(Router), C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_void_p]),
    "b200moe_forward_logits": (C.c_int, [C.POINTER(Cfg), C.POINTER(Router), C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.POINTER(Quant), C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_profile_begin": (C.c_int, [C.c_int]),
    "b200moe_profile_end": (C.c_int, [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                      C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "b200moe_ep_heap_bytes": (C.c_size_t, [C.POINTER(Cfg), C.POINTER(EpCfg)]),
    "b200moe_ep_workspace_bytes": (C.c_size_t, [C.POINTER(Cfg), C.POINTER(EpCfg)]),
    "b200moe_ep_heap_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "b200moe_ep_heap_free": (C.c_int, [C.c_void_p]),
    "b200moe_ep_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200moe_ep_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200moe_ep_ipc_close": (C.c_int, [C.c_void_p]),
    "b200moe_ep_forward": (C.c_int, [C.POINTER(Cfg), C.POINTER(EpCfg), C.POINTER(C.c_void_p), C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.POINTER(Quant), C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_debug_resident_cta_pairs": (C.c_int, []),
    "b200moe_launch_stats": (C.c_int, [C.POINTER(C.c_longlong), C.c_char_p, C.c_size_t]),
    "b200moe_selftest_timeout": (C.c_int, [C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_per_token_group_quant_fp8": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                    C.c_void_p, C.c_void_p]),
}

_lib = None


class ExtensionMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the shared object; there is no fallback when it is missing."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get("B200MOE_LIB", LIB_PATH))   # override: development builds
        if not path.exists():
            raise ExtensionMissing(
                f"{path} is not built. Run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(or `python -m flaggems_sglang_b200._build`) first; this package has no CPU or "
                "PyTorch fallback for the fused-MoE path.")
        handle = C.CDLL(str(path))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        if handle.b200moe_version() != VERSION:
            raise ExtensionMissing(f"{path} has ABI version {handle.b200moe_version()}, expected {VERSION}")
        _lib = handle
    return _lib


def launch_stats():
    """(kernels launched since the library was loaded, names of the most recent forward call's kernels)."""
    total = C.c_longlong()
    buf = C.create_string_buffer(4096)
    lib().b200moe_launch_stats(C.byref(total), buf, len(buf))
    names = buf.value.decode()
    return total.value, (names.split(",") if names else [])


def status_string(code: int) -> str:
    return lib().b200moe_status_string(code).decode()


def check(code: int, what: str) -> None:
    if code == OK:
        return
    msg = f"{what}: {status_string(code)} ({code})"
    if code in (ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_TOO_LARGE):
        raise ValueError(msg)
    raise RuntimeError(msg)
