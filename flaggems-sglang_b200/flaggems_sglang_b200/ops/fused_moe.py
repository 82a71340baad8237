"""Fused Mixture-of-Experts operator for B200 (sm_100a).

Drop-in for the fused-MoE entry points of ``flaggems_sglang.ops``
(src/flaggems_sglang/ops/fused_moe.py in the reference tree): the same names,
positional order, defaults and exception types, implemented by a C-ABI CUDA
library instead of Triton.  Python here only validates, allocates and launches.
"""
from __future__ import annotations

import ctypes as C
import logging
import os
from types import SimpleNamespace
from typing import Optional

import torch
from torch.utils.weak import WeakIdKeyDictionary

from .. import _lib
from ..routing import topk_to_routing

logger = logging.getLogger(__name__)

_UNSUPPORTED_FEATURE_MSG = "{name} is not supported"

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}
_ACTS = {"silu": _lib.ACT_SILU, "gelu": _lib.ACT_GELU, "swiglu_oai": _lib.ACT_SWIGLU_OAI}

# ---------------------------------------------------------------------------- state
_workspaces: dict = {}     # (device index, stream handle) -> uint8 tensor
_status: dict = {}         # device index -> int32[1]
# re-laid-out weights, keyed by the identity of the caller's tensor object (a dictionary keyed by
# tensor *value* would compare two tensors with ==, which has no truth value)
_relayout = WeakIdKeyDictionary()


MAX_CACHED_WORKSPACES = 8     # (device, stream) pairs that keep a scratch buffer between calls
_captured: list = []          # buffers a CUDA graph under capture was given: a replay writes to them


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch buffer of the calling (device, stream), kept between calls so that the hot path
    does not allocate; it grows to the largest call seen on that stream.  At most
    MAX_CACHED_WORKSPACES pairs keep one (the least recently used goes first) and
    ``release_workspaces`` drops them all.  A buffer handed out while the stream is being
    captured into a CUDA graph is never dropped: replays of the graph keep using it."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.pop(key, None)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(int(nbytes * 1.25) + 4096, dtype=torch.uint8, device=dev)
    _workspaces[key] = ws                     # re-inserted last: dict order is the LRU order
    while len(_workspaces) > MAX_CACHED_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))
    if torch.cuda.is_current_stream_capturing() and not any(ws is c for c in _captured):
        _captured.append(ws)
    return ws


def release_workspaces(device=None) -> None:
    """Drop the cached scratch buffers (of one device, or of all), e.g. after a one-off
    prefill-sized call whose scratch should not stay allocated.  Buffers that a captured CUDA
    graph uses are kept."""
    idx = None if device is None else (torch.device(device).index or 0)
    for key in [k for k in _workspaces if idx is None or k[0] == idx]:
        _workspaces.pop(key)


def _status_word(dev: torch.device) -> torch.Tensor:
    st = _status.get(dev.index)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[dev.index] = st
    return st


_status_host: dict = {}    # device index -> pinned int32[1] that trails the device word
_status_calls: dict = {}
STATUS_COPY_EVERY = 16     # calls between two asynchronous copies of the status word to the host


def _deferred_status_check(dev: torch.device, status: torch.Tensor) -> None:
    """Catches a device-side time-out without ever synchronising: after every
    ``STATUS_COPY_EVERY``-th call the status word is copied (asynchronously, four bytes) to pinned
    host memory, and every call looks at the host copy first.  A time-out therefore surfaces a
    few calls after the kernels that hit it have finished, even in a host that never calls
    ``check_status()``.  ``B200MOE_DEFERRED_STATUS=0`` switches it off."""
    if os.environ.get("B200MOE_DEFERRED_STATUS", "1") == "0":
        return
    host = _status_host.get(dev.index)
    if host is None:
        host = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_host[dev.index] = host
        _status_calls[dev.index] = 0
    elif not torch.cuda.is_current_stream_capturing():
        code = int(host[0])          # plain host read: whatever an earlier copy has delivered
        if code != 0:
            host.zero_()
            status.zero_()
            raise RuntimeError(f"b200moe: a device-side wait timed out (code {code}) in an earlier call on "
                               f"cuda:{dev.index}; that call's output is invalid")
    _status_calls[dev.index] += 1
    if _status_calls[dev.index] % STATUS_COPY_EVERY == 1 and not torch.cuda.is_current_stream_capturing():
        host.copy_(status, non_blocking=True)


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel reported a device-side time-out since
    the last check.  Never called on the hot path."""
    devs = list(_status) if device is None else [torch.device(device).index or 0]
    for idx in devs:
        st = _status.get(idx)
        if st is None:
            continue
        code = int(st.item())
        if code != 0:
            st.zero_()
            if idx in _status_host:
                _status_host[idx].zero_()
            raise RuntimeError(f"b200moe: device-side wait timed out (code {code}) on cuda:{idx}")


def _cached(w: torch.Tensor, kind: str, stamp: tuple, make):
    """One derived layout per (tensor object, kind), rebuilt when the tensor was written to
    in place (version counter), re-pointed at other storage, or `stamp` changed."""
    per_tensor = _relayout.get(w)
    if per_tensor is None:
        per_tensor = {}
        _relayout[w] = per_tensor
    stamp = (w._version, w.data_ptr()) + stamp
    ent = per_tensor.get(kind)
    if ent is None or ent[0] != stamp:
        ent = (stamp, make())
        per_tensor[kind] = ent
    return ent[1]


def _layer_layout(w: torch.Tensor) -> torch.Tensor:
    """Op-level weights are [E, K, N] (reference layout, output dim contiguous);
    the kernels stream [E, N, K].  A transposed view of a [E, N, K] tensor is used
    as is; anything else is re-laid out once and remembered per tensor object."""
    wt = w.transpose(-1, -2)
    if wt.is_contiguous():
        return wt
    return _cached(w, "layer", (), wt.contiguous)


def _awq_repacked(qweight: torch.Tensor, scales: torch.Tensor, qzeros: torch.Tensor):
    """AWQ checkpoint tensors -> kernel layout, once per qweight tensor object."""
    from ..quant import repack_awq_for_kernel
    return _cached(qweight, "awq", (scales._version, scales.data_ptr(), qzeros._version, qzeros.data_ptr()),
                   lambda: repack_awq_for_kernel(qweight, scales, qzeros))


def _make_cfg(m, h, i, e, k, dtype, wmode, activation, flags, block_tokens, routed_scaling,
              n_global_experts=0) -> _lib.Cfg:
    return _lib.Cfg(C.sizeof(_lib.Cfg), m, h, i, e, k, dtype, wmode, _lib.LAYOUT_LAYER, activation, flags,
                    block_tokens, routed_scaling, 0, n_global_experts)


def _env_flags() -> int:
    f = 0
    if os.environ.get("B200MOE_SIMT", "0") == "1":
        f |= _lib.FLAG_SIMT
    if os.environ.get("B200MOE_ALIGN_ONE_CTA", "0") == "1":
        f |= _lib.FLAG_ALIGN_ONE_CTA
    if os.environ.get("B200MOE_NO_SPLIT_K", "0") == "1":
        f |= _lib.FLAG_NO_SPLIT_K
    if os.environ.get("B200MOE_NO_GRID_BALANCE", "0") == "1":
        f |= _lib.FLAG_NO_GRID_BALANCE
    if os.environ.get("B200MOE_NO_PDL", "0") == "1":
        f |= _lib.FLAG_NO_PDL
    if os.environ.get("B200MOE_W4_SMEM_OPERANDS", "0") == "1":
        f |= _lib.FLAG_W4_SMEM_OPERANDS
    if os.environ.get("B200MOE_CTA_PAIR", "0") == "1":
        f |= _lib.FLAG_CTA_PAIR
    return f


def _block_tokens_env() -> int:
    return int(os.environ.get("B200MOE_BLOCK_TOKENS", "0"))


# ---------------------------------------------------------------------------- layer-layout core
def fused_experts(
    hidden_states: torch.Tensor,
    w13: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: Optional[torch.Tensor] = None,
    topk_ids: Optional[torch.Tensor] = None,
    *,
    routing=None,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    expert_map: Optional[torch.Tensor] = None,
    routed_scaling_factor: float = 1.0,
    mimic_reference_rounding: bool = True,
    block_tokens: int = 0,
    use_fp8_w8a8: bool = False,
    w13_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    use_int4_w4a16: bool = False,
    w13_sz: Optional[torch.Tensor] = None,
    w2_sz: Optional[torch.Tensor] = None,
    b13: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None,
    swiglu_alpha: float = 1.0,
    swiglu_limit: Optional[float] = None,
    no_combine: bool = False,
    router=None,
    x_scale: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Fused experts on layer-layout weights ``w13 [E, 2I, H]``, ``w2 [E, H, I]``.

    ``x_scale`` (FP8 weights only): ``hidden_states`` is already ``float8_e4m3fn``, quantised per
    1x128 group with these scales ``[M, H/128]`` (as ``per_token_group_quant_fp8`` returns them);
    ``out_dtype`` (default bfloat16) then names the type of the intermediate and of the result.

    ``router``: ``(make_router(...) result, topk)``; the call then starts from the gating
    logits and runs the router kernel in front (see ``fused_moe``).

    ``no_combine``: return ``[M, topk, H]``, one weighted expert output per (token, choice)
    pair instead of their sum; ``routed_scaling_factor`` is not applied (the reference's
    adapter skips it too, src/flaggems_sglang/ops/fused_moe.py:399-404).

    ``b13 [E, 2I]`` / ``b2 [E, H]`` (any weight mode): per-expert biases added to
    the two projections.  ``activation="swiglu_oai"``: ``s = g * sigmoid(alpha * g)``,
    ``out = s * (linear + 1)`` with the gate clamped from above and the linear half
    clamped to ``[-limit, limit]`` when ``swiglu_limit`` is given.

    ``use_int4_w4a16``: ``w13`` / ``w2`` are the packed int4 rows ``[E, 2I, H/8]`` /
    ``[E, H, I/8]`` int32 and ``w13_sz`` / ``w2_sz`` the scale/zero tables from
    ``quant.repack_awq_for_kernel``; activations must be fp16.

    Routing is either ``(topk_weights [M, k], topk_ids [M, k])`` or
    ``routing=(hist [E], topk_indx [P], gate_scal [P])`` taken from the
    reference's routing triple.  Returns a new ``[M, H]`` tensor.
    """
    if activation not in _ACTS:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    if not hidden_states.is_cuda:
        raise RuntimeError("hidden_states must be a CUDA tensor: this package has no CPU path")
    x = hidden_states.contiguous()
    dev = x.device
    m, h = x.shape
    e, two_i, hw = w13.shape
    i = two_i // 2
    pack = 8 if use_int4_w4a16 else 1
    assert hw * pack == h, "hidden size mismatch"
    assert w2.shape[0] == e and w2.shape[1] == h and w2.shape[2] * pack == i, "intermediate size mismatch"
    assert w13.is_contiguous() and w2.is_contiguous(), "weights must be contiguous"
    flags = _env_flags()
    odt = x.dtype
    xs_keep = None
    if x.dtype == torch.float8_e4m3fn:
        assert use_fp8_w8a8 and x_scale is not None, "FP8 activations need FP8 weights and x_scale"
        assert h % 128 == 0 and x_scale.shape == (m, h // 128), "x_scale must be [M, H/128]"
        odt = out_dtype or torch.bfloat16
        xs_keep = x_scale.to(torch.float32).contiguous()
        flags |= _lib.FLAG_X_FP8
    else:
        assert x_scale is None, "x_scale goes with float8_e4m3fn hidden_states"
    dtype = _DTYPES[odt]

    if apply_router_weight_on_input:
        flags |= _lib.FLAG_WEIGHT_ON_INPUT
    if mimic_reference_rounding:
        flags |= _lib.FLAG_MIMIC_ROUNDING

    quant = None
    wmode = _lib.W_16BIT
    keep = []                    # converted tensors whose storage the call reads
    if use_fp8_w8a8:
        wmode = _lib.W_FP8_BLOCK
        assert w13.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn, "FP8 weights must be float8_e4m3fn"
        assert w13_scale is not None and w2_scale is not None, "block scales are required"
        s1 = w13_scale.to(torch.float32).contiguous()
        s2 = w2_scale.to(torch.float32).contiguous()
        keep += [s1, s2]
        quant = _lib.Quant(s1.data_ptr(), s2.data_ptr(), None, None)
        if xs_keep is not None:
            quant.x_scale = xs_keep.data_ptr()
    elif use_int4_w4a16:
        wmode = _lib.W_INT4_AWQ
        assert x.dtype == torch.float16, "int4 w4a16 takes fp16 activations"
        assert w13.dtype == torch.int32 and w2.dtype == torch.int32, "packed int4 weights must be int32"
        assert w13_sz is not None and w2_sz is not None, "scale/zero tables are required"
        assert w13_sz.dtype == torch.int32 and w13_sz.shape == (e, h // 128, 2 * i), "w13_sz must be [E, H/128, 2I] int32"
        assert w2_sz.dtype == torch.int32 and w2_sz.shape == (e, i // 128, h), "w2_sz must be [E, I/128, H] int32"
        z1, z2 = w13_sz.contiguous(), w2_sz.contiguous()
        keep += [z1, z2]
        quant = _lib.Quant(None, None, z1.data_ptr(), z2.data_ptr())
    else:
        assert w13.dtype == x.dtype and w2.dtype == x.dtype, "weights must have the activation dtype"
    if b13 is not None or b2 is not None or activation == "swiglu_oai":
        # per-expert biases and the clamped swiglu, for every weight mode
        bias1 = b13.to(torch.float32).contiguous() if b13 is not None else None
        bias2 = b2.to(torch.float32).contiguous() if b2 is not None else None
        if bias1 is not None:
            assert bias1.shape == (e, 2 * i), "b13 must be [E, 2I]"
        if bias2 is not None:
            assert bias2.shape == (e, h), "b2 must be [E, H]"
        keep += [bias1, bias2]
        if quant is None:
            quant = _lib.Quant(None, None, None, None)
        quant.b1 = bias1.data_ptr() if bias1 is not None else None
        quant.b2 = bias2.data_ptr() if bias2 is not None else None
        quant.swiglu_alpha = float(swiglu_alpha)
        quant.swiglu_limit = float(swiglu_limit) if swiglu_limit else 0.0

    lib = _lib.lib()
    if router is not None:
        assert routing is None and topk_weights is None and topk_ids is None, "router excludes other routing inputs"
        (rt, logits, _bias_keepalive), k = router
        assert logits.shape == (m, e), "gating_output must be [tokens, experts]"
    elif routing is None:
        assert topk_weights is not None and topk_ids is not None, "routing or (topk_weights, topk_ids) required"
        k = topk_ids.shape[1]
        ids = topk_ids.contiguous()
        assert ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64"
        if ids.dtype == torch.int64:
            flags |= _lib.FLAG_IDS_I64
        tw = topk_weights.to(torch.float32).contiguous()
    else:
        hist, topk_indx, gate_scal, k = routing
        hist = hist.to(torch.int32).contiguous()
        topk_indx = topk_indx.to(torch.int32).contiguous()
        gate_scal = gate_scal.to(torch.float32).contiguous()

    if no_combine:
        flags |= _lib.FLAG_NO_COMBINE
    if expert_map is not None:
        assert expert_map.ndim == 1 and expert_map.numel() >= e, "expert_map must list every global expert"
    cfg = _make_cfg(m, h, i, e, k, dtype, wmode, _ACTS[activation], flags,
                    block_tokens or _block_tokens_env(), float(routed_scaling_factor),
                    expert_map.numel() if expert_map is not None else 0)
    out = torch.empty((m, k, h) if no_combine else (m, h), dtype=odt, device=dev)
    if m == 0:
        return out
    nbytes = lib.b200moe_workspace_bytes(C.byref(cfg))
    if nbytes == 0:
        rc = lib.b200moe_pick_block_tokens(C.byref(cfg))
        _lib.check(rc if rc < 0 else _lib.ERR_UNSUPPORTED, "fused_experts")
    ws = _workspace(dev, nbytes)
    base = (ws.data_ptr() + 255) & ~255
    avail = ws.numel() - (base - ws.data_ptr())
    status = _status_word(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    qref = C.byref(quant) if quant is not None else None
    with torch.cuda.device(dev):
        if router is not None:
            emap = None
            if expert_map is not None:
                emap = expert_map.to(device=dev, dtype=torch.int32).contiguous()
            rc = lib.b200moe_forward_logits(
                C.byref(cfg), C.byref(rt), x.data_ptr(), w13.data_ptr(), w2.data_ptr(), qref, logits.data_ptr(),
                emap.data_ptr() if emap is not None else None, base, avail, out.data_ptr(),
                status.data_ptr(), stream)
        elif routing is None:
            emap = None
            if expert_map is not None:
                emap = expert_map.to(device=dev, dtype=torch.int32).contiguous()
            rc = lib.b200moe_forward_topk(
                C.byref(cfg), x.data_ptr(), w13.data_ptr(), w2.data_ptr(), qref, tw.data_ptr(), ids.data_ptr(),
                emap.data_ptr() if emap is not None else None, base, avail, out.data_ptr(),
                status.data_ptr(), stream)
        else:
            rc = lib.b200moe_forward_routed(
                C.byref(cfg), x.data_ptr(), w13.data_ptr(), w2.data_ptr(), qref, hist.data_ptr(),
                topk_indx.data_ptr(), gate_scal.data_ptr(), base, avail, out.data_ptr(),
                status.data_ptr(), stream)
    _lib.check(rc, "fused_experts")
    _deferred_status_check(dev, status)
    if os.environ.get("B200MOE_CHECK_STATUS", "0") == "1":
        check_status(dev)
    return out


def fused_moe(
    hidden_states: torch.Tensor,
    w13: torch.Tensor,
    w2: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool = True,
    *,
    num_expert_group: int = 0,
    topk_group: int = 0,
    scoring_func: str = "softmax",
    correction_bias: Optional[torch.Tensor] = None,
    **kwargs,
) -> torch.Tensor:
    """Whole MoE layer from the gating logits ``[M, E]``: router (softmax or sigmoid scores,
    optional expert groups and selection bias, see ``ops.router``), alignment, both grouped
    GEMMs and the combine in one C call with no host read in between.  Remaining keyword
    arguments are those of ``fused_experts``."""
    from .router import make_router
    rt = make_router(gating_output, topk, renormalize, num_expert_group=num_expert_group, topk_group=topk_group,
                     scoring_func=scoring_func, correction_bias=correction_bias)
    return fused_experts(hidden_states, w13, w2, router=(rt, topk), **kwargs)


# ---------------------------------------------------------------------------- reference-compatible entry points
def triton_kernel_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    routing_data,
    gather_indx,
    scatter_indx,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    expert_map: Optional[torch.Tensor] = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
    *,
    use_int4_w4a16: bool = False,
    w1_zp: Optional[torch.Tensor] = None,
    w2_zp: Optional[torch.Tensor] = None,
    group_size: int = 128,
) -> torch.Tensor:
    """Same signature and results as the reference's op
    (src/flaggems_sglang/ops/fused_moe.py:133-216): ``w1 [E, H, 2I]``,
    ``w2 [E, I, H]``, routing as the dependency's triple (read by attribute).

    Beyond the reference: ``use_fp8_w8a8=True`` with ``w1_scale``/``w2_scale``
    and ``block_shape=[128, 128]`` runs the block-quantised FP8 path (weights
    then come in layer layout ``[E, 2I, H]`` / ``[E, H, I]``).  Keyword-only
    ``use_int4_w4a16=True`` takes AWQ checkpoint tensors: ``w1`` / ``w2`` =
    qweight ``[E, K, N/8]`` int32, ``w1_scale`` / ``w2_scale`` = fp16 scales
    ``[E, K/128, N]``, ``w1_zp`` / ``w2_zp`` = qzeros ``[E, K/128, N/8]`` (K the
    reduction dim), fp16 activations; they are repacked once per tensor object.
    """
    logger.debug("FLAGGEMS_SGLANG FUSED_MOE")
    assert per_channel_quant is False, _UNSUPPORTED_FEATURE_MSG.format(name="per_channel_quant")
    assert expert_map is None, _UNSUPPORTED_FEATURE_MSG.format(name="expert_map")
    assert a1_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a1_scale")
    assert a2_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a2_scale")
    assert inplace is False, "Inplace is not supported"
    assert hidden_states.ndim == 2, "hidden_states must be 2D"
    if activation not in _ACTS:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")

    top_k = routing_data.n_expts_act
    routing = (routing_data.expt_hist, gather_indx.src_indx, routing_data.gate_scal, top_k)

    if use_int4_w4a16:
        assert group_size == 128, "only group_size 128 is supported"
        assert hidden_states.dtype == torch.float16, "int4 w4a16 takes fp16 activations"
        assert w1_scale is not None and w2_scale is not None and w1_zp is not None and w2_zp is not None, \
            "scales and zero points are required"
        p1, z1 = _awq_repacked(w1, w1_scale, w1_zp)
        p2, z2 = _awq_repacked(w2, w2_scale, w2_zp)
        return fused_experts(hidden_states, p1, p2, routing=routing, activation=activation,
                             apply_router_weight_on_input=apply_router_weight_on_input,
                             use_int4_w4a16=True, w13_sz=z1, w2_sz=z2)

    if use_fp8_w8a8:
        assert block_shape is not None and list(block_shape) == [128, 128], "block_shape must be [128, 128]"
        assert w1_scale is not None and w2_scale is not None, "w1_scale and w2_scale are required"
        return fused_experts(hidden_states, w1, w2, routing=routing, activation=activation,
                             apply_router_weight_on_input=apply_router_weight_on_input,
                             use_fp8_w8a8=True, w13_scale=w1_scale, w2_scale=w2_scale)

    assert w1_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="w1_scale")
    assert w2_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="w2_scale")
    assert block_shape is None, _UNSUPPORTED_FEATURE_MSG.format(name="block_shape")
    assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
    assert w1.dtype == torch.bfloat16, "w1 must be bfloat16"
    assert w2.dtype == torch.bfloat16, "w2 must be bfloat16"
    assert hidden_states.shape[-1] == w1.shape[-2], "hidden size mismatch"
    assert w2.shape[-1] == w1.shape[1], "intermediate size mismatch"

    out = fused_experts(hidden_states, _layer_layout(w1), _layer_layout(w2), routing=routing,
                        activation=activation, apply_router_weight_on_input=apply_router_weight_on_input)
    return out.view(hidden_states.shape[0], hidden_states.shape[1])


def _deinterleaved(w1: torch.Tensor, b1: torch.Tensor, layer_layout: bool = False):
    """The bias variant stores gate and linear outputs interleaved (even = gate, odd =
    linear; the dependency's swiglu splits them that way).  The kernels want the gate rows
    first and the linear rows after them: re-laid out once per weight tensor object.
    ``w1`` is ``[E, H, 2I]`` (op level) or, with ``layer_layout``, ``[E, 2I, H]``."""
    def make():
        rows = w1 if layer_layout else w1.transpose(1, 2)                                   # [E, 2I, H]
        w13 = torch.cat([rows[:, 0::2, :], rows[:, 1::2, :]], dim=1).contiguous()
        b13 = torch.cat([b1[:, 0::2], b1[:, 1::2]], dim=1).to(torch.float32).contiguous()   # [E, 2I]
        return w13, b13
    return _cached(w1, "split_ll" if layer_layout else "split_op", (b1._version, b1.data_ptr()), make)


def triton_kernel_fused_experts_with_bias(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w1_pcg,
    b1: torch.Tensor,
    w2: torch.Tensor,
    w2_pcg,
    b2: torch.Tensor,
    routing_data,
    gather_indx,
    scatter_indx,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    global_num_experts: int = -1,
    gemm1_alpha: Optional[float] = None,
    gemm1_clamp_limit: Optional[float] = None,
) -> torch.Tensor:
    """Bias variant of the op, same signature as the reference's
    (src/flaggems_sglang/ops/fused_moe.py:219-309): ``w1 [E, H, 2I]`` with gate and linear
    columns interleaved, ``b1 [E, 2I]`` likewise, ``w2 [E, I, H]``, ``b2 [E, H]``.
    GEMM-1 adds ``b1`` and applies ``s = g * sigmoid(alpha * g)``, ``s * (linear + 1)``
    (gate clamped to ``<= limit``, linear to ``[-limit, limit]``) in its epilogue; GEMM-2 adds
    ``b2`` before the routing weight.  ``w1_pcg`` / ``w2_pcg`` (the dependency's precision
    configs) must be None or plain bf16 configs: they carry nothing this path uses."""
    logger.debug("FLAGGEMS_SGLANG FUSED_MOE_WITH_BIAS")
    assert inplace is False, "Inplace is not supported"
    assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
    if activation != "silu":
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    assert w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16, "weights must be bfloat16"
    assert hidden_states.shape[-1] == w1.shape[-2], "hidden size mismatch"
    assert w2.shape[-1] == w1.shape[1], "intermediate size mismatch"
    w13, b13 = _deinterleaved(w1, b1)
    routing = (routing_data.expt_hist, gather_indx.src_indx, routing_data.gate_scal, routing_data.n_expts_act)
    out = fused_experts(hidden_states, w13, _layer_layout(w2), routing=routing, activation="swiglu_oai",
                        apply_router_weight_on_input=apply_router_weight_on_input, b13=b13, b2=b2,
                        swiglu_alpha=1.0 if gemm1_alpha is None else float(gemm1_alpha),
                        swiglu_limit=gemm1_clamp_limit)
    return out.view(hidden_states.shape[0], hidden_states.shape[1])


def fused_moe_flagos(obj, layer: torch.nn.Module, dispatch_output):
    """SGLang plugin hook (src/flaggems_sglang/ops/fused_moe.py:312-406).

    ``layer.w13_weight [E, 2I, H]`` and ``layer.w2_weight [E, H, I]`` are used
    where they lie (the reference transposes and copies both on every call), the
    top-k output goes straight to the device-side alignment, and the routed
    scaling factor is folded into the output conversion.
    """
    cfg = obj.runner.config
    hidden_states = dispatch_output.hidden_states
    topk_output = dispatch_output.topk_output
    no_combine = bool(getattr(cfg, "no_combine", False))
    b13 = getattr(layer, "w13_weight_bias", None)
    b2 = getattr(layer, "w2_weight_bias", None)
    has_bias = b13 is not None or b2 is not None
    if has_bias:
        assert b13 is not None and b2 is not None, "Bias execution requires both w13_bias and w2_bias"
    scale = getattr(cfg, "routed_scaling_factor", None)
    scale = 1.0 if scale is None else float(scale)
    common = dict(activation=cfg.activation,
                  apply_router_weight_on_input=bool(getattr(cfg, "apply_router_weight_on_input", False)),
                  routed_scaling_factor=scale, no_combine=no_combine)
    w13 = layer.w13_weight
    if has_bias:
        if cfg.activation != "silu":
            raise ValueError(f"Unsupported FusedMoe activation: {cfg.activation}")
        # biased layers keep gate and linear rows interleaved: split them once per weight object
        w13, b13 = _deinterleaved(layer.w13_weight, b13, layer_layout=True)
        alpha = getattr(cfg, "gemm1_alpha", None)
        common.update(activation="swiglu_oai", b13=b13, b2=b2, swiglu_alpha=1.0 if alpha is None else float(alpha),
                      swiglu_limit=getattr(cfg, "gemm1_clamp_limit", None))
    if hasattr(topk_output, "topk_weights"):
        out = fused_experts(hidden_states, w13, layer.w2_weight,
                            topk_output.topk_weights, topk_output.topk_ids, **common)
    else:
        routing_data, gather_indx, _ = topk_output
        routing = (routing_data.expt_hist, gather_indx.src_indx, routing_data.gate_scal, routing_data.n_expts_act)
        out = fused_experts(hidden_states, w13, layer.w2_weight, routing=routing, **common)
    try:
        from sglang.srt.layers.moe.token_dispatcher.standard import StandardCombineInput
        return StandardCombineInput(hidden_states=out)
    except Exception:
        return SimpleNamespace(hidden_states=out)


_standard_topk_to_triton_kernels = topk_to_routing
