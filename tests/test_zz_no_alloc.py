"""GPU: the allocation-free forward entry point against the regular one.

`b200moe_forward_topk_noalloc` serves callers that cannot pass a workspace and may
not allocate one (a runtime whose pools own all device memory, a plugin slot with
no scratch argument, a thread barred from the CUDA allocator): its scratch is an
array inside the library image.  Both entry points are driven here directly
through the C ABI on the same inputs, twice in a row, because the second call
finds the first call's leftovers in the shared array and must not be disturbed
by them.  The file name sorts last so that a run that stops at the first failure
has already covered everything else.
"""
import ctypes as C

import pytest
import torch

from parity import assert_parity

pytestmark = pytest.mark.gpu


def _cfg(_lib, m, h, i, e, k):
    flags = _lib.FLAG_MIMIC_ROUNDING
    return _lib.Cfg(C.sizeof(_lib.Cfg), m, h, i, e, k, _lib.DTYPE_BF16, _lib.W_16BIT, _lib.LAYOUT_LAYER,
                    _lib.ACT_SILU, flags, 0, 1.0, 0)


def _forward_regular(lib, _lib, cfg, x, w13, w2, tw, ids, status):
    nbytes = lib.b200moe_workspace_bytes(C.byref(cfg))
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=x.device)
    base = (ws.data_ptr() + 255) & ~255
    out = torch.empty_like(x)
    rc = lib.b200moe_forward_topk(C.byref(cfg), x.data_ptr(), w13.data_ptr(), w2.data_ptr(), None, tw.data_ptr(),
                                  ids.data_ptr(), None, base, nbytes, out.data_ptr(), status.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.OK, _lib.status_string(rc)
    torch.cuda.synchronize()
    return out


def _forward_noalloc(lib, _lib, cfg, x, w13, w2, tw, ids, status):
    out = torch.empty_like(x)
    rc = lib.b200moe_forward_topk_noalloc(C.byref(cfg), x.data_ptr(), w13.data_ptr(), w2.data_ptr(), None,
                                          tw.data_ptr(), ids.data_ptr(), None, out.data_ptr(), status.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.OK, _lib.status_string(rc)
    torch.cuda.synchronize()
    return out


def test_noalloc_matches_regular_entry_point_twice(cuda_device):
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    lib = _lib.lib()
    torch.cuda.set_device(cuda_device)
    h, i, e, k = 1024, 512, 8, 2
    w13, w2 = make_weights(h, i, e, device=cuda_device, seed=0)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    # two different batches back to back: the second runs on the first one's leftovers
    for call, (m, seed) in enumerate([(48, 0), (17, 1)]):
        x, tw, ids = make_tokens(m, h, e, k, device=cuda_device, seed=seed)
        cfg = _cfg(_lib, m, h, i, e, k)
        assert lib.b200moe_workspace_bytes(C.byref(cfg)) <= _lib.NOALLOC_SCRATCH_BYTES
        ref = _forward_regular(lib, _lib, cfg, x, w13, w2, tw, ids, status)
        got = _forward_noalloc(lib, _lib, cfg, x, w13, w2, tw, ids, status)
        assert_parity(got, ref, what=f"noalloc call {call}")
        assert int(status.item()) == 0
    # and once more with the first batch: identical to its first result
    x, tw, ids = make_tokens(48, h, e, k, device=cuda_device, seed=0)
    cfg = _cfg(_lib, 48, h, i, e, k)
    again = _forward_noalloc(lib, _lib, cfg, x, w13, w2, tw, ids, status)
    assert_parity(again, _forward_regular(lib, _lib, cfg, x, w13, w2, tw, ids, status), what="noalloc repeat")


def test_noalloc_against_the_oracle_and_at_the_size_limit(cuda_device):
    """Directly against the CPU oracle, at the largest token count whose scratch still fits the
    array (one token more must be refused)."""
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    from oracle import moe as OM
    lib = _lib.lib()
    torch.cuda.set_device(cuda_device)
    h, i, e, k = 1024, 512, 8, 2
    fits = lambda m: 0 < lib.b200moe_workspace_bytes(C.byref(_cfg(_lib, m, h, i, e, k))) <= _lib.NOALLOC_SCRATCH_BYTES
    lo, hi = 1, 1 << 16
    assert fits(lo) and not fits(hi)
    while hi - lo > 1:
        mid = (lo + hi) // 2
        lo, hi = (mid, hi) if fits(mid) else (lo, mid)
    m = lo                                                   # fits; m + 1 does not
    w13, w2 = make_weights(h, i, e, seed=0)
    x, tw, ids = make_tokens(m, h, e, k, seed=3)
    d = cuda_device
    status = torch.zeros(1, dtype=torch.int32, device=d)
    got = _forward_noalloc(lib, _lib, _cfg(_lib, m, h, i, e, k), x.to(d), w13.to(d), w2.to(d), tw.to(d), ids.to(d), status)
    assert int(status.item()) == 0
    assert_parity(got, OM.fused_experts(x, w13, w2, tw, ids), what=f"noalloc vs oracle, M={m} (largest that fits)")
    dummy = torch.zeros(64, dtype=torch.int32, device=d)
    rc = lib.b200moe_forward_topk_noalloc(C.byref(_cfg(_lib, m + 1, h, i, e, k)), dummy.data_ptr(), dummy.data_ptr(),
                                          dummy.data_ptr(), None, dummy.data_ptr(), dummy.data_ptr(), None,
                                          dummy.data_ptr(), dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_TOO_LARGE


def test_noalloc_fp8_decode_uses_the_scale_regions(cuda_device):
    """A decode-sized FP8 call: its layout adds the activation-scale tables to the shared array."""
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    from oracle import moe as OM
    lib = _lib.lib()
    torch.cuda.set_device(cuda_device)
    h, i, e, k, m = 1024, 512, 8, 2, 24
    w13, w2 = make_weights(h, i, e, seed=2)
    w13q, s13 = quantize_fp8_block(w13)
    w2q, s2 = quantize_fp8_block(w2)
    d = cuda_device
    dw13, ds13, dw2, ds2 = (t.to(d) for t in (w13q, s13, w2q, s2))
    cfg = _lib.Cfg(C.sizeof(_lib.Cfg), m, h, i, e, k, _lib.DTYPE_BF16, _lib.W_FP8_BLOCK, _lib.LAYOUT_LAYER,
                   _lib.ACT_SILU, 0, 0, 1.0, 0)
    quant = _lib.Quant(ds13.data_ptr(), ds2.data_ptr(), None, None)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    for seed in (5, 6):                                      # twice in a row on the shared array
        x, tw, ids = make_tokens(m, h, e, k, seed=seed)
        dx, dtw, dids = x.to(d), tw.to(d), ids.to(d)
        out = torch.empty_like(dx)
        rc = lib.b200moe_forward_topk_noalloc(C.byref(cfg), dx.data_ptr(), dw13.data_ptr(), dw2.data_ptr(),
                                              C.byref(quant), dtw.data_ptr(), dids.data_ptr(), None, out.data_ptr(),
                                              status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == _lib.OK, _lib.status_string(rc)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_parity(out, OM.fused_experts_fp8(x, w13q, w2q, s13, s2, tw, ids), what=f"noalloc fp8 seed {seed}")


def test_noalloc_rejects_problems_beyond_the_array(cuda_device):
    from flaggems_sglang_b200 import _lib
    lib = _lib.lib()
    torch.cuda.set_device(cuda_device)
    cfg = _cfg(_lib, 4096, 4096, 14336, 8, 2)      # hundreds of MB of scratch
    assert lib.b200moe_workspace_bytes(C.byref(cfg)) > _lib.NOALLOC_SCRATCH_BYTES
    dummy = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    rc = lib.b200moe_forward_topk_noalloc(C.byref(cfg), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None,
                                          dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(),
                                          dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_TOO_LARGE
    assert "too large" in _lib.status_string(rc)
