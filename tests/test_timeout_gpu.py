"""GPU: the device-side time-out path, driven to its end without faulting anything.

Every wait inside the kernels is bounded; in a healthy run none runs out.  The library's
self-test kernel makes one run out on purpose -- a warp waits ~1 ms on a barrier nobody arrives
on -- and this test follows the consequence through the same plumbing a real time-out would
use: the status word, ``check_status()`` raising, and the next ordinary call working."""
import ctypes as C

import pytest
import torch

from oracle import moe as OM
from parity import assert_parity

pytestmark = pytest.mark.gpu


def test_wait_runs_out_sets_status_and_context_survives(cuda_device):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.ops.fused_moe import _status_word
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    lib = _lib.lib()
    d = cuda_device
    torch.cuda.set_device(d)
    F.check_status()                                           # clean slate
    status = _status_word(d)                                   # the word the operators report into
    observed = torch.full((3,), -1, dtype=torch.int32, device=d)
    limit_ns = 1_000_000                                       # 1 ms
    rc = lib.b200moe_selftest_timeout(limit_ns, status.data_ptr(), observed.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.OK
    torch.cuda.synchronize()                                   # the kernel returned by itself
    short_ok, long_ok, waited_us = observed.tolist()
    assert short_ok == 0, "the 1 ms wait did not run out"
    assert long_ok == 0, "the sibling wait was not released by the abort flag"
    assert 500 <= waited_us < 100_000, f"sibling waited {waited_us} us: released by its own clock, not by the flag?"
    assert int(status.item()) == 105
    with pytest.raises(RuntimeError, match="timed out"):
        F.check_status()
    F.check_status()                                           # the word was cleared by the raise

    # the context is intact: an ordinary call right after gives the right answer
    h, i, e, k, m = 512, 256, 8, 2, 40
    w13, w2 = make_weights(h, i, e, seed=1, scale=0.05)
    x, tw, ids = make_tokens(m, h, e, k, seed=1)
    out = F.fused_experts(x.to(d), w13.to(d), w2.to(d), tw.to(d), ids.to(d))
    F.check_status()
    assert_parity(out, OM.fused_experts(x, w13, w2, tw, ids), what="call after a provoked time-out")


def test_timeout_surfaces_without_anyone_calling_check_status(cuda_device):
    """A serving host never calls check_status(): the operator itself notices, a few calls later
    and without synchronising, through the host copy of the status word."""
    import importlib
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib
    fm = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    lib = _lib.lib()
    d = cuda_device
    torch.cuda.set_device(d)
    F.check_status()
    h, i, e, k, m = 512, 256, 8, 2, 40
    w13, w2 = make_weights(h, i, e, seed=1, scale=0.05)
    x, tw, ids = make_tokens(m, h, e, k, seed=1)
    args = (x.to(d), w13.to(d), w2.to(d), tw.to(d), ids.to(d))
    F.fused_experts(*args)                                     # makes sure the host copy exists
    observed = torch.zeros(3, dtype=torch.int32, device=d)
    assert lib.b200moe_selftest_timeout(1_000_000, fm._status_word(d).data_ptr(), observed.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream) == _lib.OK
    raised = 0
    for _ in range(2 * fm.STATUS_COPY_EVERY + 2):
        try:
            F.fused_experts(*args)
        except RuntimeError as ex:
            assert "timed out" in str(ex)
            raised += 1
        torch.cuda.synchronize()
    assert raised == 1, f"the provoked time-out surfaced {raised} times"
    out = F.fused_experts(*args)
    F.check_status()
    assert_parity(out, OM.fused_experts(x, w13, w2, tw, ids), what="after the deferred status report")


def test_selftest_argument_checks(cuda_device):
    from flaggems_sglang_b200 import _lib
    lib = _lib.lib()
    buf = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    assert lib.b200moe_selftest_timeout(0, buf.data_ptr(), buf.data_ptr(), None) == _lib.ERR_BAD_ARG
    assert lib.b200moe_selftest_timeout(10**10, buf.data_ptr(), buf.data_ptr(), None) == _lib.ERR_BAD_ARG
    assert lib.b200moe_selftest_timeout(1000, None, buf.data_ptr(), None) == _lib.ERR_BAD_ARG
