"""``flaggems_sglang.testing`` (reference: src/flaggems_sglang/testing/__init__.py:60-78): the
two comparison helpers the reference's tests import, with its per-dtype relative tolerances."""
import torch

RESOLUTION = {
    torch.bool: 0, torch.uint8: 0, torch.int8: 0, torch.int16: 0, torch.int32: 0, torch.int64: 0,
    torch.float8_e4m3fn: 1e-3, torch.float8_e5m2: 1e-3,
    torch.float16: 1e-3, torch.bfloat16: 0.016, torch.float32: 1.3e-6, torch.float64: 1e-7,
}


def assert_close(res, ref, dtype, equal_nan=False, reduce_dim=1, atol=1e-4):
    """``res`` must have ``dtype`` and match ``ref`` within that type's relative tolerance and
    ``atol * reduce_dim``."""
    dtype = torch.float32 if dtype is None else dtype
    assert res.dtype == dtype
    torch.testing.assert_close(res.cpu(), ref.to(dtype).cpu(), atol=atol * reduce_dim, rtol=RESOLUTION[dtype],
                               equal_nan=equal_nan)


def assert_equal(res, ref, equal_nan=False):
    torch.testing.assert_close(res, ref, atol=0, rtol=0, equal_nan=equal_nan)
