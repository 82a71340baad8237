"""CPU: the router restatement against the recipe the reference's test uses for its routing
(tests/test_fused_moe.py:21-27) and against a direct torch formulation of group-limited
selection; argument errors of the C entry point (no GPU work is launched)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.router import route_topk


@pytest.mark.parametrize("m,e,k", [(1, 8, 2), (7, 8, 2), (33, 16, 4), (64, 64, 8), (257, 128, 8), (100, 60, 6)])
def test_softmax_topk_matches_reference_recipe(m, e, k):
    torch.manual_seed(m + e + k)
    logits = torch.randn(m, e, dtype=torch.float32)
    tw = torch.softmax(logits, dim=-1)
    tw, ids = torch.topk(tw, k=k, dim=-1)
    tw = tw / tw.sum(dim=-1, keepdim=True)
    w, i = route_topk(logits.numpy(), k, renormalize=True)
    assert np.array_equal(i, ids.numpy().astype(np.int32))
    np.testing.assert_allclose(w, tw.numpy(), rtol=2e-6, atol=1e-8)
    w2, _ = route_topk(logits.numpy(), k, renormalize=False)
    np.testing.assert_allclose(w2, torch.softmax(logits, -1).gather(1, ids).numpy(), rtol=2e-6, atol=1e-8)


def test_ties_go_to_the_lower_expert():
    logits = np.zeros((3, 16), dtype=np.float32)
    logits[1, 5] = logits[1, 9] = 2.0
    w, i = route_topk(logits, 3)
    assert i[0].tolist() == [0, 1, 2] and i[1].tolist() == [5, 9, 0]
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)


@pytest.mark.parametrize("biased", [False, True])
def test_grouped_selection_matches_direct_formulation(biased):
    torch.manual_seed(3)
    m, e, g, kg, k = 150, 256, 8, 4, 8
    logits = torch.randn(m, e)
    bias = torch.randn(e) * 0.1 if biased else None
    scores = torch.sigmoid(logits) if biased else torch.softmax(logits, -1)
    choice = scores + bias if biased else scores
    grouped = choice.view(m, g, -1)
    gscore = grouped.topk(2, -1)[0].sum(-1) if biased else grouped.max(-1)[0]
    gi = gscore.topk(kg, -1)[1]
    mask = torch.zeros(m, g).scatter_(1, gi, 1).bool().repeat_interleave(e // g, 1)
    ids = choice.masked_fill(~mask, float("-inf")).topk(k, -1)[1]
    tw = scores.gather(1, ids)
    tw = tw / tw.sum(-1, keepdim=True) * 2.5
    w, i = route_topk(logits.numpy(), k, True, "sigmoid" if biased else "softmax", g, kg,
                      bias.numpy() if biased else None, 2.5)
    assert np.array_equal(i, ids.numpy().astype(np.int32))
    np.testing.assert_allclose(w, tw.numpy(), rtol=3e-6, atol=1e-8)


def test_router_argument_errors(built_lib):
    from flaggems_sglang_b200 import _lib
    lib = _lib.lib()

    def call(e=64, k=4, **kw):
        f = dict(struct_bytes=C.sizeof(_lib.Router), scoring=0, renormalize=1, n_group=0, topk_group=0,
                 logits_dtype=_lib.DTYPE_FP32, scale=1.0, reserved=0, bias=None)
        f.update(kw)
        r = _lib.Router(*[f[n] for n, _ in _lib.Router._fields_])
        return lib.b200moe_route_topk(C.byref(r), None, 0, e, k, None, None, None)

    assert call() == _lib.OK                                  # zero tokens: nothing to do
    assert call(struct_bytes=8) == _lib.ERR_BAD_ARG
    assert call(scoring=7) == _lib.ERR_BAD_ARG
    assert call(k=65) == _lib.ERR_BAD_ARG
    assert call(k=33) == _lib.ERR_TOO_LARGE
    assert call(e=2048) == _lib.ERR_TOO_LARGE
    assert call(n_group=7, topk_group=2) == _lib.ERR_UNSUPPORTED      # 64 % 7 != 0
    assert call(n_group=8, topk_group=9) == _lib.ERR_BAD_ARG
    assert call(n_group=8, topk_group=1, k=9) == _lib.ERR_BAD_ARG     # one group holds 8 experts
    assert lib.b200moe_route_topk(None, None, 0, 8, 2, None, None, None) == _lib.ERR_BAD_ARG
