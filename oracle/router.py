"""CPU restatement of the router front-end (TEST INFRASTRUCTURE: only tests, the smoke
check and the benchmark's CPU baseline may import this).

Softmax / top-k / renormalise follows the recipe the reference's own test uses to make its
routing (tests/test_fused_moe.py:21-27).  Group-limited selection restates the published
DeepSeek-V2 / -V3 gating rule (no reference source: parity unpinned for that mode; it is
checked against a direct torch formulation in the CPU tests).  fp32 arithmetic throughout;
ties go to the lower expert id.
"""
from __future__ import annotations

import numpy as np


def _topk_stable(keys: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest per row, larger first, lower index on ties."""
    order = np.argsort(-keys, axis=1, kind="stable")
    return order[:, :k]


def route_topk(logits, topk: int, renormalize: bool = True, scoring: str = "softmax", n_group: int = 0,
               topk_group: int = 0, bias=None, scale: float = 1.0):
    """logits [M, E] (array-like, any float dtype) -> (weights fp32 [M, topk], ids int32 [M, topk])."""
    l = np.asarray(logits, dtype=np.float32)
    m, e = l.shape
    if scoring == "softmax":
        mx = l.max(axis=1, keepdims=True)
        num = np.exp(l - mx, dtype=np.float32)
        den = num.sum(axis=1, keepdims=True, dtype=np.float32)
        scores = (num / den).astype(np.float32)
        keys = l.copy() if bias is None else scores + np.asarray(bias, dtype=np.float32)[None, :]
    elif scoring == "sigmoid":
        scores = (np.float32(1.0) / (np.float32(1.0) + np.exp(-l, dtype=np.float32))).astype(np.float32)
        keys = scores.copy() if bias is None else scores + np.asarray(bias, dtype=np.float32)[None, :]
    else:
        raise ValueError(f"Unsupported scoring function: {scoring}")
    if n_group and n_group > 1:
        g = e // n_group
        kg = keys.reshape(m, n_group, g)
        if bias is not None and g > 1:
            top2 = -np.sort(-kg, axis=2)[:, :, :2]
            gscore = (top2[:, :, 0] + top2[:, :, 1]).astype(np.float32)
        else:
            gscore = kg.max(axis=2)
        keep = _topk_stable(gscore, topk_group)
        mask = np.zeros((m, n_group), dtype=bool)
        np.put_along_axis(mask, keep, True, axis=1)
        keys = np.where(np.repeat(mask, g, axis=1), keys, -np.inf).astype(np.float32)
    ids = _topk_stable(keys, topk)
    w = np.take_along_axis(scores, ids, axis=1).astype(np.float32)
    if renormalize:
        w = (w / w.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    w = (w * np.float32(scale)).astype(np.float32)
    return w, ids.astype(np.int32)
