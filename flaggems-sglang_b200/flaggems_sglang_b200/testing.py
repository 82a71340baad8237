"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no real checkpoints are involved anywhere)."""
from __future__ import annotations

import math

import torch

# name -> (H, I, E, topk)
CONFIGS = {
    "tiny": (1024, 512, 8, 2),
    "mixtral": (4096, 14336, 8, 2),
    "qwen3-30b-a3b": (2048, 768, 128, 8),
    "deepseek-v3": (7168, 2048, 256, 8),
    "reference-bench": (1280, 3072, 64, 8),
}


def route(logits: torch.Tensor, topk: int):
    """softmax -> top-k -> renormalise, as in the reference's test
    (tests/test_fused_moe.py:21-27)."""
    w = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(w, k=topk, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def zipf_bias(n_experts: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """log of a Zipf(s) pmf laid over a seeded random permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_experts, generator=g)
    ranks = torch.arange(1, n_experts + 1, dtype=torch.float64)
    pmf = ranks.pow(-s)
    pmf = pmf / pmf.sum()
    bias = torch.empty(n_experts, dtype=torch.float32)
    bias[perm] = pmf.log().float()
    return bias


def make_weights(h: int, i: int, e: int, dtype=torch.bfloat16, device="cpu", scale=0.02, seed=0,
                 expert_ids=None):
    """Layer-layout weights w13 [E, 2I, H], w2 [E, H, I] ~ randn * scale, generated
    expert by expert on the target device.  With ``expert_ids`` only those experts
    are generated, each from its own seed, so that an expert-parallel shard holds
    the same values whatever the number of ranks."""
    if expert_ids is None:
        g = torch.Generator(device=device).manual_seed(seed)
        w13 = torch.empty(e, 2 * i, h, dtype=dtype, device=device)
        w2 = torch.empty(e, h, i, dtype=dtype, device=device)
        for ei in range(e):
            w13[ei] = (torch.randn(2 * i, h, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)
            w2[ei] = (torch.randn(h, i, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)
        return w13, w2
    ids = list(expert_ids)
    w13 = torch.empty(len(ids), 2 * i, h, dtype=dtype, device=device)
    w2 = torch.empty(len(ids), h, i, dtype=dtype, device=device)
    for j, ei in enumerate(ids):
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + ei + 1)
        w13[j] = (torch.randn(2 * i, h, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)
        w2[j] = (torch.randn(h, i, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)
    return w13, w2


def make_tokens(m: int, h: int, e: int, topk: int, dtype=torch.bfloat16, device="cpu", seed=0, skew=False,
                bias_seed=None):
    """Tokens and their routing.  ``skew``: the router's logits carry the layer's zipf bias, drawn from
    ``bias_seed`` (default: ``seed``) -- two batches with different ``seed`` and the same ``bias_seed``
    are different traffic through the same layer."""
    g = torch.Generator(device=device).manual_seed(seed + 1)
    x = torch.randn(m, h, generator=g, device=device, dtype=torch.float32).to(dtype)
    logits = torch.randn(m, e, generator=g, device=device, dtype=torch.float32)
    if skew:
        logits = logits + zipf_bias(e, 1.1, seed if bias_seed is None else bias_seed).to(device)
    w, ids = route(logits, topk)
    return x, w, ids
