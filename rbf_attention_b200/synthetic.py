"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations."""

from __future__ import annotations

import torch


def make_inputs(B, H, N, D, *, seed=0, dtype=torch.bfloat16, std=1.0, key_norm_sigma=0.0):
    """Q, K, V ~ N(0, std^2), dO ~ N(0, 1) on the CPU from one seeded generator. With ``key_norm_sigma`` > 0
    every key row is scaled by one LogNormal(0, sigma) draw, so that a few keys have outlier norms.
    Returns (q, k, v, dout) rounded to ``dtype``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, H, N, D, generator=g) * std
    k = torch.randn(B, H, N, D, generator=g) * std
    v = torch.randn(B, H, N, D, generator=g) * std
    do = torch.randn(B, H, N, D, generator=g)
    if key_norm_sigma > 0:
        k = k * torch.exp(torch.randn(B, H, N, 1, generator=g) * key_norm_sigma)
    return tuple(t.to(dtype) for t in (q, k, v, do))
