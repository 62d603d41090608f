"""Seeded synthetic K/V/Q with the distributions the benchmark configurations name.

K and V entries ~ N(0,1); K channels are scaled per channel by exp(N(0, 0.5)) to mimic outlier channels;
queries ~ N(0,1); everything is cast to fp16.  These tensors stand in for real rollouts (no model
weights or datasets are available offline).
"""
from __future__ import annotations

import numpy as np


def channel_scales(kv_dim: int, seed: int = 0) -> np.ndarray:
    return np.exp(np.random.default_rng(seed + 7919).normal(0.0, 0.5, kv_dim)).astype(np.float32)


def kv_batch(rng: np.random.Generator, n: int, kv_dim: int, scales: np.ndarray):
    """(k, v) fp16 arrays [n, kv_dim]."""
    k = (rng.standard_normal((n, kv_dim), dtype=np.float32) * scales).astype(np.float16)
    v = rng.standard_normal((n, kv_dim), dtype=np.float32).astype(np.float16)
    return k, v


def q_batch(rng: np.random.Generator, n: int, q_dim: int) -> np.ndarray:
    return rng.standard_normal((n, q_dim), dtype=np.float32).astype(np.float16)


def torch_kv(gen, n: int, kv_dim: int, scales_t, device="cuda"):
    """Same distributions generated on the device (large benchmark caches)."""
    import torch
    k = (torch.randn(n, kv_dim, generator=gen, device=device) * scales_t).to(torch.float16)
    v = torch.randn(n, kv_dim, generator=gen, device=device).to(torch.float16)
    return k, v
