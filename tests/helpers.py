"""Seeded inputs and comparison helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np

SEED0 = 0x4C4D4D4D


def fp16_inputs(seed, M, N, K):
    """A[M,K], B[K,N] fp32 drawn uniform[-1,1) (the FP16 GEMM configs)."""
    rng = np.random.default_rng(SEED0 + seed)
    return (rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (K, N)).astype(np.float32))


def fp8_sources(seed, M, N, K, w_std=1.0):
    """x[M,K] ~ N(0,1) activations and w[N,K] ~ N(0,w_std) weights, fp32."""
    rng = np.random.default_rng(SEED0 + seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * w_std).astype(np.float32)
    return x, w


def e4m3_ulp(v: np.ndarray) -> np.ndarray:
    """Spacing of e4m3 at |v| (v in e4m3 code units, i.e. after dividing by the scale)."""
    a = np.abs(v).astype(np.float64)
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -6)))
    e = np.clip(e, -6, 8)
    return 2.0 ** (e - 3)
