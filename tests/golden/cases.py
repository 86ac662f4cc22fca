"""Seeded inputs shared by the fixture generator and the tests.

Every array comes from numpy's PCG64 (``default_rng(seed)``), whose stream is stable across
numpy versions, so the generator run in the authoring container and the tests run elsewhere
see the same bits; small cases also store their inputs inside the fixture itself.
"""
from __future__ import annotations

import numpy as np

LAYOUT_KN, LAYOUT_NK = 0, 1
PER_TENSOR, PER_ROW = 0, 1


def normal(seed: int, shape, std: float = 1.0) -> np.ndarray:
    return (np.random.default_rng(seed).standard_normal(shape) * std).astype(np.float32)


def weight_with_outliers(seed: int, shape, std: float = 0.02, frac: float = 0.01, mult: float = 20.0) -> np.ndarray:
    """N(0, std) with a Bernoulli(frac) mask of entries multiplied by `mult`."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(shape) * std).astype(np.float32)
    mask = rng.random(shape) < frac
    w[mask] *= np.float32(mult)
    return w


def special_values() -> np.ndarray:
    """Ties at .5 after scaling, an all-zero group, denormals, a single huge outlier,
    NaN and +-Inf (their quantized values are fixed by the reference's min/max ordering)."""
    return np.array(
        [2.5, -2.5, 0.5, -0.5, 7.0, -7.0, 3.5, 1.5,
         0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0,
         1e-40, -1e-40, 1e-30, -3e-39, 1e-8, -1e-8, 9.9e-9, 2e-8,
         1e4, 1.0, -1.0, 0.25, -0.75, 0.125, 3.0, -2.0,
         np.nan, 1.0, -1.0, 0.5, np.inf, 1.0, -2.0, 3.0,
         -np.inf, np.nan, 1.0, 0.0, 1.0, 2.0, 3.0, 4.0, 5.0],
        dtype=np.float32)


# (name, shape, generator)
QUANT_CASES = [
    ("suite_randn_16x32", (16, 32), lambda: normal(11, (16, 32))),            # src/test_suite.cpp:677
    ("ragged_3x20", (3, 20), lambda: normal(12, (3, 20), 0.02)),              # groups straddle rows, short tail
    ("odd_7x33", (7, 33), lambda: weight_with_outliers(13, (7, 33))),
    ("vec_5", (5,), lambda: normal(14, (5,))),                                # rank 1 -> per-tensor branch
    ("single", (1, 1), lambda: np.array([[0.3]], np.float32)),
    ("special", (49,), special_values),
    ("special_7x7", (7, 7), lambda: special_values().reshape(7, 7)),
    ("outliers_64x256", (64, 256), lambda: weight_with_outliers(15, (64, 256))),
    ("rank3_4x6x10", (4, 6, 10), lambda: normal(16, (4, 6, 10), 0.5)),
]
INT4_GROUPS = [32, 16, 7, 0, 64, 128]

# (name, M, K, N)
FORWARD_CASES = [
    ("suite_linear_32_16", 4, 32, 16),   # src/test_suite.cpp:707-725
    ("gemv_1", 1, 256, 96),
    ("gemv_4", 4, 512, 160),
    ("gemv_16", 16, 384, 64),
    ("tails_17", 17, 130, 70),
    ("tile_40", 40, 160, 72),
    ("prefill_136", 136, 192, 128),
]


# (name, M, K, N): gradient with respect to x of a frozen quantized layer
BACKWARD_CASES = [
    ("bw_decode_1", 1, 256, 96),
    ("bw_decode_4", 4, 512, 160),
    ("bw_tails_17", 17, 130, 72),
    ("bw_tile_40", 40, 160, 64),
]


def backward_seed(name: str, M: int, N: int) -> np.ndarray:
    """The upstream gradient dy[M, N] of a backward case."""
    return normal(sum(ord(c) for c in name) * 11 + 3, (M, N))


def forward_inputs(name: str, M: int, K: int, N: int, layout: int):
    seed = sum(ord(c) for c in name) * 7 + layout
    x = normal(seed, (M, K))
    w = weight_with_outliers(seed + 1, (K, N) if layout == LAYOUT_KN else (N, K))
    b = normal(seed + 2, (N,), 0.1)
    return x, w, b


def config1_inputs():
    """benchmark configuration 1: X[128,1024]~N(0,1), W[1024,1024]~N(0,0.02), bias zeros, seed 0."""
    return normal(0, (128, 1024)), normal(1, (1024, 1024), 0.02), np.zeros(1024, np.float32)
