"""Helpers shared by the GPU parity tests."""
import numpy as np


def rel_err(y, want):
    """max_i |y_i - want_i| / max(|want_i|, rms(want)): relative error with an rms floor, so that
    outputs that happen to lie near zero do not turn rounding noise into a huge ratio."""
    y = np.asarray(y, np.float64)
    want = np.asarray(want, np.float64)
    floor = float(np.sqrt(np.mean(want ** 2))) if want.size else 1.0
    if floor == 0.0:
        floor = 1.0
    return float(np.max(np.abs(y - want) / np.maximum(np.abs(want), floor))) if want.size else 0.0


def norm_err(y, want):
    """Normwise relative error: max |y - want| / max |want|."""
    y = np.asarray(y, np.float64)
    want = np.asarray(want, np.float64)
    d = float(np.max(np.abs(want))) if want.size else 1.0
    return float(np.max(np.abs(y - want))) / (d if d else 1.0) if want.size else 0.0


def bf16_round(a):
    """round-to-nearest-even to bfloat16, returned as float32 (numpy has no bf16)."""
    a = np.ascontiguousarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(a.shape)


TOL_FP32 = 1e-3   # fp32-dequant paths (SIMT, decode)
TOL_BF16 = 2e-2   # bf16 / int8 tensor-core paths
