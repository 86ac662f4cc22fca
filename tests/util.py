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


def block_fixed_point(x, block=32):
    """What the decode kernels make of fp32 activations x[M, K], as float64: every `block` consecutive k
    of a row (32 for INT4 weights, 128 for INT8) share one scale gmax / Q, Q = 8355000 (24 bits: three
    int8 digits); values are rounded to the nearest multiple of it.  In batches of three rows or more the
    lowest digit is dropped (rounding to the nearest multiple of 256 scale units) except in blocks that
    one value dominates, gmax > 4 rms(block).  All steps in fp32 as on the device: P = Q / gmax,
    q = rint(x * P), scale = gmax / Q."""
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    Q = np.float32(8355000.0)
    out = np.zeros((M, K), np.float64)
    for b0 in range(0, K, block):
        blk = x[:, b0:b0 + block]
        gmax = np.max(np.abs(blk), axis=1, keepdims=True).astype(np.float32)
        ok = gmax >= np.float32(1e-30)
        safe = np.where(ok, gmax, np.float32(1.0))
        P = (Q / safe).astype(np.float32)
        sx = (safe / Q).astype(np.float32)
        q = np.rint((blk * P).astype(np.float32)).astype(np.float64)
        if M >= 3:
            keep_low = (q ** 2).sum(axis=1, keepdims=True) < 2.0 * (block // 32) * float(Q) ** 2
            q = np.where(keep_low, q, np.floor((q + 128.0) / 256.0) * 256.0)     # balanced digits: the low one lies in [-128, 127]
        out[:, b0:b0 + block] = np.where(ok, q * sx.astype(np.float64), 0.0)
    return out


def heavy_tailed_rows(seed, M, K, factor, channels):
    """N(0,1) activation rows in which `channels` positions (the same for every row, as the outlier
    channels of a normalised decoder activation are) are multiplied by `factor`."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    idx = rng.choice(K, size=channels, replace=False)
    x[:, idx] *= np.float32(factor)
    return x
