"""TEST INFRASTRUCTURE — numpy/ctypes front end of the two checkers.

* ``port``  : oracle/libsgq_oracle.so, the plain-C restatement (oracle/sgq_oracle.c).
* ``ref``   : oracle/_ref/libsgref.so, the unmodified reference sources compiled by
              ``make -C oracle ref`` (None when that library was not built).

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline legs of bench.py may import
this package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LAYOUT_KN, LAYOUT_NK = 0, 1
PER_TENSOR, PER_ROW = 0, 1

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64 = C.c_int64


def build_port() -> str:
    """Compile the C restatement if its .so is missing or older than its source."""
    so = os.path.join(_HERE, "libsgq_oracle.so")
    src = [os.path.join(_HERE, n) for n in ("sgq_oracle.c", "sgq_oracle.h")]
    if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "port"])
    return so


def build_ref(reference_dir: str | None = None) -> str | None:
    """Compile the unmodified reference when its sources are reachable (reference_dir, else the
    environment variable SGQ_REFERENCE_DIR, else a sibling directory `reference` of this
    repository); else keep what exists."""
    so = os.path.join(_HERE, "_ref", "libsgref.so")
    if reference_dir is None:
        reference_dir = os.environ.get("SGQ_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference"))
    if os.path.isdir(os.path.join(reference_dir, "src")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={reference_dir}"])
    return so if os.path.exists(so) else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Port:
    """The C restatement."""

    def __init__(self):
        L = C.CDLL(build_port())
        L.sgqo_quantize_int8_tensor.argtypes = [_f32p, _i64, _i8p, _f32p]
        L.sgqo_quantize_int8_rows.argtypes = [_f32p, _i64, _i64, _i8p, _f32p]
        L.sgqo_quantize_int4.argtypes = [_f32p, _i64, _i64, _u8p, _f32p]
        L.sgqo_pack_int4_codes.argtypes = [_f32p, _i64, _u8p]
        L.sgqo_unpack_int4_codes.argtypes = [_u8p, _i64, _f32p]
        L.sgqo_pack_int8_codes.argtypes = [_f32p, _i64, _i8p]
        L.sgqo_unpack_int8_codes.argtypes = [_i8p, _i64, _f32p]
        L.sgqo_dequantize_int8.argtypes = [_i8p, _f32p, _i64, _i64, C.c_int, _f32p]
        L.sgqo_dequantize_int4.argtypes = [_u8p, _f32p, _i64, _i64, _f32p]
        L.sgqo_linear_f32.argtypes = [_f32p, _i64, _i64, _i64, _f32p, C.c_int, C.c_void_p, _f32p]
        L.sgqo_linear_f64.argtypes = [_f32p, _i64, _i64, _i64, _f32p, C.c_int, C.c_void_p, _f64p]
        L.sgqo_qlinear_int4.argtypes = [_f32p, _i64, _i64, _i64, _u8p, _f32p, C.c_int, _i64, C.c_void_p, _f32p]
        L.sgqo_qlinear_int8.argtypes = [_f32p, _i64, _i64, _i64, _i8p, _f32p, C.c_int, C.c_int, C.c_void_p, _f32p]
        L.sgqo_igemm_s8.argtypes = [_i8p, _i8p, _i64, _i64, _i64, C.c_int, _i32p]
        L.sgqo_qlinear_w8a8.argtypes = [_f32p, _i64, _i64, _i64, _i8p, _f32p, C.c_int, C.c_int, C.c_void_p,
                                        _i8p, _f32p, _i32p, _f32p]
        for name in dir(L):
            pass
        self.L = L

    @staticmethod
    def _bias(bias):
        if bias is None:
            return None, None
        b = _f32(bias).reshape(-1)
        return b, b.ctypes.data_as(C.c_void_p)

    # -- quantizers -------------------------------------------------------------------
    def quantize_int8(self, x, scheme=PER_ROW):
        x = _f32(x)
        codes = np.empty(x.shape, np.int8)
        if scheme == PER_TENSOR or x.ndim < 2:  # src/quantization.cpp:22
            scale = np.empty(1, np.float32)
            self.L.sgqo_quantize_int8_tensor(x.reshape(-1), x.size, codes.reshape(-1), scale)
            return codes, scale
        rows = x.shape[0]
        scales = np.empty(rows, np.float32)
        self.L.sgqo_quantize_int8_rows(x.reshape(-1), rows, x.size // max(rows, 1), codes.reshape(-1), scales)
        return codes, scales

    def quantize_int4(self, x, group=32):
        x = _f32(x)
        g = 32 if group <= 0 else group
        packed = np.zeros((x.size + 1) // 2, np.uint8)
        scales = np.empty((x.size + g - 1) // g, np.float32)
        self.L.sgqo_quantize_int4(x.reshape(-1), x.size, group, packed, scales)
        return packed, scales

    def pack_int4_codes(self, codes_f32):
        c = _f32(codes_f32).reshape(-1)
        out = np.zeros((c.size + 1) // 2, np.uint8)
        self.L.sgqo_pack_int4_codes(c, c.size, out)
        return out

    def unpack_int4_codes(self, packed, n):
        out = np.empty(n, np.float32)
        self.L.sgqo_unpack_int4_codes(np.ascontiguousarray(packed, np.uint8), n, out)
        return out

    def dequantize_int8(self, codes, scales, scheme):
        codes = np.ascontiguousarray(codes, np.int8)
        rows = codes.shape[0] if codes.ndim >= 2 else 1
        out = np.empty(codes.shape, np.float32)
        sch = PER_TENSOR if (scheme == PER_TENSOR or np.size(scales) == 1) else PER_ROW
        self.L.sgqo_dequantize_int8(codes.reshape(-1), _f32(scales), rows, codes.size // max(rows, 1), sch,
                                    out.reshape(-1))
        return out

    def dequantize_int4(self, packed, scales, shape, group=32):
        n = int(np.prod(shape))
        out = np.empty(n, np.float32)
        self.L.sgqo_dequantize_int4(np.ascontiguousarray(packed, np.uint8), _f32(scales), n, group, out)
        return out.reshape(shape)

    # -- forward ----------------------------------------------------------------------
    def linear_f32(self, x, w, layout, bias=None):
        x, w = _f32(x), _f32(w)
        M, K = x.shape
        N = w.shape[1] if layout == LAYOUT_KN else w.shape[0]
        y = np.empty((M, N), np.float32)
        keep, bp = self._bias(bias)
        self.L.sgqo_linear_f32(x, M, K, N, w, layout, bp, y)
        return y

    def linear_f64(self, x, w, layout, bias=None):
        x, w = _f32(x), _f32(w)
        M, K = x.shape
        N = w.shape[1] if layout == LAYOUT_KN else w.shape[0]
        y = np.empty((M, N), np.float64)
        keep, bp = self._bias(bias)
        self.L.sgqo_linear_f64(x, M, K, N, w, layout, bp, y)
        return y

    def qlinear_int4(self, x, packed, scales, K, N, layout, group=32, bias=None):
        x = _f32(x)
        M = x.shape[0]
        y = np.empty((M, N), np.float32)
        keep, bp = self._bias(bias)
        self.L.sgqo_qlinear_int4(x, M, K, N, np.ascontiguousarray(packed, np.uint8), _f32(scales), layout, group, bp, y)
        return y

    def qlinear_int8(self, x, codes, scales, K, N, layout, scheme, bias=None):
        x = _f32(x)
        M = x.shape[0]
        y = np.empty((M, N), np.float32)
        keep, bp = self._bias(bias)
        self.L.sgqo_qlinear_int8(x, M, K, N, np.ascontiguousarray(codes, np.int8).reshape(-1), _f32(scales), layout,
                                 scheme, bp, y)
        return y

    def igemm_s8(self, xq, wq, K, N, layout):
        xq = np.ascontiguousarray(xq, np.int8)
        M = xq.shape[0]
        acc = np.empty((M, N), np.int32)
        self.L.sgqo_igemm_s8(xq.reshape(-1), np.ascontiguousarray(wq, np.int8).reshape(-1), M, K, N, layout, acc)
        return acc

    def qlinear_w8a8(self, x, wq, wscales, K, N, layout, scheme, bias=None):
        x = _f32(x)
        M = x.shape[0]
        xq = np.empty((M, K), np.int8)
        sx = np.empty(M, np.float32)
        acc = np.empty((M, N), np.int32)
        y = np.empty((M, N), np.float32)
        keep, bp = self._bias(bias)
        self.L.sgqo_qlinear_w8a8(x, M, K, N, np.ascontiguousarray(wq, np.int8).reshape(-1), _f32(wscales), layout,
                                 scheme, bp, xq.reshape(-1), sx, acc.reshape(-1), y)
        return xq, sx, acc, y


class Ref:
    """The compiled, unmodified reference (CPU configuration)."""

    def __init__(self, path: str | None = None):
        path = path or os.path.join(_HERE, "_ref", "libsgref.so")
        L = C.CDLL(path)
        i64p = C.POINTER(_i64)
        L.sgref_last_error.restype = C.c_char_p
        L.sgref_num_threads.restype = C.c_int
        L.sgref_quantize_int8.argtypes = [_f32p, i64p, C.c_int, C.c_int, _f32p, _f32p, i64p]
        L.sgref_quantize_int4.argtypes = [_f32p, i64p, C.c_int, _i64, _f32p, _f32p, i64p]
        L.sgref_dequantize_int8.argtypes = [_f32p, _f32p, _i64, i64p, C.c_int, C.c_int, _f32p]
        L.sgref_dequantize_int4.argtypes = [_f32p, _f32p, _i64, i64p, C.c_int, _i64, _f32p]
        L.sgref_linear_create.restype = C.c_void_p
        L.sgref_linear_create.argtypes = [_f32p, C.c_int, _i64, _i64, C.c_int, C.c_int, _i64, C.c_void_p, C.c_int]
        L.sgref_linear_destroy.argtypes = [C.c_void_p]
        L.sgref_linear_num_scales.restype = _i64
        L.sgref_linear_num_scales.argtypes = [C.c_void_p]
        L.sgref_linear_codes.argtypes = [C.c_void_p, _f32p, _f32p]
        L.sgref_linear_forward.argtypes = [C.c_void_p, _f32p, _i64, C.c_int, _f32p]
        if hasattr(L, "sgref_linear_backward_x"):
            L.sgref_linear_backward_x.argtypes = [C.c_void_p, _f32p, _i64, _f32p, _f32p]
        if hasattr(L, "sgref_read_tensor"):
            L.sgref_read_tensor.argtypes = [C.c_int, C.c_char_p, C.c_char_p, _f32p, _i64, C.POINTER(_i64)]
        L.sgref_linear_time.restype = C.c_double
        L.sgref_linear_time.argtypes = [C.c_void_p, _f32p, _i64, C.c_int, C.c_int]
        L.sgref_quantize_time.restype = C.c_double
        L.sgref_quantize_time.argtypes = [_f32p, i64p, C.c_int, C.c_int, C.c_int, _i64, C.c_int]
        if hasattr(L, "sgref_rms_norm"):
            L.sgref_rms_norm.argtypes = [_f32p, _i64, _i64, _f32p, C.c_float, _f32p]
            L.sgref_silu.argtypes = [_f32p, _i64, _f32p]
            L.sgref_softmax_rows.argtypes = [_f32p, _i64, _i64, _f32p]
            L.sgref_rope_tables.argtypes = [_i64, _i64, C.c_float, _f32p, _f32p]
            L.sgref_rope.argtypes = [_f32p, _i64, _i64, _i64, C.c_float, _f32p]
            L.sgref_swiglu.argtypes = [_f32p, _i64, _i64, _i64, _f32p, _f32p, _f32p, _f32p]
        self.L = L

    # -- decode-glue ops (pin oracle/nanollama_oracle.py) -------------------------------------
    def rms_norm(self, x, gamma, eps=1e-5):
        x = _f32(x)
        out = np.empty_like(x)
        self._check(self.L.sgref_rms_norm(x, x.shape[0], x.shape[1], _f32(gamma), eps, out))
        return out

    def silu(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self._check(self.L.sgref_silu(x.reshape(-1), x.size, out.reshape(-1)))
        return out

    def softmax_rows(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self._check(self.L.sgref_softmax_rows(x, x.shape[0], x.shape[1], out))
        return out

    def rope_tables(self, head_dim, max_seq, base=10000.0):
        cos = np.empty((max_seq, head_dim // 2), np.float32)
        sin = np.empty_like(cos)
        self._check(self.L.sgref_rope_tables(head_dim, max_seq, base, cos, sin))
        return cos, sin

    def rope(self, x, max_seq, base=10000.0):
        x = _f32(x)
        out = np.empty_like(x)
        self._check(self.L.sgref_rope(x, x.shape[0], x.shape[1], max_seq, base, out))
        return out

    def swiglu(self, x, w_gate, w_up, w_down):
        """nn::SwiGLU with float weights stored [in, out] (w_down [hidden, in])."""
        x = _f32(x)
        D, H = w_gate.shape
        out = np.empty_like(x)
        self._check(self.L.sgref_swiglu(x, x.shape[0], D, H, _f32(w_gate), _f32(w_up), _f32(w_down), out))
        return out

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.L.sgref_last_error().decode())

    @staticmethod
    def _shape(x):
        s = (_i64 * x.ndim)(*x.shape)
        return s, x.ndim

    def num_threads(self):
        return int(self.L.sgref_num_threads())

    def set_num_threads(self, n):
        self.L.sgref_set_num_threads(int(n))

    def quantize_int8(self, x, scheme=PER_ROW):
        """Returns (codes fp32 of x.shape, scales fp32) exactly as the reference holds them."""
        x = _f32(x)
        codes = np.empty(x.shape, np.float32)
        scales = np.empty(max(x.shape[0] if x.ndim else 1, 1), np.float32)
        ns = _i64(0)
        s, nd = self._shape(x)
        self._check(self.L.sgref_quantize_int8(x.reshape(-1), s, nd, scheme, codes.reshape(-1), scales, C.byref(ns)))
        return codes, scales[: ns.value].copy()

    def quantize_int4(self, x, group=32):
        x = _f32(x)
        g = 32 if group <= 0 else group
        codes = np.empty(x.shape, np.float32)
        scales = np.empty((x.size + g - 1) // g, np.float32)
        ns = _i64(0)
        s, nd = self._shape(x)
        self._check(self.L.sgref_quantize_int4(x.reshape(-1), s, nd, group, codes.reshape(-1), scales, C.byref(ns)))
        assert ns.value == scales.size
        return codes, scales

    def dequantize_int8(self, codes_f32, scales, scheme):
        c = _f32(codes_f32)
        out = np.empty(c.shape, np.float32)
        s, nd = self._shape(c)
        sc = _f32(scales)
        self._check(self.L.sgref_dequantize_int8(c.reshape(-1), sc, sc.size, s, nd, scheme, out.reshape(-1)))
        return out

    def dequantize_int4(self, codes_f32, scales, group=32):
        c = _f32(codes_f32)
        out = np.empty(c.shape, np.float32)
        s, nd = self._shape(c)
        sc = _f32(scales)
        self._check(self.L.sgref_dequantize_int4(c.reshape(-1), sc, sc.size, s, nd, group, out.reshape(-1)))
        return out

    class Linear:
        def __init__(self, ref, w, layout, bits, scheme=PER_ROW, group=32, bias=None, via_module=False):
            self.ref = ref
            w = _f32(w)
            if layout == LAYOUT_KN:
                self.K, self.N = w.shape
            else:
                self.N, self.K = w.shape
            self._bias = None if bias is None else _f32(bias).reshape(-1)
            bp = None if self._bias is None else self._bias.ctypes.data_as(C.c_void_p)
            self.h = ref.L.sgref_linear_create(w.reshape(-1), layout, self.K, self.N, bits, scheme, group, bp,
                                               1 if via_module else 0)
            if not self.h:
                raise RuntimeError(ref.L.sgref_last_error().decode())
            self.shape = w.shape

        def codes(self):
            codes = np.empty(self.shape, np.float32)
            scales = np.empty(self.ref.L.sgref_linear_num_scales(self.h), np.float32)
            self.ref._check(self.ref.L.sgref_linear_codes(self.h, codes.reshape(-1), scales))
            return codes, scales

        def forward(self, x, with_bias=True):
            x = _f32(x)
            y = np.empty((x.shape[0], self.N), np.float32)
            self.ref._check(self.ref.L.sgref_linear_forward(self.h, x, x.shape[0], 1 if with_bias else 0, y))
            return y

        def backward_x(self, x, dy):
            """Gradient with respect to x of sum(forward(x) * dy), by the reference's autograd."""
            x, dy = _f32(x), _f32(dy)
            dx = np.empty_like(x)
            self.ref._check(self.ref.L.sgref_linear_backward_x(self.h, x, x.shape[0], dy, dx))
            return dx

        def time_forward(self, x, iters, with_bias=False):
            x = _f32(x)
            t = self.ref.L.sgref_linear_time(self.h, x, x.shape[0], 1 if with_bias else 0, iters)
            if t < 0:
                raise RuntimeError(self.ref.L.sgref_last_error().decode())
            return t

        def close(self):
            if self.h:
                self.ref.L.sgref_linear_destroy(self.h)
                self.h = None

        def __del__(self):
            try:
                self.close()
            except Exception:
                pass

    def linear(self, *a, **kw):
        return Ref.Linear(self, *a, **kw)

    def read_tensor(self, path, name, capacity, native=True):
        """One fp32 tensor of a checkpoint file, read by the reference's own reader (native .sgrd or SafeTensors)."""
        out = np.empty(capacity, np.float32)
        n = _i64(0)
        self._check(self.L.sgref_read_tensor(0 if native else 1, str(path).encode(), name.encode(), out, capacity, C.byref(n)))
        return out[: n.value].copy()

    def time_quantize(self, x, bits, scheme=PER_TENSOR, group=32, iters=1):
        x = _f32(x)
        s, nd = self._shape(x)
        t = self.L.sgref_quantize_time(x.reshape(-1), s, nd, bits, scheme, group, iters)
        if t < 0:
            raise RuntimeError(self.L.sgref_last_error().decode())
        return t


def load_ref() -> Ref | None:
    path = os.path.join(_HERE, "_ref", "libsgref.so")
    return Ref(path) if os.path.exists(path) else None
