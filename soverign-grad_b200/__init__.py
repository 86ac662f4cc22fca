"""ctypes binding of libsgq.so (include/sgq.h) plus a thin mirror of the reference's
`sovereigngrad::quantization` / `nn::QuantizedLinear*` names over torch CUDA tensors.

torch is used for device memory and streams only: every computation below is a call through
the C ABI into the hand-written sm_100a kernels.  There is no CPU path and no fallback — if the
shared library is missing, importing this package raises.

The directory name contains a hyphen, so load it with `__graft_entry__.load_package()` (which
registers it as module `sgq_b200`).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libsgq.so")

LAYOUT_KN, LAYOUT_NK = 0, 1
PER_TENSOR, PER_ROW = 0, 1
PATH_AUTO, PATH_SIMT, PATH_GEMV, PATH_TC_BF16, PATH_TC_I8 = 0, 1, 2, 3, 4
PATH_NAMES = {PATH_AUTO: "auto", PATH_SIMT: "simt", PATH_GEMV: "gemv", PATH_TC_BF16: "tc_bf16", PATH_TC_I8: "tc_i8"}

# every symbol include/sgq.h declares
EXPORTS = [
    "sgq_status_string", "sgq_last_error", "sgq_abi_version", "sgq_device_status",
    "sgq_quantize_int8", "sgq_quantize_int4", "sgq_dequantize_int8", "sgq_dequantize_int4",
    "sgq_codes_to_f32_int8", "sgq_codes_to_f32_int4", "sgq_codes_from_f32_int8", "sgq_codes_from_f32_int4",
    "sgq_linear_workspace_bytes", "sgq_linear_int4", "sgq_linear_int8",
    "sgq_linear_w8a8", "sgq_linear_w8a8_workspace_bytes", "sgq_interleave_slices", "sgq_linear_int4_decode_noalloc",
    "sgq_prepared_x_bytes", "sgq_prepare_x", "sgq_linear_int4_prepared", "sgq_set_stream_overlap",
    "sgq_linear_int4_allgather", "sgq_linear_int4_allgather_deferred", "sgq_peer_barrier", "sgq_peer_scatter",
    "sgq_set_peer_wait_budget", "sgq_linear_int4_backward_x", "sgq_linear_int8_backward_x",
    "sgq_linear_backward_x_workspace_bytes", "sgq_quantize_activations_int8",
]

# every symbol include/sgq_decoder.h declares
DECODER_EXPORTS = ["sgqd_add_rmsnorm", "sgqd_rope_kv_store", "sgqd_attn_decode", "sgqd_silu_mul", "sgqd_embedding",
                   "sgqd_argmax_rows", "sgqd_attn_prefill", "sgqd_attn_prefill_bf16", "sgqd_attn_decode_allgather",
                   "sgqd_silu_mul_allgather"]


class SgqError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"{what}: {detail}" if detail else what)
        self.status = status


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python soverign-grad_b200/build.py` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    p, i64, i32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t
    lib.sgq_status_string.restype = C.c_char_p
    lib.sgq_status_string.argtypes = [i32]
    lib.sgq_last_error.restype = C.c_char_p
    lib.sgq_device_status.argtypes = [C.POINTER(C.c_uint), i32]
    lib.sgq_quantize_int8.argtypes = [p, i64, i64, i32, p, p, p]
    lib.sgq_quantize_int4.argtypes = [p, i64, i64, p, p, p]
    lib.sgq_dequantize_int8.argtypes = [p, p, i64, i64, i32, p, p]
    lib.sgq_dequantize_int4.argtypes = [p, p, i64, i64, p, p]
    for n in ("sgq_codes_to_f32_int8", "sgq_codes_to_f32_int4", "sgq_codes_from_f32_int8", "sgq_codes_from_f32_int4"):
        getattr(lib, n).argtypes = [p, i64, p, p]
    lib.sgq_linear_workspace_bytes.restype = sz
    lib.sgq_linear_workspace_bytes.argtypes = [i32, i64, i64, i64, i32, i32]
    lib.sgq_linear_int4.argtypes = [p, i64, i64, i64, p, p, i32, i64, p, p, i64, i32, p, sz, p]
    lib.sgq_linear_int8.argtypes = [p, i64, i64, i64, p, p, i32, i32, p, p, i64, i32, p, sz, p]
    lib.sgq_linear_int4_backward_x.argtypes = [p, i64, i64, i64, p, p, i32, i64, p, i64, i32, p, sz, p]
    lib.sgq_linear_int8_backward_x.argtypes = [p, i64, i64, i64, p, p, i32, i32, p, i64, i32, p, sz, p]
    lib.sgq_linear_backward_x_workspace_bytes.restype = sz
    lib.sgq_linear_backward_x_workspace_bytes.argtypes = [i32, i64, i64, i64, i32, i32]
    lib.sgq_quantize_activations_int8.argtypes = [p, i64, i64, p, p, p]
    lib.sgq_linear_w8a8_workspace_bytes.restype = sz
    lib.sgq_linear_w8a8_workspace_bytes.argtypes = [i64, i64, i64]
    lib.sgq_linear_w8a8.argtypes = [p, i64, i64, i64, p, p, i32, p, p, i64, p, p, p, p, sz, p]
    lib.sgq_interleave_slices.argtypes = [p, i64, i64, i64, p, i64, p]
    lib.sgq_linear_int4_decode_noalloc.argtypes = [p, i64, i64, i64, p, p, p, p, i64, p]
    lib.sgq_set_stream_overlap.argtypes = [i32]
    lib.sgq_set_peer_wait_budget.argtypes = [C.c_uint]
    lib.sgq_set_peer_wait_budget.restype = C.c_uint
    lib.sgq_linear_int4_allgather.argtypes = [p, i64, i64, i64, p, p, p, C.POINTER(p), i32, i64, i64, p, sz, C.POINTER(p), i32, p, p]
    lib.sgq_linear_int4_allgather_deferred.argtypes = lib.sgq_linear_int4_allgather.argtypes
    lib.sgq_peer_barrier.argtypes = [C.POINTER(p), i32, i32, p, p]
    lib.sgq_peer_scatter.argtypes = [p, i64, i64, C.POINTER(p), i32, i64, i64, p]
    lib.sgq_prepared_x_bytes.restype = sz
    lib.sgq_prepared_x_bytes.argtypes = [i64, i64]
    lib.sgq_prepare_x.argtypes = [p, i64, i64, p, sz, p]
    lib.sgq_linear_int4_prepared.argtypes = [p, sz, i64, i64, i64, p, p, p, p, i64, p]
    lib.sgqd_add_rmsnorm.argtypes = [p, p, p, C.c_float, i64, i64, p, p, sz, p]
    lib.sgqd_rope_kv_store.argtypes = [p, i64, i64, i64, i64, p, p, p, p, p, i64, p]
    lib.sgqd_attn_decode.argtypes = [p, i64, i64, i64, i64, p, p, p, p, i64, p, p, i64, p, C.c_size_t, p]
    lib.sgqd_silu_mul.argtypes = [p, i64, i64, p, p, sz, p]
    lib.sgqd_attn_prefill.argtypes = [p, i64, i64, i64, i64, i64, p, p, i64, p, p, i64, p]
    lib.sgqd_attn_prefill_bf16.argtypes = [p, i64, i64, i64, i64, i64, p, p, i64, p, p, i64, p]
    lib.sgqd_embedding.argtypes = [p, i64, i64, p, i64, p, p]
    lib.sgqd_attn_decode_allgather.argtypes = [p, i64, i64, i64, i64, p, p, p, p, i64, p, p, C.c_int, i64, i64, p]
    lib.sgqd_silu_mul_allgather.argtypes = [p, i64, i64, p, C.c_int, i64, i64, p]
    lib.sgqd_argmax_rows.argtypes = [p, i64, i64, i64, p, p]
    return lib


lib = _load()


def check(status: int, what: str = "sgq call") -> None:
    if status != 0:
        raise SgqError(status, f"{what} failed: {lib.sgq_status_string(status).decode()}", lib.sgq_last_error().decode())


def set_stream_overlap(enabled) -> int:
    """Programmatic dependent launch for every kernel of the library (see sgq_set_stream_overlap in
    include/sgq.h for the one rule it adds).  Returns the previous setting."""
    return int(lib.sgq_set_stream_overlap(int(enabled)))


def device_status(clear: bool = True) -> int:
    """Synchronising read of the device status word (0 = every bounded wait completed)."""
    w = C.c_uint(0)
    lib.sgq_device_status(C.byref(w), 1 if clear else 0)
    return int(w.value)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32_cuda(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("this library computes on CUDA tensors only")
    return x.contiguous().float()


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


@dataclass
class QuantizedTensor:
    """Mirror of quantization::QuantizedTensor (include/sovereigngrad/quantization.hpp:17-25) with
    the codes held packed (int8, or two nibbles per uint8) instead of one fp32 per code."""
    qdata: torch.Tensor                  # int8 [shape] or uint8 [ceil(numel/2)]
    scales: torch.Tensor                 # fp32
    scheme: int                          # PER_TENSOR | PER_ROW (INT8); unused for INT4
    original_shape: tuple
    group_size: int                      # INT8: numel (as in the reference); INT4: group
    bits: int
    zero_points: Optional[torch.Tensor] = field(default=None)   # never written, as in the reference

    def codes_f32(self) -> torch.Tensor:
        """The reference's `qdata` view: integer codes as fp32, original shape."""
        n = _numel(self.original_shape)
        out = torch.empty(self.original_shape, dtype=torch.float32, device=self.qdata.device)
        fn = lib.sgq_codes_to_f32_int8 if self.bits == 8 else lib.sgq_codes_to_f32_int4
        check(fn(_ptr(self.qdata), n, _ptr(out), _stream()), "codes_to_f32")
        return out


def quantize_int8(x: torch.Tensor, scheme: int = PER_ROW) -> QuantizedTensor:
    """quantization::quantize_int8 (src/quantization.cpp:11-78)."""
    x = _f32_cuda(x)
    shape = tuple(x.shape)
    n = x.numel()
    if scheme == PER_TENSOR or x.dim() < 2:            # :22
        rows, cols, sch, nscales = 1, n, PER_TENSOR, 1
    else:
        rows = shape[0]
        cols = n // rows if rows else 0
        sch, nscales = PER_ROW, rows
    codes = torch.empty(shape, dtype=torch.int8, device=x.device)
    scales = torch.empty(nscales, dtype=torch.float32, device=x.device)
    check(lib.sgq_quantize_int8(_ptr(x), rows, cols, sch, _ptr(codes), _ptr(scales), _stream()), "sgq_quantize_int8")
    return QuantizedTensor(codes, scales, scheme, shape, n, 8)


def quantize_int4(x: torch.Tensor, group_size: int = 32) -> QuantizedTensor:
    """quantization::quantize_int4 (src/quantization.cpp:113-159)."""
    x = _f32_cuda(x)
    g = 32 if group_size <= 0 else group_size
    n = x.numel()
    packed = torch.empty((n + 1) // 2, dtype=torch.uint8, device=x.device)
    scales = torch.empty((n + g - 1) // g, dtype=torch.float32, device=x.device)
    check(lib.sgq_quantize_int4(_ptr(x), n, g, _ptr(packed), _ptr(scales), _stream()), "sgq_quantize_int4")
    return QuantizedTensor(packed, scales, PER_TENSOR, tuple(x.shape), g, 4)


def dequantize_int8(q: QuantizedTensor) -> torch.Tensor:
    """quantization::dequantize_int8 (src/quantization.cpp:80-111)."""
    out = torch.empty(q.original_shape, dtype=torch.float32, device=q.qdata.device)
    n = _numel(q.original_shape)
    per_tensor = q.scheme == PER_TENSOR or q.scales.numel() == 1       # :91
    rows = 1 if per_tensor else q.original_shape[0]
    cols = n // rows if rows else 0
    check(lib.sgq_dequantize_int8(_ptr(q.qdata), _ptr(q.scales), rows, cols, PER_TENSOR if per_tensor else PER_ROW,
                                  _ptr(out), _stream()), "sgq_dequantize_int8")
    return out


def dequantize_int4(q: QuantizedTensor) -> torch.Tensor:
    """quantization::dequantize_int4 (src/quantization.cpp:161-187)."""
    out = torch.empty(q.original_shape, dtype=torch.float32, device=q.qdata.device)
    check(lib.sgq_dequantize_int4(_ptr(q.qdata), _ptr(q.scales), _numel(q.original_shape), q.group_size, _ptr(out),
                                  _stream()), "sgq_dequantize_int4")
    return out


def linear_workspace_bytes(bits: int, M: int, K: int, N: int, layout: int, path: int = PATH_AUTO) -> int:
    return int(lib.sgq_linear_workspace_bytes(bits, M, K, N, layout, path))


class Workspace:
    """Grow-only scratch buffer (256-byte aligned: torch's caching allocator aligns to 512)."""

    def __init__(self, device):
        self.device = device
        self.buf: Optional[torch.Tensor] = None

    def get(self, nbytes: int) -> Optional[torch.Tensor]:
        if nbytes <= 0:
            return self.buf
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buf


def _weight_kn(q: QuantizedTensor, layout: int):
    if len(q.original_shape) != 2:
        raise RuntimeError("matmul currently requires 2D tensors!")          # src/ops.cpp:380-382
    return (q.original_shape[0], q.original_shape[1]) if layout == LAYOUT_KN else (q.original_shape[1], q.original_shape[0])


def quantized_matmul(x: torch.Tensor, q: QuantizedTensor, bias: Optional[torch.Tensor] = None, *, layout: int = LAYOUT_KN,
                     path: int = PATH_AUTO, out: Optional[torch.Tensor] = None, workspace: Optional[Workspace] = None,
                     ldy: Optional[int] = None, workspace_limit: Optional[int] = None) -> torch.Tensor:
    """quantization::quantized_matmul_int8 / _int4 (src/quantization.cpp:189-206) in one launch.
    layout=LAYOUT_KN is the reference's own convention (weight [K,N], y = x*W).  workspace_limit caps the scratch
    bytes offered to the library (the bf16 tensor-core path then dequantizes [N,K] weights tile by tile in shared
    memory instead of expanding them into the scratch first)."""
    x = _f32_cuda(x)
    if x.dim() != 2:
        raise RuntimeError("matmul currently requires 2D tensors!")
    K, N = _weight_kn(q, layout)
    M = x.shape[0]
    if x.shape[1] != K:
        raise RuntimeError("Matrix inner dimensions must match for matmul!")   # src/ops.cpp:387-389
    b = None if bias is None else _f32_cuda(bias).reshape(-1)
    if b is not None and b.numel() != N:
        raise RuntimeError("Incompatible shapes for broadcasting!")            # src/ops.cpp:60
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        ldy = N
    elif ldy is None:
        ldy = out.stride(0)
    need = linear_workspace_bytes(q.bits, M, K, N, layout, path)
    if workspace_limit is not None:
        need = min(need, workspace_limit)
    ws = None
    if need:
        ws = (workspace or Workspace(x.device)).get(need)
    wsp, wsb = (_ptr(ws), ws.numel()) if ws is not None else (None, 0)
    if workspace_limit is not None:
        wsb = min(wsb, workspace_limit)
    if q.bits == 4:
        rc = lib.sgq_linear_int4(_ptr(x), M, K, N, _ptr(q.qdata), _ptr(q.scales), layout, q.group_size, _ptr(b), _ptr(out),
                                 ldy, path, wsp, wsb, _stream())
    else:
        per_tensor = q.scheme == PER_TENSOR or q.scales.numel() == 1
        rc = lib.sgq_linear_int8(_ptr(x), M, K, N, _ptr(q.qdata), _ptr(q.scales), layout,
                                 PER_TENSOR if per_tensor else PER_ROW, _ptr(b), _ptr(out), ldy, path, wsp, wsb, _stream())
    check(rc, "sgq_linear")
    return out


def quantized_matmul_backward_x(dy: torch.Tensor, q: QuantizedTensor, *, layout: int = LAYOUT_KN, path: int = PATH_AUTO,
                                workspace: Optional[Workspace] = None) -> torch.Tensor:
    """Gradient with respect to x of quantized_matmul(x, q): what the reference's autograd computes through
    quantized_matmul_int8 / _int4 when x requires a gradient (src/ops.cpp:367-370, 451-453)."""
    dy = _f32_cuda(dy)
    K, N = _weight_kn(q, layout)
    M = dy.shape[0]
    if dy.dim() != 2 or dy.shape[1] != N:
        raise RuntimeError("Matrix inner dimensions must match for matmul!")
    dx = torch.empty((M, K), dtype=torch.float32, device=dy.device)
    need = int(lib.sgq_linear_backward_x_workspace_bytes(q.bits, M, K, N, layout, path))
    ws = (workspace or Workspace(dy.device)).get(need) if need else None
    wsp, wsb = (_ptr(ws), ws.numel()) if ws is not None else (None, 0)
    if q.bits == 4:
        rc = lib.sgq_linear_int4_backward_x(_ptr(dy), M, K, N, _ptr(q.qdata), _ptr(q.scales), layout, q.group_size, _ptr(dx), K, path,
                                            wsp, wsb, _stream())
    else:
        per_tensor = q.scheme == PER_TENSOR or q.scales.numel() == 1
        rc = lib.sgq_linear_int8_backward_x(_ptr(dy), M, K, N, _ptr(q.qdata), _ptr(q.scales), layout,
                                            PER_TENSOR if per_tensor else PER_ROW, _ptr(dx), K, path, wsp, wsb, _stream())
    check(rc, "sgq_linear_backward_x")
    return dx


def quantize_activations_int8(x: torch.Tensor):
    """Per-row (per-token) INT8 quantization of activations: (codes int8 [M,K], scales fp32 [M])."""
    x = _f32_cuda(x)
    M, K = x.shape
    xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
    sx = torch.empty(M, dtype=torch.float32, device=x.device)
    check(lib.sgq_quantize_activations_int8(_ptr(x), M, K, _ptr(xq), _ptr(sx), _stream()), "sgq_quantize_activations_int8")
    return xq, sx


def prepared_x_bytes(M: int, K: int) -> int:
    """Bytes of the decode kernel's prepared form of x[M, K]; 0 when this shape has none."""
    return int(lib.sgq_prepared_x_bytes(M, K))


def prepare_x(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[M, K] fp32 -> prepared activations (an opaque uint8 buffer) for linear_int4_prepared."""
    x = _f32_cuda(x)
    M, K = x.shape
    nb = prepared_x_bytes(M, K)
    if nb == 0:
        raise SgqError(4, "prepare_x", "no prepared form for this shape (M <= 16, K % 256 == 0)")
    if out is None:
        out = torch.empty(nb, dtype=torch.uint8, device=x.device)
    check(lib.sgq_prepare_x(_ptr(x), M, K, _ptr(out), out.numel(), _stream()), "sgq_prepare_x")
    return out


def linear_int4_prepared(prepared: torch.Tensor, M: int, q: QuantizedTensor, bias: Optional[torch.Tensor] = None,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode forward of an INT4 g=32 weight stored [N, K] on activations already in prepared form."""
    N, K = q.original_shape
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=prepared.device)
    check(lib.sgq_linear_int4_prepared(_ptr(prepared), prepared.numel(), M, K, N, _ptr(q.qdata), _ptr(q.scales), _ptr(bias), _ptr(out),
                                       out.stride(0), _stream()), "sgq_linear_int4_prepared")
    return out


def quantized_matmul_int8(x, q_weight, bias=None, **kw):
    return quantized_matmul(x, q_weight, bias, **kw)


def quantized_matmul_int4(x, q_weight, bias=None, **kw):
    return quantized_matmul(x, q_weight, bias, **kw)


def linear_w8a8(x: torch.Tensor, q: QuantizedTensor, bias: Optional[torch.Tensor] = None, *, want_parts: bool = False):
    """Integer sub-path (no counterpart in the reference): per-row INT8 activations, exact int32
    accumulation on tcgen05 kind::i8.  Weight must be INT8 stored [N,K]."""
    x = _f32_cuda(x)
    N, K = q.original_shape
    M = x.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    xq = sx = acc = None
    if want_parts:
        xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
        sx = torch.empty(M, dtype=torch.float32, device=x.device)
        acc = torch.empty((M, N), dtype=torch.int32, device=x.device)
    nb = int(lib.sgq_linear_w8a8_workspace_bytes(M, K, N))
    ws = torch.empty(max(nb, 256), dtype=torch.uint8, device=x.device)
    b = None if bias is None else _f32_cuda(bias).reshape(-1)
    per_tensor = q.scheme == PER_TENSOR or q.scales.numel() == 1
    check(lib.sgq_linear_w8a8(_ptr(x), M, K, N, _ptr(q.qdata), _ptr(q.scales), PER_TENSOR if per_tensor else PER_ROW, _ptr(b),
                              _ptr(y), N, _ptr(xq), _ptr(sx), _ptr(acc), _ptr(ws), ws.numel(), _stream()), "sgq_linear_w8a8")
    return (y, xq, sx, acc) if want_parts else y


def interleave_slices(gathered: torch.Tensor, world: int, M: int, n_local: int, out: Optional[torch.Tensor] = None):
    """[world][M][n_local] (all-gather order) -> row-major [M, world*n_local]."""
    if out is None:
        out = torch.empty((M, world * n_local), dtype=torch.float32, device=gathered.device)
    check(lib.sgq_interleave_slices(_ptr(gathered), world, M, n_local, _ptr(out), out.stride(0), _stream()),
          "sgq_interleave_slices")
    return out


class QuantizedLinear:
    """nn::QuantizedLinear (include/sovereigngrad/nn.hpp:928-963): INT8, one scale per row of the
    stored [in, out] weight, bias [1, out]."""

    def __init__(self, q_weight: QuantizedTensor, bias: Optional[torch.Tensor], in_features: int, out_features: int,
                 layout: int = LAYOUT_KN):
        self.q_weight, self.bias = q_weight, bias
        self.in_features, self.out_features, self.layout = in_features, out_features, layout
        self._ws = Workspace(q_weight.qdata.device)

    @classmethod
    def from_float(cls, W: torch.Tensor, b: Optional[torch.Tensor], scheme: int = PER_ROW, layout: int = LAYOUT_KN):
        """W is the float layer's weight, [in, out] for LAYOUT_KN (nn.hpp:946-954)."""
        K, N = (W.shape[0], W.shape[1]) if layout == LAYOUT_KN else (W.shape[1], W.shape[0])
        return cls(quantize_int8(W, scheme), None if b is None else b.clone(), K, N, layout)

    def parameters(self):
        return {"qdata": self.q_weight.qdata, "scales": self.q_weight.scales, "bias": self.bias}

    def forward(self, x: torch.Tensor, path: int = PATH_AUTO) -> torch.Tensor:
        return quantized_matmul(x, self.q_weight, self.bias, layout=self.layout, path=path, workspace=self._ws)

    __call__ = forward


class QuantizedLinear4Bit(QuantizedLinear):
    """nn::QuantizedLinear4Bit (include/sovereigngrad/nn.hpp:965-1001)."""

    @classmethod
    def from_float(cls, W: torch.Tensor, b: Optional[torch.Tensor], group_size: int = 32, layout: int = LAYOUT_KN):
        K, N = (W.shape[0], W.shape[1]) if layout == LAYOUT_KN else (W.shape[1], W.shape[0])
        m = cls(quantize_int4(W, group_size), None if b is None else b.clone(), K, N, layout)
        m.group_size = m.q_weight.group_size
        return m
