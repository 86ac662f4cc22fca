"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, validates arguments before touching a device, and refuses to compute without a B200."""
import ctypes as C
import os
import re

import pytest

from __graft_entry__ import ROOT, load_package


@pytest.fixture(scope="module")
def sgq():
    return load_package()


def header_symbols(name="sgq.h", prefix="sgq_"):
    text = open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(sgq):
    declared = header_symbols()
    assert len(declared) >= 15
    assert sorted(sgq.EXPORTS) == declared, "python binding list and header disagree"
    for name in declared:
        assert hasattr(sgq.lib, name), f"{name} is declared in sgq.h but not exported by libsgq.so"


def test_library_exports_every_decoder_symbol(sgq):
    declared = header_symbols("sgq_decoder.h", "sgqd_")
    assert sorted(sgq.DECODER_EXPORTS) == declared
    for name in declared:
        assert hasattr(sgq.lib, name), f"{name} is declared in sgq_decoder.h but not exported by libsgq.so"


def test_decoder_argument_validation_needs_no_device(sgq):
    L = sgq.lib
    one = C.c_void_p(256)
    assert L.sgqd_add_rmsnorm(one, None, one, 1e-5, -1, 8, one, None, 0, None) == 2
    assert L.sgqd_add_rmsnorm(None, None, one, 1e-5, 2, 8, one, None, 0, None) == 1
    assert L.sgqd_add_rmsnorm(one, None, one, 1e-5, 2, 8, one, None, 0, None) == 3     # out aliases h
    assert L.sgqd_add_rmsnorm(None, None, None, 1e-5, 0, 8, None, None, 0, None) == 0  # empty
    two = C.c_void_p(512)
    assert L.sgqd_add_rmsnorm(one, None, one, 1e-5, 2, 100, two, two, 4096, None) == 4  # no prepared form for dim 100
    assert L.sgqd_add_rmsnorm(one, None, one, 1e-5, 2, 256, two, two, 16, None) == 5    # prepared buffer too small
    assert int(L.sgq_prepared_x_bytes(8, 2048)) == (2048 // 32) * (3 * 288 + 16)      # digits + group scales of 2 main sets + 1 low set, flags
    assert L.sgq_linear_int4_prepared(one, 64, 8, 2048, 64, one, one, None, one, 64, None) == 5
    assert L.sgq_linear_int4_prepared(one, 1 << 20, 8, 2050, 64, one, one, None, one, 64, None) == 4
    assert L.sgqd_rope_kv_store(one, 1, 1, 2, 12, one, one, one, one, one, 8, None) == 2   # head_dim % 8
    assert L.sgqd_attn_decode(one, 768, 1, 2, 96, one, one, one, one, 8, one, one, 256, None, 0, None) == 4    # head_dim 96
    assert L.sgqd_attn_decode(one, 100, 1, 2, 128, one, one, one, one, 8, one, one, 256, None, 0, None) == 2   # stride too small
    assert L.sgqd_attn_decode(None, 768, 1, 2, 128, one, one, one, one, 8, one, one, 256, None, 0, None) == 1
    assert L.sgqd_silu_mul(None, 2, 8, None, None, 0, None) == 1


def test_abi_version_and_status_strings(sgq):
    assert sgq.lib.sgq_abi_version() == 1
    seen = {sgq.lib.sgq_status_string(i).decode() for i in range(10)}
    assert len(seen) == 10 and "ok" in seen
    assert sgq.lib.sgq_status_string(99).decode() == "unknown status"


def test_argument_validation_needs_no_device(sgq):
    L = sgq.lib
    assert L.sgq_quantize_int4(None, -1, 32, None, None, None) == 2           # bad shape
    assert L.sgq_quantize_int4(None, 64, 32, None, None, None) == 1           # null pointer
    assert L.sgq_quantize_int8(None, 4, 4, 7, None, None, None) == 3          # unknown scheme
    assert L.sgq_quantize_int8(None, -4, 4, 0, None, None, None) == 2
    assert L.sgq_dequantize_int4(None, None, 8, 32, None, None) == 1
    one = C.c_void_p(256)  # never dereferenced: validation fails first
    assert L.sgq_linear_int4(one, 1, 64, 64, one, one, 5, 32, None, one, 64, 0, None, 0, None) == 3   # layout
    assert L.sgq_linear_int4(one, 1, 64, 64, one, one, 1, 32, None, one, 8, 0, None, 0, None) == 2    # ldy < N
    assert L.sgq_linear_int4(one, 1, 64, 64, one, one, 1, 32, None, None, 64, 0, None, 0, None) == 1  # y NULL
    assert L.sgq_linear_int8(one, 1, 64, 64, one, one, 1, 9, None, one, 64, 0, None, 0, None) == 3    # scheme
    assert L.sgq_linear_int4(one, 1, 64, 64, one, one, 1, 32, None, one, 64, 42, None, 0, None) == 3  # path
    assert L.sgq_linear_int4(one, 1, 64, 64, one, one, 1, 32, None, one, 64, 0, C.c_void_p(8), 64, None) == 5  # ws align
    assert b"256-byte" in L.sgq_last_error()
    # empty problems are fine and touch nothing
    assert L.sgq_linear_int4(None, 0, 64, 64, None, None, 1, 32, None, None, 64, 0, None, 0, None) == 0
    assert L.sgq_interleave_slices(None, 2, 4, 8, None, 8, None) == 2         # ldd < world*n_local


def test_workspace_queries(sgq):
    assert sgq.linear_workspace_bytes(4, 1, 4096, 11008, sgq.LAYOUT_NK, sgq.PATH_GEMV) == 0
    assert sgq.linear_workspace_bytes(4, 2048, 4096, 4096, sgq.LAYOUT_NK, sgq.PATH_TC_BF16) == 2048 * 4096 * 2 + 4096 * 4096 * 2 + 256   # bf16 x + expanded weight + progress counters
    assert sgq.linear_workspace_bytes(4, 2048, 4096, 4096, sgq.LAYOUT_NK, sgq.PATH_SIMT) == 0
    assert sgq.linear_workspace_bytes(4, 0, 4096, 4096, sgq.LAYOUT_NK, sgq.PATH_AUTO) == 0
    assert int(sgq.lib.sgq_linear_w8a8_workspace_bytes(128, 1024, 1024)) == 128 * 1024 + 512
    # INT8 decode kernel: digit planes (256 B) and scales (32 B) of the whole batch per 32-k group and set of 8 columns
    # (16 rows: 4 main sets + 2 low sets), 16 flag bytes per group
    assert sgq.linear_workspace_bytes(8, 16, 8192, 64, sgq.LAYOUT_NK, sgq.PATH_GEMV) == (8192 // 32) * (6 * 288 + 16)
    assert sgq.linear_workspace_bytes(8, 4, 100, 64, sgq.LAYOUT_NK, sgq.PATH_GEMV) == 0          # K % 128 != 0: no such path
    assert sgq.linear_workspace_bytes(8, 2048, 4096, 64, sgq.LAYOUT_NK, sgq.PATH_TC_BF16) == 2048 * 4096 * 2 + 64 * 4096 * 2 + 256
    # an INT4 batch of more than 8 rows whose planes exceed shared memory runs as blocks of at most 8 rows
    # that share one scratch: 2 main sets + 1 low set
    assert sgq.linear_workspace_bytes(4, 16, 8192, 64, sgq.LAYOUT_NK, sgq.PATH_GEMV) == (8192 // 32) * (3 * 288 + 16)


def test_no_cpu_fallback(sgq):
    """Without a compute-capability-10 device a compute call must fail loudly, not fall back."""
    import torch
    if torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10:
        pytest.skip("a B200 is present")
    one = C.c_void_p(256)
    rc = sgq.lib.sgq_quantize_int4(one, 64, 32, one, one, None)
    assert rc in (7, 8), rc   # CUDA error or "device is not sm_100"
    with pytest.raises(ValueError):
        sgq.quantize_int4(torch.zeros(64), 32)   # CPU tensors are rejected by the binding
