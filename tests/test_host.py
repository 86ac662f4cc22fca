"""The C++17 host layer (pool, tensor, quantization API, layers), driven through its test
executable: on CPU against a stand-in device backend, on the GPU against the oracle."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import cases
from __graft_entry__ import ROOT
from util import TOL_FP32, rel_err

EXE = os.path.join(ROOT, "soverign-grad_b200", "lib", "sgq_host_test")


def ensure_built():
    if not os.path.exists(EXE):
        import __graft_entry__ as g
        g.build()
    assert os.path.exists(EXE)


def test_host_layer_on_cpu():
    ensure_built()
    r = subprocess.run([EXE, "cpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    for line in ("ok cpu pool statistics", "ok device pool on the stand-in backend", "ok tensor metadata", "ok no cpu fallback",
                 "ok packed checkpoint"):
        assert line in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,group", [(4, 32, 16, 16), (8, 256, 96, 32), (3, 70, 45, 7)])
def test_host_layer_on_gpu(port, M, K, N, group):
    """The flow of the reference's own quantization test (src/test_suite.cpp:672-726), first case
    with its very shapes, checked element for element instead of element 0 only."""
    ensure_built()
    x = cases.normal(M + K, (M, K))
    w = cases.normal(K + N, (K, N), float(np.sqrt(2.0 / (K + N))))
    b = cases.normal(N, (N,), 0.1)
    with tempfile.TemporaryDirectory() as d:
        for name, a in (("w", w), ("b", b), ("x", x)):
            a.tofile(os.path.join(d, name + ".bin"))
        r = subprocess.run([EXE, "gpu", d, str(M), str(K), str(N), str(group)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "ok gpu" in r.stdout

        def load(name, dtype, shape=None):
            a = np.fromfile(os.path.join(d, name), dtype=dtype)
            return a if shape is None else a.reshape(shape)

        codes8, scales8 = port.quantize_int8(w, cases.PER_ROW)
        assert np.array_equal(load("q8_codes.bin", np.int8, (K, N)), codes8)
        assert load("q8_scales.bin", np.float32).tobytes() == scales8.tobytes()
        packed4, scales4 = port.quantize_int4(w, group)
        assert np.array_equal(load("q4_packed.bin", np.uint8), packed4)
        assert load("q4_scales.bin", np.float32).tobytes() == scales4.tobytes()
        assert np.array_equal(load("q4_codes_f32.bin", np.float32), port.unpack_int4_codes(packed4, K * N))
        assert np.array_equal(load("deq8.bin", np.float32, (K, N)), port.dequantize_int8(codes8, scales8, cases.PER_ROW))
        assert np.array_equal(load("deq4.bin", np.float32, (K, N)), port.dequantize_int4(packed4, scales4, (K, N), group))
        want8 = port.qlinear_int8(x, codes8, scales8, K, N, cases.LAYOUT_KN, cases.PER_ROW, b)
        want4 = port.qlinear_int4(x, packed4, scales4, K, N, cases.LAYOUT_KN, group, b)
        assert rel_err(load("y8.bin", np.float32, (M, N)), want8) <= TOL_FP32
        assert rel_err(load("y4.bin", np.float32, (M, N)), want4) <= TOL_FP32
        codes8t, scale8t = port.quantize_int8(w, cases.PER_TENSOR)
        assert load("q8t_scales.bin", np.float32).tobytes() == scale8t.tobytes()
        want8t = port.qlinear_int8(x, codes8t, scale8t, K, N, cases.LAYOUT_KN, cases.PER_TENSOR, b)
        assert rel_err(load("y8t.bin", np.float32, (M, N)), want8t) <= TOL_FP32
        w_nk = np.ascontiguousarray(w.T)
        packed_nk, scales_nk = port.quantize_int4(w_nk, 32)
        assert np.array_equal(load("q4_nk_packed.bin", np.uint8), packed_nk)
        want_nk = port.qlinear_int4(x, packed_nk, scales_nk, K, N, cases.LAYOUT_NK, 32, b)
        assert rel_err(load("y4_nk.bin", np.float32, (M, N)), want_nk) <= TOL_FP32
