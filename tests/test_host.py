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
                 "ok packed checkpoint", "ok sgrd checkpoint"):
        assert line in r.stdout


def test_reference_reads_checkpoints_written_here(ref):
    """Files written by the host layer, read by the compiled reference's OWN readers: a version-1 .sgrd file
    (serialization::load_checkpoint) and the fp32 tensors of a SafeTensors file that also carries a packed INT4
    tensor (safetensors::load_file; the reference knows no 8-bit dtype and simply ignores what it cannot use)."""
    if ref is None or not hasattr(ref.L, "sgref_read_tensor"):
        pytest.skip("the compiled reference is not available")
    ensure_built()
    with tempfile.TemporaryDirectory() as d:
        r = subprocess.run([EXE, "compat", d], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "ok compat files" in r.stdout, r.stdout + r.stderr
        w = (0.125 * np.arange(30, dtype=np.float32) - 1.5).astype(np.float32)
        b = (1.0 / np.arange(1, 6, dtype=np.float32)).astype(np.float32)
        for native, name in ((True, "f32.sgrd"), (False, "mixed.safetensors")):
            path = os.path.join(d, name)
            assert ref.read_tensor(path, "linear.W", 64, native=native).tobytes() == w.tobytes()
            assert ref.read_tensor(path, "linear.b", 64, native=native).tobytes() == b.tobytes()
        scales = ref.read_tensor(os.path.join(d, "mixed.safetensors"), "packed.w.scales", 64, native=False)
        assert scales.tobytes() == (0.01 * np.arange(1, 5, dtype=np.float32)).astype(np.float32).tobytes()


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
        assert "ok gpu" in r.stdout and "ok packed checkpoints on the device" in r.stdout

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
        # gradient into x (the upstream gradient is the forward's own output) = the forward read with the other layout
        y4, y8 = load("y4.bin", np.float32, (M, N)), load("y8.bin", np.float32, (M, N))
        want_dx4 = port.qlinear_int4(y4, packed4, scales4, N, K, cases.LAYOUT_NK, group, None)
        want_dx8 = port.qlinear_int8(y8, codes8, scales8, N, K, cases.LAYOUT_NK, cases.PER_ROW, None)
        assert rel_err(load("dx4.bin", np.float32, (M, K)), want_dx4) <= TOL_FP32
        assert rel_err(load("dx8.bin", np.float32, (M, K)), want_dx8) <= 1e-6         # the any-shape kernel: the reference's chain
        xa_codes, xa_scales = port.quantize_int8(x, cases.PER_ROW)
        assert np.array_equal(load("xa_codes.bin", np.int8, (M, K)), xa_codes)
        assert load("xa_scales.bin", np.float32).tobytes() == xa_scales.tobytes()
        w_nk = np.ascontiguousarray(w.T)
        packed_nk, scales_nk = port.quantize_int4(w_nk, 32)
        want_dx_nk = port.qlinear_int4(y4, packed_nk, scales_nk, N, K, cases.LAYOUT_KN, 32, None)
        assert rel_err(load("dx4_nk.bin", np.float32, (M, K)), want_dx_nk) <= TOL_FP32
        assert np.array_equal(load("q4_nk_packed.bin", np.uint8), packed_nk)
        want_nk = port.qlinear_int4(x, packed_nk, scales_nk, K, N, cases.LAYOUT_NK, 32, b)
        assert rel_err(load("y4_nk.bin", np.float32, (M, N)), want_nk) <= TOL_FP32
