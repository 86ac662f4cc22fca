"""GPU parity of the quantize / pack / dequantize kernels, through the C ABI, against the
golden fixtures (outputs of the compiled reference) and the oracle port.  Integer and byte
results must match bit for bit."""
import numpy as np
import pytest

import cases

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sgq():
    from __graft_entry__ import load_package
    return load_package()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("name,shape,gen", cases.QUANT_CASES, ids=[c[0] for c in cases.QUANT_CASES])
def test_golden_quantize(sgq, golden, name, shape, gen):
    g = golden["quantize"]
    x = gen()
    xd = dev(x)
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        q = sgq.quantize_int8(xd, scheme)
        assert np.array_equal(host(q.qdata), g[f"{name}/int8_s{scheme}/codes"])
        assert host(q.scales).tobytes() == g[f"{name}/int8_s{scheme}/scales"].tobytes()
        assert np.array_equal(host(sgq.dequantize_int8(q)), g[f"{name}/int8_s{scheme}/deq"], equal_nan=True)
        assert np.array_equal(host(q.codes_f32()), g[f"{name}/int8_s{scheme}/codes"].astype(np.float32))
    for grp in cases.INT4_GROUPS:
        q = sgq.quantize_int4(xd, grp)
        assert np.array_equal(host(q.qdata), g[f"{name}/int4_g{grp}/packed"]), (name, grp)
        assert host(q.scales).tobytes() == g[f"{name}/int4_g{grp}/scales"].tobytes(), (name, grp)
        assert np.array_equal(host(sgq.dequantize_int4(q)), g[f"{name}/int4_g{grp}/deq"], equal_nan=True)
        assert np.array_equal(host(q.codes_f32()), g[f"{name}/int4_g{grp}/codes"].astype(np.float32))


def test_empty_and_tiny(sgq):
    e = torch.empty(0, device="cuda")
    q = sgq.quantize_int4(e, 32)
    assert q.qdata.numel() == 0 and q.scales.numel() == 0
    q = sgq.quantize_int8(torch.empty((0, 8), device="cuda"), cases.PER_ROW)
    assert q.qdata.numel() == 0 and q.scales.numel() == 0
    q = sgq.quantize_int8(e, cases.PER_TENSOR)          # absmax of nothing is the 1e-8 floor
    assert host(q.scales)[0] == np.float32(1e-8) / np.float32(127.0)
    q = sgq.quantize_int4(torch.tensor([1.0], device="cuda"), 32)
    assert host(q.qdata).tolist() == [0x07] and host(q.scales)[0] == np.float32(1.0) / np.float32(7.0)


@pytest.mark.parametrize("n,group", [(32 * 1000 + 17, 32), (4096 * 33, 32), (100003, 32), (100003, 24), (64 * 129, 128),
                                     (1 << 20, 1), (999, 1000)])
def test_int4_ragged_against_port(sgq, port, n, group):
    rng = np.random.default_rng(n + group)
    x = (rng.standard_normal(n) * rng.choice([1e-3, 0.02, 3.0])).astype(np.float32)
    x[rng.random(n) < 0.01] *= 20
    x[:40] = 0.0
    q = sgq.quantize_int4(dev(x), group)
    packed, scales = port.quantize_int4(x, group)
    assert np.array_equal(host(q.qdata), packed)
    assert host(q.scales).tobytes() == scales.tobytes()


def test_int4_unaligned_views(sgq, port):
    """Inputs and outputs that start off a 16-byte boundary take the generic kernels."""
    rng = np.random.default_rng(3)
    base = dev(rng.standard_normal(4096 + 3).astype(np.float32))
    x = base[3:]                                   # 12-byte offset
    q = sgq.quantize_int4(x, 32)
    packed, scales = port.quantize_int4(host(x), 32)
    assert np.array_equal(host(q.qdata), packed) and host(q.scales).tobytes() == scales.tobytes()


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (128, 4096), (77, 1000), (5, 40000), (2048, 64), (4, 8192 * 4 + 4)])
def test_int8_against_port(sgq, port, rows, cols):
    rng = np.random.default_rng(rows * 31 + cols)
    x = (rng.standard_normal((rows, cols)) * 0.5).astype(np.float32)
    x[0, 0] = 0.0
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        q = sgq.quantize_int8(dev(x), scheme)
        codes, scales = port.quantize_int8(x, scheme)
        assert np.array_equal(host(q.qdata), codes), (rows, cols, scheme)
        assert host(q.scales).tobytes() == scales.tobytes()
        assert np.array_equal(host(sgq.dequantize_int8(q)), port.dequantize_int8(codes, scales, scheme))


@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096)])
def test_config3_pack_full_size(sgq, port, shape):
    """benchmark configuration 3: N(0,0.02) with 1% entries x20, INT8 per tensor and INT4 g=32, at full size:
    bytes and scales bit-exact against the oracle, plus a round-trip bound that needs no oracle."""
    w = cases.weight_with_outliers(42, shape)
    wd = dev(w)
    q4 = sgq.quantize_int4(wd, 32)
    packed, scales = port.quantize_int4(w, 32)
    assert np.array_equal(host(q4.qdata), packed)
    assert host(q4.scales).tobytes() == scales.tobytes()
    deq = sgq.dequantize_int4(q4)
    err = (deq - wd).abs().reshape(-1, 32)
    assert bool((err <= q4.scales[:, None] * 0.5000001).all())      # |x - q*s| <= s/2 inside every group
    q8 = sgq.quantize_int8(wd, cases.PER_TENSOR)
    codes, scale = port.quantize_int8(w, cases.PER_TENSOR)
    assert np.array_equal(host(q8.qdata), codes) and host(q8.scales).tobytes() == scale.tobytes()
    assert int(q8.qdata.abs().max()) == 127
    q8r = sgq.quantize_int8(wd, cases.PER_ROW)
    codes, scales = port.quantize_int8(w, cases.PER_ROW)
    assert np.array_equal(host(q8r.qdata), codes) and host(q8r.scales).tobytes() == scales.tobytes()


def test_code_views_round_trip(sgq):
    rng = np.random.default_rng(9)
    c8 = rng.integers(-127, 128, 1001).astype(np.float32)
    c4 = rng.integers(-8, 8, 1001).astype(np.float32)
    for bits, c in ((8, c8), (4, c4)):
        src = dev(c)
        out = torch.empty(1001 if bits == 8 else 501, dtype=torch.int8 if bits == 8 else torch.uint8, device="cuda")
        fn = sgq.lib.sgq_codes_from_f32_int8 if bits == 8 else sgq.lib.sgq_codes_from_f32_int4
        sgq.check(fn(src.data_ptr(), 1001, out.data_ptr(), None))
        back = torch.empty(1001, dtype=torch.float32, device="cuda")
        fn = sgq.lib.sgq_codes_to_f32_int8 if bits == 8 else sgq.lib.sgq_codes_to_f32_int4
        sgq.check(fn(out.data_ptr(), 1001, back.data_ptr(), None))
        torch.cuda.synchronize()
        assert np.array_equal(host(back), c)
