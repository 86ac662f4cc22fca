"""GPU parity of the QuantizedLinear forward, through the C ABI.

Bounds (relative error with an rms floor, tests/util.py):
  1e-3  fp32-dequant paths: tiled SIMT kernel and the decode kernel;
  2e-2  tensor-core paths (bf16 operands, or int8 activations).
The oracle is the C port pinned to the compiled reference; the golden fixtures are outputs of
the compiled reference itself."""
import numpy as np
import pytest

import cases
from util import TOL_BF16, TOL_FP32, bf16_round, block_fixed_point, heavy_tailed_rows, norm_err, rel_err

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sgq():
    from __graft_entry__ import load_package
    return load_package()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def quantize(sgq, wd, tag):
    if tag.startswith("int4"):
        return sgq.quantize_int4(wd, int(tag.split("_g")[1]))
    return sgq.quantize_int8(wd, cases.PER_TENSOR if tag == "int8_tensor" else cases.PER_ROW)


def check_status(sgq):
    assert sgq.device_status() == 0, "a bounded device-side wait ran out"


@pytest.mark.parametrize("name,M,K,N", cases.FORWARD_CASES, ids=[c[0] for c in cases.FORWARD_CASES])
def test_golden_forward_simt(sgq, golden, name, M, K, N):
    """The any-shape kernel reproduces the reference CPU forward: bit for bit where the reference
    runs one fused-multiply-add chain per output, within a few ulp in its <8-column tails."""
    g = golden["forward"]
    for layout in (cases.LAYOUT_KN, cases.LAYOUT_NK):
        x, w, b = cases.forward_inputs(name, M, K, N, layout)
        xd, wd, bd = dev(x), dev(w), dev(b)
        single_chain = (M % 32) < 8 and M < 32 or N % 8 == 0
        for tag in ("int4_g32", "int4_g16", "int8_tensor", "int8_row"):
            q = quantize(sgq, wd, tag)
            y = sgq.quantized_matmul(xd, q, bd, layout=layout, path=sgq.PATH_SIMT).cpu().numpy()
            want = g[f"{name}/L{layout}/{tag}/y_bias"]
            if single_chain:
                assert np.array_equal(y, want), (name, layout, tag)
            else:
                assert rel_err(y, want) <= 1e-6
        q = quantize(sgq, wd, "int4_g32")
        y = sgq.quantized_matmul(xd, q, None, layout=layout, path=sgq.PATH_SIMT).cpu().numpy()
        assert rel_err(y, g[f"{name}/L{layout}/int4_g32/y_nobias"]) <= 1e-6
        if layout == cases.LAYOUT_KN:
            for tag, cls, kw in (("module_int8", sgq.QuantizedLinear, {}),
                                 ("module_int4_g16", sgq.QuantizedLinear4Bit, {"group_size": 16}),
                                 ("module_int4_g32", sgq.QuantizedLinear4Bit, {"group_size": 32})):
                m = cls.from_float(wd, bd, **kw)
                assert m.q_weight.scales.cpu().numpy().tobytes() == g[f"{name}/L{layout}/{tag}/scales"].tobytes()
                y = m(xd).cpu().numpy()                       # AUTO path
                if M >= 64 and K % 64 == 0 and N % 32 == 0:
                    # prefill-sized batches go to the tensor cores in this layout too (bf16 operands)
                    assert norm_err(y, g[f"{name}/L{layout}/{tag}/y"]) <= TOL_BF16
                else:
                    assert rel_err(y, g[f"{name}/L{layout}/{tag}/y"]) <= TOL_FP32


def test_config1_forward(sgq, golden):
    """benchmark configuration 1 (X[128,1024], W[1024,1024], INT8 per tensor, the reference's CPU case)."""
    g = golden["config1"]
    x, w, b = cases.config1_inputs()
    xd, wd, bd = dev(x), dev(w), dev(b)
    for tag, scheme in (("tensor", cases.PER_TENSOR), ("row", cases.PER_ROW)):
        q = sgq.quantize_int8(wd, scheme)
        assert q.scales.cpu().numpy().tobytes() == g[f"{tag}/scales"].tobytes()
        y = sgq.quantized_matmul(xd, q, bd, layout=cases.LAYOUT_KN, path=sgq.PATH_SIMT).cpu().numpy()
        assert np.array_equal(y[::8, ::8], g[f"{tag}/y_sample"])
    q = sgq.quantize_int4(wd, 32)
    y = sgq.quantized_matmul(xd, q, bd, layout=cases.LAYOUT_KN, path=sgq.PATH_SIMT).cpu().numpy()
    assert rel_err(y[::8, ::8], g["int4/y_sample"]) <= TOL_FP32
    y = sgq.quantized_matmul(xd, q, bd, layout=cases.LAYOUT_KN).cpu().numpy()       # AUTO: 128 rows go to the tensor cores (bf16)
    assert norm_err(y[::8, ::8], g["int4/y_sample"]) <= TOL_BF16


DECODE_SHAPES = [(1, 256, 16), (1, 512, 40), (2, 768, 17), (3, 1024, 100), (4, 4096, 512), (5, 1280, 48), (6, 2048, 129),
                 (8, 2048, 129), (7, 4096, 64), (3, 5632, 64), (1, 8192, 256), (4, 11008, 96), (9, 1024, 33), (12, 4096, 80),
                 (16, 4096, 272), (16, 5632, 64), (16, 8192, 80), (12, 11008, 40)]


@pytest.mark.parametrize("M,K,N", DECODE_SHAPES)
def test_decode_kernel_against_port(sgq, port, M, K, N):
    rng = np.random.default_rng(M * 1000003 + K * 101 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(K + N, (N, K))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_NK, 32, b)
    q = sgq.quantize_int4(dev(w), 32)
    # batches whose activation digit planes do not fit in shared memory (K * ceil(M * digits / 8) * 9
    # bytes > ~150 KB) run as several launches over row blocks: still this kernel, same contract
    for bias, ref in ((dev(b), want), (None, want - b[None, :])):
        y = sgq.quantized_matmul(dev(x), q, bias, layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV).cpu().numpy()
        check_status(sgq)
        assert rel_err(y, ref) <= TOL_FP32, (M, K, N, rel_err(y, ref))
    # same launch twice -> identical bits (fixed reduction order)
    y2 = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV).cpu().numpy()
    assert np.array_equal(y2, sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV).cpu().numpy())


DECODE_I8_SHAPES = [(1, 128, 16), (1, 1024, 40), (2, 1152, 17), (3, 4096, 100), (4, 4096, 512), (5, 2304, 48), (6, 2048, 129),
                    (8, 2048, 1000), (9, 8192, 33), (16, 8192, 272), (16, 640, 64), (1, 8192, 2400)]


@pytest.mark.parametrize("M,K,N", DECODE_I8_SHAPES)
def test_decode_int8_kernel_against_port(sgq, port, M, K, N):
    """INT8 weights (per tensor and per row) on the integer decode kernel against the reference-order
    fp32 forward of the port, and against an exact model of the kernel's own arithmetic."""
    rng = np.random.default_rng(M * 1000003 + K * 101 + N + 5)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30.0, (M, 1))).astype(np.float32)     # rows of different magnitude
    w = cases.weight_with_outliers(K + N + 1, (N, K))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    ws = sgq.Workspace(torch.device("cuda"))
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        wq, sw = port.quantize_int8(w, scheme)
        want = port.qlinear_int8(x, wq, sw, K, N, cases.LAYOUT_NK, scheme, b)
        q = sgq.quantize_int8(dev(w), scheme)
        assert sgq.linear_workspace_bytes(8, M, K, N, cases.LAYOUT_NK, sgq.PATH_GEMV) > 0
        y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
        check_status(sgq)
        assert rel_err(y, want) <= TOL_FP32, (M, K, N, scheme, rel_err(y, want))
        # the kernel's own arithmetic: block-scaled fixed-point activations (tests/util.py), exact integer
        # dot products per 128-k step, then fp32 scaling
        model = (block_fixed_point(x, 128) @ wq.astype(np.float64).T) * np.asarray(sw, np.float64).reshape(1, -1) + b[None, :]
        # (three rows or more: a block right at the threshold of the low-digit rule may fall either side of it in fp32)
        assert rel_err(y, model) <= (2e-6 if M <= 2 else 1e-4), ("layout/pipeline error, not rounding", rel_err(y, model))
        y_auto = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
        assert np.array_equal(y_auto, y)                         # AUTO takes this kernel when a workspace is supplied
    with pytest.raises(sgq.SgqError) as err:                     # no workspace: refused, never silently rerouted
        sgq.lib  # noqa: B018
        sgq.check(sgq.lib.sgq_linear_int8(q.qdata.data_ptr(), M, K, N, q.qdata.data_ptr(), q.scales.data_ptr(), cases.LAYOUT_NK,
                                          cases.PER_ROW, None, q.qdata.data_ptr(), N, sgq.PATH_GEMV, None, 0, None))
    assert err.value.status == 5


def test_decode_kernel_rejects_what_it_cannot_run(sgq):
    w = torch.randn(64, 96, device="cuda")       # K = 96 is not a multiple of 256
    q = sgq.quantize_int4(w, 32)
    with pytest.raises(sgq.SgqError) as e:
        sgq.quantized_matmul(torch.randn(1, 96, device="cuda"), q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV)
    assert e.value.status == 4
    # AUTO silently uses the any-shape kernel instead
    sgq.quantized_matmul(torch.randn(1, 96, device="cuda"), q, None, layout=cases.LAYOUT_NK)
    with pytest.raises(RuntimeError):             # inner dimensions must match, as in the reference
        sgq.quantized_matmul(torch.randn(1, 95, device="cuda"), q, None, layout=cases.LAYOUT_NK)


HEAVY = [(M, f, ch) for M in (1, 2, 3, 4, 8, 16) for f, ch in ((30.0, 1), (100.0, 8), (300.0, 1), (300.0, 40))]


@pytest.mark.parametrize("M,factor,channels", HEAVY)
def test_decode_kernels_heavy_tailed_activations(sgq, port, M, factor, channels):
    """Activation rows with a few channels at 30x / 100x / 300x the rest, as normalised decoder
    activations have them: the 1e-3 bound of the decode kernels must not depend on the activation
    distribution.  INT4 g=32 and INT8 (per tensor, per row), against the reference-order forward."""
    K, N = 4096, 272
    x = heavy_tailed_rows(M * 131 + int(factor) + channels, M, K, factor, channels)
    w = cases.weight_with_outliers(K + N + M, (N, K))
    b = (np.random.default_rng(M).standard_normal(N) * 0.1).astype(np.float32)
    ws = sgq.Workspace(torch.device("cuda"))
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_NK, 32, b)
    q = sgq.quantize_int4(dev(w), 32)
    y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
    check_status(sgq)
    assert rel_err(y, want) <= TOL_FP32, ("int4", M, factor, channels, rel_err(y, want))
    codes = port.unpack_int4_codes(packed, N * K).reshape(N, K).astype(np.float64)
    wd = codes * np.repeat(scales.reshape(N, K // 32).astype(np.float64), 32, axis=1)
    model = block_fixed_point(x) @ wd.T + b[None, :]
    # a group right at the threshold of the low-digit rule may fall either side of it in fp32: 5e-5 covers that
    assert rel_err(y, model) <= (5e-6 if M <= 2 else 5e-5), ("layout/pipeline error, not rounding", rel_err(y, model))
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        wq, sw = port.quantize_int8(w, scheme)
        want8 = port.qlinear_int8(x, wq, sw, K, N, cases.LAYOUT_NK, scheme, b)
        q8 = sgq.quantize_int8(dev(w), scheme)
        y8 = sgq.quantized_matmul(dev(x), q8, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
        check_status(sgq)
        assert rel_err(y8, want8) <= TOL_FP32, ("int8", scheme, M, factor, channels, rel_err(y8, want8))


@pytest.mark.parametrize("M", [1, 4, 8])
def test_decode_kernels_non_finite_and_vanishing_activations(sgq, M):
    """A NaN or Inf activation makes its own output row NaN and leaves the other rows alone (the
    reference's fp32 chain would give NaN or Inf there too); an all-zero row gives the bias; rows of
    denormal-sized values are treated as zero."""
    K, N = 1024, 64
    g = torch.Generator(device="cuda").manual_seed(M)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    b = torch.randn(N, device="cuda", generator=g)
    x = torch.randn(M, K, device="cuda", generator=g)
    clean = x.clone()
    x[0, 5] = float("inf")
    if M > 1:
        x[1] = 0.0
    if M > 2:
        x[2] = 1e-38
        x[M - 1, 700] = float("nan")
    ws = sgq.Workspace(torch.device("cuda"))
    for q in (sgq.quantize_int4(w, 32), sgq.quantize_int8(w, sgq.PER_ROW)):
        y = sgq.quantized_matmul(x, q, b, layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws)
        y_clean = sgq.quantized_matmul(clean, q, b, layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws)
        check_status(sgq)
        assert torch.isnan(y[0]).all()
        if M > 1:
            assert torch.equal(y[1], b)
        if M > 2:
            assert torch.equal(y[2], b)
            assert torch.isnan(y[M - 1]).all()
            for m in range(3, M - 1):
                assert torch.equal(y[m], y_clean[m])


@pytest.mark.parametrize("M", [1, 4, 16])
def test_config2_decode_full_size(sgq, port, M):
    """benchmark configuration 2: W[11008,4096] INT4 g=32, X[M,4096], M in {1,4,16}."""
    K, N = 4096, 11008
    x = cases.normal(100 + M, (M, K))
    w = cases.normal(7, (N, K), 0.02)
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_NK, 32, None)
    q = sgq.quantize_int4(dev(w), 32)
    assert np.array_equal(q.qdata.cpu().numpy(), packed)
    y = sgq.quantized_matmul(dev(x), q, None, layout=cases.LAYOUT_NK).cpu().numpy()      # AUTO
    check_status(sgq)
    assert rel_err(y, want) <= TOL_FP32, rel_err(y, want)
    y = sgq.quantized_matmul(dev(x), q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_SIMT).cpu().numpy()
    assert np.array_equal(y, want)     # one fma chain per output: the reference's own bits


def bf16_model(x, packed, scales, port, N, K):
    """What the bf16 tensor-core path computes, in float64: x and code*bf16(scale) rounded to bf16."""
    codes = port.unpack_int4_codes(packed, N * K).reshape(N, K)
    sb = bf16_round(scales).reshape(N, K // 32)
    wb = bf16_round(codes * np.repeat(sb, 32, axis=1))
    return bf16_round(x).astype(np.float64) @ wb.astype(np.float64).T


TC_SHAPES = [(128, 64, 256), (128, 256, 256), (256, 512, 512), (100, 192, 300), (300, 1024, 260), (1, 64, 8), (520, 128, 1000)]


@pytest.mark.parametrize("M,K,N", TC_SHAPES)
def test_tc_bf16_against_port(sgq, port, M, K, N):
    rng = np.random.default_rng(M + 7 * K + 13 * N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(M + K + N, (N, K))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_NK, 32, b)
    q = sgq.quantize_int4(dev(w), 32)
    # two forms: the weight expanded to bf16 in the scratch in front of a TMA-fed GEMM (default), and, with only
    # the activations' scratch, dequantized tile by tile in shared memory (scale rounded to bf16 first)
    wd = port.dequantize_int4(packed, scales, (N, K), 32)
    models = {None: bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64).T + b[None, :],
              M * K * 2 + 256: bf16_model(x, packed, scales, port, N, K) + b[None, :]}
    for limit, model in models.items():
        y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_TC_BF16, workspace_limit=limit).cpu().numpy()
        check_status(sgq)
        assert rel_err(y, model) <= 2e-4, ("layout/pipeline error, not rounding", limit, rel_err(y, model))
        # Operands rounded to 8 significant bits: the bound is normwise (max |error| over max |output|).
        # With 1% x20 outliers and a short K one product can dominate an output, so the rms-floored
        # elementwise ratio is only held to 2e-2 from K >= 1024 on (the benchmark's shapes have K >= 4096).
        assert norm_err(y, want) <= TOL_BF16, norm_err(y, want)
        assert rel_err(y, want) <= (TOL_BF16 if K >= 1024 else 8e-2), rel_err(y, want)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,K,N", [(2048, 4096, 11008), (512, 2048, 4096), (200, 192, 1000), (64, 64, 40), (300, 384, 520),
                                   (130, 256, 70), (1100, 5632, 2048)])
def test_tc_bf16_gemm_that_starts_during_the_expansion(sgq, bits, M, K, N):
    """With overlapped launches the GEMM starts while the weight is still being expanded into the scratch and waits
    on per-part counters.  Forwards with DIFFERENT weights through the SAME scratch, back to back, must give the
    bits of the serial launches: a tile read before its rows were rewritten would show the previous weight."""
    g = torch.Generator(device="cuda").manual_seed(M + N + bits)
    x = torch.randn(M, K, device="cuda", generator=g)
    ws = []
    for i in range(4):
        w = torch.randn(N, K, device="cuda", generator=g) * (0.02 * (i + 1))
        ws.append(sgq.quantize_int4(w, 32) if bits == 4 else sgq.quantize_int8(w, cases.PER_ROW))
    space = sgq.Workspace(torch.device("cuda"))
    outs = {}
    for mode in (0, 1):
        prev = sgq.set_stream_overlap(mode)
        try:
            ys = [torch.empty(M, N, device="cuda") for _ in range(12)]
            for i, y in enumerate(ys):
                sgq.quantized_matmul(x, ws[i % 4], None, layout=cases.LAYOUT_NK, path=sgq.PATH_TC_BF16, out=y, workspace=space)
            torch.cuda.synchronize()
            outs[mode] = ys
        finally:
            sgq.set_stream_overlap(prev)
    check_status(sgq)
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    assert not torch.equal(outs[1][0], outs[1][1])


@pytest.mark.parametrize("M,K,N", TC_SHAPES)
def test_tc_bf16_int8_weights_against_port(sgq, port, M, K, N):
    """INT8 weight codes on the bf16 tensor-core path: the codes are exact in bf16 and the weight
    scale is applied in fp32 by the epilogue, so the only rounding is x -> bf16."""
    rng = np.random.default_rng(3 * M + 7 * K + 13 * N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(M + K + N + 1, (N, K))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        wq, ws = port.quantize_int8(w, scheme)
        want = port.qlinear_int8(x, wq, ws, K, N, cases.LAYOUT_NK, scheme, b)
        q = sgq.quantize_int8(dev(w), scheme)
        sw = np.broadcast_to(np.asarray(ws, np.float32).reshape(-1, 1) if scheme == cases.PER_ROW else np.float32(ws[0]), (N, 1))
        acc = (bf16_round(x).astype(np.float64) @ wq.astype(np.float64).T).astype(np.float32)
        model = (acc * sw.reshape(1, N)).astype(np.float32) + b[None, :]
        for limit in (None, M * K * 2 + 256):      # codes expanded to bf16 in the scratch | expanded tile by tile in shared memory
            y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_TC_BF16, workspace_limit=limit).cpu().numpy()
            check_status(sgq)
            assert rel_err(y, model) <= 2e-5, ("layout/pipeline error, not rounding", limit, rel_err(y, model))
            assert norm_err(y, want) <= TOL_BF16, norm_err(y, want)
            assert rel_err(y, want) <= (TOL_BF16 if K >= 1024 else 8e-2), rel_err(y, want)
    if M >= 64:     # AUTO takes this path for INT8 weights stored [N,K] when a workspace is supplied
        y_auto = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO,
                                      workspace=sgq.Workspace(torch.device("cuda"))).cpu().numpy()
        assert np.array_equal(y_auto, y)


KN_TC_SHAPES = [(128, 64, 256), (256, 512, 512), (100, 192, 288), (300, 1024, 288), (64, 128, 32), (520, 128, 1024)]


@pytest.mark.parametrize("M,K,N", KN_TC_SHAPES)
def test_tc_bf16_kn_layout_against_port(sgq, port, M, K, N):
    """Weights kept in the reference module's own [in, out] layout on the tensor cores: the weight is expanded
    to bf16 (code * scale in fp32, rounded once) and transposed in front of a GEMM whose operands both arrive by TMA."""
    rng = np.random.default_rng(5 * M + 7 * K + 11 * N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(M + K + N + 3, (K, N))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    ws = sgq.Workspace(torch.device("cuda"))
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_KN, 32, b)
    q = sgq.quantize_int4(dev(w), 32)
    y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_TC_BF16, workspace=ws).cpu().numpy()
    check_status(sgq)
    wd = port.dequantize_int4(packed, scales, (K, N), 32)
    model = bf16_round(x).astype(np.float64) @ bf16_round(wd).astype(np.float64) + b[None, :]
    assert rel_err(y, model) <= 2e-5, ("layout/pipeline error, not rounding", rel_err(y, model))
    assert norm_err(y, want) <= TOL_BF16, norm_err(y, want)
    assert rel_err(y, want) <= (TOL_BF16 if K >= 1024 else 8e-2), rel_err(y, want)
    if M >= 64:         # AUTO takes the tensor-core path for this layout too when the workspace is there
        y_auto = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
        assert np.array_equal(y_auto, y)
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        codes, sw = port.quantize_int8(w, scheme)
        want8 = port.qlinear_int8(x, codes, sw, K, N, cases.LAYOUT_KN, scheme, b)
        q8 = sgq.quantize_int8(dev(w), scheme)
        y8 = sgq.quantized_matmul(dev(x), q8, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_TC_BF16, workspace=ws).cpu().numpy()
        check_status(sgq)
        wd8 = port.dequantize_int8(codes, sw, scheme).reshape(K, N)
        model8 = bf16_round(x).astype(np.float64) @ bf16_round(wd8).astype(np.float64) + b[None, :]
        assert rel_err(y8, model8) <= 2e-5, (scheme, rel_err(y8, model8))
        assert norm_err(y8, want8) <= TOL_BF16, (scheme, norm_err(y8, want8))


@pytest.mark.parametrize("group", [8, 16, 64, 128, 96])
def test_tc_bf16_other_group_sizes(sgq, port, group):
    """INT4 groups other than 32 (any multiple of 8, also ones that straddle rows) on the tensor cores, both layouts:
    the weight is expanded word by word, so the group size only selects the scale."""
    M, K, N = 128, 256, 160
    rng = np.random.default_rng(group)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    for layout, shape in ((cases.LAYOUT_NK, (N, K)), (cases.LAYOUT_KN, (K, N))):
        w = cases.weight_with_outliers(group + layout, shape)
        packed, scales = port.quantize_int4(w, group)
        want = port.qlinear_int4(x, packed, scales, K, N, layout, group, b)
        q = sgq.quantize_int4(dev(w), group)
        y = sgq.quantized_matmul(dev(x), q, dev(b), layout=layout, path=sgq.PATH_TC_BF16).cpu().numpy()
        check_status(sgq)
        wd = port.dequantize_int4(packed, scales, shape, group).astype(np.float64)
        wb = bf16_round(wd).astype(np.float64)
        model = bf16_round(x).astype(np.float64) @ (wb.T if layout == cases.LAYOUT_NK else wb) + b[None, :]
        assert rel_err(y, model) <= 2e-5, (group, layout, rel_err(y, model))
        assert norm_err(y, want) <= TOL_BF16, (group, layout, norm_err(y, want))


def test_tc_bf16_kn_layout_rejects_ragged_groups(sgq):
    q = sgq.quantize_int4(torch.randn(64, 48, device="cuda"), 32)          # N = 48: groups straddle rows of the stored tensor
    with pytest.raises(sgq.SgqError) as e:
        sgq.quantized_matmul(torch.randn(128, 64, device="cuda"), q, None, layout=cases.LAYOUT_KN, path=sgq.PATH_TC_BF16)
    assert e.value.status == 4


@pytest.mark.parametrize("M", [17, 33, 63])
def test_batches_between_decode_and_prefill_take_the_decode_kernels(sgq, port, M):
    """AUTO runs 17 .. 63 rows as blocks of 16 rows on the decode kernels (same fp32 contract), not on the
    any-shape kernel: bit-identical to running the blocks by hand."""
    K, N = 1024, 320
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(M + 5, (N, K))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    ws = sgq.Workspace(torch.device("cuda"))
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_NK, 32, b)
    q = sgq.quantize_int4(dev(w), 32)
    y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
    assert rel_err(y, want) <= TOL_FP32, rel_err(y, want)
    blocks = [sgq.quantized_matmul(dev(x[m0:m0 + 16]), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
              for m0 in range(0, M, 16)]
    assert np.array_equal(y, np.concatenate(blocks, axis=0))
    codes, sw = port.quantize_int8(w, cases.PER_TENSOR)
    want8 = port.qlinear_int8(x, codes, sw, K, N, cases.LAYOUT_NK, cases.PER_TENSOR, b)
    q8 = sgq.quantize_int8(dev(w), cases.PER_TENSOR)
    y8 = sgq.quantized_matmul(dev(x), q8, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
    assert rel_err(y8, want8) <= TOL_FP32, rel_err(y8, want8)
    blocks8 = [sgq.quantized_matmul(dev(x[m0:m0 + 16]), q8, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
               for m0 in range(0, M, 16)]
    assert np.array_equal(y8, np.concatenate(blocks8, axis=0))
    check_status(sgq)


I8_SHAPES = [(128, 128, 256), (128, 512, 256), (200, 1024, 300), (1, 16, 8), (260, 272, 520), (64, 4096, 128)]


@pytest.mark.parametrize("M,K,N", I8_SHAPES)
def test_tc_i8_exact(sgq, port, M, K, N):
    """kind::i8: activation codes/scales and the int32 accumulators are exact; the scaled output
    follows the stated formula bit for bit.  The reference has no such path (parity unpinned);
    the float result is additionally compared with the reference-equivalent fp32 forward."""
    rng = np.random.default_rng(M * 3 + K * 5 + N * 7)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.normal(M + K + N, (N, K), 0.02)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        wq, ws = port.quantize_int8(w, scheme)
        xq, sx, acc, want = port.qlinear_w8a8(x, wq, ws, K, N, cases.LAYOUT_NK, scheme, b)
        q = sgq.quantize_int8(dev(w), scheme)
        y, xq_d, sx_d, acc_d = sgq.linear_w8a8(dev(x), q, dev(b), want_parts=True)
        check_status(sgq)
        assert np.array_equal(xq_d.cpu().numpy(), xq)
        assert sx_d.cpu().numpy().tobytes() == sx.tobytes()
        assert np.array_equal(acc_d.cpu().numpy(), acc), "int32 accumulators must be exact"
        assert np.array_equal(y.cpu().numpy(), want)
        y2 = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_NK, path=sgq.PATH_TC_I8).cpu().numpy()
        assert np.array_equal(y2, want)
        fp32 = port.qlinear_int8(x, wq, ws, K, N, cases.LAYOUT_NK, scheme, b)
        if K >= 128:
            assert rel_err(want, fp32) <= 6e-2     # activation rounding to 8 bits, reported not gated at 2e-2


def test_config3_prefill_full_size(sgq, port):
    """benchmark configuration 3: X[2048,4096], W[4096,4096] (1% x20 outliers), INT4 g=32 on the bf16
    tensor-core path.  Full-size check without a full-size CPU product: 16 sampled rows against
    the oracle, everything against the any-shape kernel."""
    M, K, N = 2048, 4096, 4096
    x = cases.normal(5, (M, K))
    w = cases.weight_with_outliers(6, (N, K))
    q = sgq.quantize_int4(dev(w), 32)
    xd = dev(x)
    y = sgq.quantized_matmul(xd, q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_TC_BF16)
    check_status(sgq)
    y_simt = sgq.quantized_matmul(xd, q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_SIMT)
    assert rel_err(y.cpu().numpy(), y_simt.cpu().numpy()) <= TOL_BF16
    rows = np.arange(0, M, M // 16)
    packed, scales = port.quantize_int4(w, 32)
    want = port.qlinear_int4(x[rows], packed, scales, K, N, cases.LAYOUT_NK, 32, None)
    assert np.array_equal(y_simt.cpu().numpy()[rows], want)
    assert rel_err(y.cpu().numpy()[rows], want) <= TOL_BF16
    # linearity in x is exact for power-of-two factors: Y(2x) == 2 Y(x)
    y2 = sgq.quantized_matmul(xd * 2.0, q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_TC_BF16)
    assert torch.equal(y2, y * 2.0)


def test_column_slices_reassemble(sgq):
    """N-sharding on one device: each slice writes its columns into the full buffer through ldy;
    with the tile-granular decode kernel and the SIMT kernel the result equals the unsharded one
    bit for bit (every output is produced by the same instruction sequence)."""
    M, K, N, world = 4, 1024, 512, 4
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.02
    b = torch.randn(N, device="cuda")
    q = sgq.quantize_int4(w, 32)
    for path in (sgq.PATH_SIMT, sgq.PATH_GEMV):
        full = sgq.quantized_matmul(x, q, b, layout=cases.LAYOUT_NK, path=path)
        out = torch.zeros(M, N, device="cuda")
        nl = N // world
        for r in range(world):
            qs = sgq.quantize_int4(w[r * nl:(r + 1) * nl].contiguous(), 32)
            sgq.quantized_matmul(x, qs, b[r * nl:(r + 1) * nl].contiguous(), layout=cases.LAYOUT_NK, path=path,
                                 out=out[:, r * nl:(r + 1) * nl], ldy=N)
        assert torch.equal(out, full)
    # all-gather order [world][M][n_local] -> row-major
    gathered = torch.stack([full[:, r * nl:(r + 1) * nl].contiguous() for r in range(world)])
    assert torch.equal(sgq.interleave_slices(gathered, world, M, nl), full)


@pytest.mark.parametrize("M", [1, 16, 128, 1024, 8192])
def test_config5_large_shapes(sgq, port, M):
    """benchmark configuration 5 at full size on one GPU: W[28672, 8192] as INT4 g=32 and INT8 per tensor,
    X[M, 8192].  Too large for a CPU forward, so: 24 sampled output features against the port on the
    GPU's own codes (the quantizer is bit-exact, tested elsewhere), and Y(2x) = 2 Y(x) exactly (a
    power-of-two factor moves no digit, no bf16 mantissa and no fp32 product)."""
    N, K = 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(5 + M)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    x = torch.randn(M, K, device="cuda", generator=g)
    b = torch.randn(N, device="cuda", generator=g) * 0.1
    rows = np.unique(np.concatenate([[0, 15, 16, N - 1], np.random.default_rng(M).integers(0, N, 20)]))
    ws = sgq.Workspace(torch.device("cuda"))
    xs = x[: min(M, 64)].cpu().numpy()                       # the port forward on 64 batch rows is enough
    bn = b.cpu().numpy()
    for bits in (4, 8):
        q = sgq.quantize_int4(w, 32) if bits == 4 else sgq.quantize_int8(w, sgq.PER_TENSOR)
        y = sgq.quantized_matmul(x, q, b, layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws)
        check_status(sgq)
        if bits == 4:
            packed = q.qdata.view(N, K // 2)[rows].cpu().numpy().reshape(-1)
            scales = q.scales.view(N, K // 32)[rows].cpu().numpy().reshape(-1)
            want = port.qlinear_int4(xs, packed, scales, K, len(rows), cases.LAYOUT_NK, 32, bn[rows])
        else:
            codes = q.qdata.view(N, K)[rows].cpu().numpy()
            want = port.qlinear_int8(xs, codes, q.scales.cpu().numpy(), K, len(rows), cases.LAYOUT_NK, cases.PER_TENSOR, bn[rows])
        got = y[: xs.shape[0]][:, torch.from_numpy(rows).cuda()].cpu().numpy()
        tensor_core = M >= 64
        assert norm_err(got, want) <= (TOL_BF16 if tensor_core else TOL_FP32), (bits, M, norm_err(got, want))
        assert rel_err(got, want) <= (TOL_BF16 if tensor_core else TOL_FP32), (bits, M, rel_err(got, want))
        y0 = sgq.quantized_matmul(x, q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws)
        y2 = sgq.quantized_matmul(x * 2, q, None, layout=cases.LAYOUT_NK, path=sgq.PATH_AUTO, workspace=ws)
        assert torch.equal(y2, y0 * 2), (bits, M)
        del q, y, y0, y2
    check_status(sgq)


KN_DECODE_SHAPES = [(1, 512, 64, 16), (3, 1000, 2048, 32), (4, 4096, 4096, 32), (16, 777, 160, 32), (7, 2048, 48, 16),
                    (2, 300, 4128, 32), (1, 4096, 11008, 32), (5, 17, 32, 32)]


@pytest.mark.parametrize("M,K,N,group", KN_DECODE_SHAPES)
def test_kn_decode_kernel_against_port(sgq, port, M, K, N, group):
    """Weights kept in the reference module's own [in, out] layout (INT4 groups along the flat index,
    INT8 per stored row or per tensor) on the streaming decode kernel for that layout."""
    rng = np.random.default_rng(M * 1000003 + K * 101 + N + group)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = cases.weight_with_outliers(K + N + 2, (K, N))
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    ws = sgq.Workspace(torch.device("cuda"))
    packed, scales = port.quantize_int4(w, group)
    want = port.qlinear_int4(x, packed, scales, K, N, cases.LAYOUT_KN, group, b)
    q = sgq.quantize_int4(dev(w), group)
    assert sgq.linear_workspace_bytes(4, M, K, N, cases.LAYOUT_KN, sgq.PATH_GEMV) > 0
    y = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
    assert rel_err(y, want) <= TOL_FP32, (M, K, N, rel_err(y, want))
    y_auto = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
    assert np.array_equal(y_auto, y)                                   # AUTO takes it when a workspace is supplied, and
    again = sgq.quantized_matmul(dev(x), q, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
    assert np.array_equal(again, y)                                    # slices are added in a fixed order
    y_none = sgq.quantized_matmul(dev(x), q, None, layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
    assert rel_err(y_none, want - b[None, :]) <= TOL_FP32
    for scheme in (cases.PER_TENSOR, cases.PER_ROW):
        codes, sw = port.quantize_int8(w, scheme)
        want8 = port.qlinear_int8(x, codes, sw, K, N, cases.LAYOUT_KN, scheme, b)
        q8 = sgq.quantize_int8(dev(w), scheme)
        y8 = sgq.quantized_matmul(dev(x), q8, dev(b), layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV, workspace=ws).cpu().numpy()
        assert rel_err(y8, want8) <= TOL_FP32, (M, K, N, scheme, rel_err(y8, want8))
    check_status(sgq)


def test_kn_decode_kernel_rejects_what_it_cannot_run(sgq):
    w = torch.randn(64, 40, device="cuda")          # N = 40 is not a multiple of 16
    q = sgq.quantize_int4(w, 32)
    with pytest.raises(sgq.SgqError) as e:
        sgq.quantized_matmul(torch.randn(1, 64, device="cuda"), q, None, layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV)
    assert e.value.status == 4
    sgq.quantized_matmul(torch.randn(1, 64, device="cuda"), q, None, layout=cases.LAYOUT_KN)      # AUTO: any-shape kernel
    q24 = sgq.quantize_int4(torch.randn(64, 48, device="cuda"), 24)                                # group 24: not a multiple of 16
    with pytest.raises(sgq.SgqError):
        sgq.quantized_matmul(torch.randn(1, 64, device="cuda"), q24, None, layout=cases.LAYOUT_KN, path=sgq.PATH_GEMV)


@pytest.mark.parametrize("name,M,K,N", cases.BACKWARD_CASES, ids=[c[0] for c in cases.BACKWARD_CASES])
def test_backward_x_against_reference_autograd(sgq, golden, name, M, K, N):
    """Gradient with respect to x through a frozen quantized layer: the any-shape kernel reproduces what the
    compiled reference's autograd returned (fixtures), the fast paths stay within 1e-3 of it."""
    g = golden["backward"]
    ws = sgq.Workspace(torch.device("cuda"))
    for layout in (cases.LAYOUT_KN, cases.LAYOUT_NK):
        _, w, _ = cases.forward_inputs(name, M, K, N, layout)
        dy = dev(cases.backward_seed(name, M, N))
        single_chain = (M % 32) < 8 and M < 32 or K % 8 == 0
        for tag in ("int4_g32", "int8_tensor", "int8_row"):
            q = quantize(sgq, dev(w), tag)
            want = g[f"{name}/L{layout}/{tag}/dx"]
            dx = sgq.quantized_matmul_backward_x(dy, q, layout=layout, path=sgq.PATH_SIMT).cpu().numpy()
            if single_chain:
                assert np.array_equal(dx, want), (name, layout, tag)
            else:
                assert rel_err(dx, want) <= 1e-6
            dx_auto = sgq.quantized_matmul_backward_x(dy, q, layout=layout, path=sgq.PATH_AUTO, workspace=ws).cpu().numpy()
            assert rel_err(dx_auto, want) <= TOL_FP32, (name, layout, tag, rel_err(dx_auto, want))
    check_status(sgq)


@pytest.mark.parametrize("M,K", [(1, 64), (8, 4096), (37, 1000), (2048, 4096)])
def test_quantize_activations_int8_bit_exact(sgq, port, M, K):
    """Dynamic per-row (per-token) activation quantization = the reference's per-channel quantizer applied to x."""
    x = (cases.normal(M + K, (M, K)) * np.random.default_rng(M).uniform(0.05, 40.0, (M, 1))).astype(np.float32)
    x[0, 0] = 0.0
    if M > 1:
        x[1, :] = 0.0                                  # an all-zero row: scale 1e-8 / 127
    xq, sx = sgq.quantize_activations_int8(dev(x))
    codes, scales = port.quantize_int8(x, cases.PER_ROW)
    assert np.array_equal(xq.cpu().numpy(), codes)
    assert sx.cpu().numpy().tobytes() == np.asarray(scales, np.float32).tobytes()
