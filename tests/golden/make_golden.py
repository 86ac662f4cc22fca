"""Regenerates tests/golden/*.npz from the compiled, UNMODIFIED reference.

Run in a container that has the reference checkout:
    make -C oracle ref REF=<reference checkout> && python tests/golden/make_golden.py

Every stored code/scale/output below is what the reference's own functions returned
(sovereigngrad::quantization::* through oracle/ref_driver.cpp).  The reference keeps codes as
fp32; they are stored here as int8, and for INT4 additionally as canonical packed bytes
(element 2i in the low nibble, 2i+1 in the high nibble) produced by the numpy packer below —
deliberately independent of the C port under oracle/.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
import oracle  # noqa: E402
import cases  # noqa: E402


def pack_nibbles(codes_f32: np.ndarray) -> np.ndarray:
    c = codes_f32.reshape(-1).astype(np.int64) & 0xF
    if c.size % 2:
        c = np.concatenate([c, np.zeros(1, np.int64)])
    return (c[0::2] | (c[1::2] << 4)).astype(np.uint8)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def glue_inputs():
    """Seeded inputs of the decode-glue fixtures (tests/golden/glue.npz)."""
    r = np.random.default_rng(20240611)
    return {
        "rms/x": (r.standard_normal((5, 256)) * 1.7).astype(np.float32),
        "rms/gamma": (1.0 + 0.1 * r.standard_normal(256)).astype(np.float32),
        "silu/x": np.concatenate([r.standard_normal(500) * 4.0, [-30.0, -0.0, 0.0, 30.0, 88.0]]).astype(np.float32),
        "softmax/x": (r.standard_normal((6, 97)) * 3.0).astype(np.float32),
        "rope/x": r.standard_normal((40, 128)).astype(np.float32),
        "swiglu/x": r.standard_normal((3, 64)).astype(np.float32),
        "swiglu/w_gate": (r.standard_normal((64, 160)) * 0.1).astype(np.float32),
        "swiglu/w_up": (r.standard_normal((64, 160)) * 0.1).astype(np.float32),
        "swiglu/w_down": (r.standard_normal((160, 64)) * 0.1).astype(np.float32),
    }


def make_glue(ref):
    """Outputs of the reference's own rms_norm / silu / softmax / RotaryEmbedding / SwiGLU."""
    g = glue_inputs()
    g["rms/y"] = ref.rms_norm(g["rms/x"], g["rms/gamma"], 1e-5)
    g["silu/y"] = ref.silu(g["silu/x"])
    g["softmax/y"] = ref.softmax_rows(g["softmax/x"])
    g["rope/cos"], g["rope/sin"] = ref.rope_tables(128, 640, 10000.0)
    g["rope/y"] = ref.rope(g["rope/x"], 640, 10000.0)
    g["swiglu/y"] = ref.swiglu(g["swiglu/x"], g["swiglu/w_gate"], g["swiglu/w_up"], g["swiglu/w_down"])
    g["rope/cos"] = g["rope/cos"][::7].copy()          # keep the file small: every 7th position
    g["rope/sin"] = g["rope/sin"][::7].copy()
    np.savez_compressed(os.path.join(HERE, "glue.npz"), **g)
    print("glue.npz", os.path.getsize(os.path.join(HERE, "glue.npz")), "bytes")


def make_backward(ref):
    """Gradient with respect to x through the reference's own autograd (MatmulNode, src/ops.cpp:362-375),
    seeded with dy."""
    bw = {}
    for name, M, K, N in cases.BACKWARD_CASES:
        for layout in (cases.LAYOUT_KN, cases.LAYOUT_NK):
            x, w, _ = cases.forward_inputs(name, M, K, N, layout)
            dy = cases.backward_seed(name, M, N)
            for tag, bits, scheme, group in (("int4_g32", 4, 0, 32), ("int8_tensor", 8, cases.PER_TENSOR, 0),
                                             ("int8_row", 8, cases.PER_ROW, 0)):
                lin = ref.linear(w, layout, bits, scheme, group, None)
                bw[f"{name}/L{layout}/{tag}/dx"] = lin.backward_x(x, dy)
                lin.close()
    np.savez_compressed(os.path.join(HERE, "backward.npz"), **bw)
    print("backward.npz", os.path.getsize(os.path.join(HERE, "backward.npz")), "bytes")


def main():
    ref = oracle.load_ref()
    assert ref is not None, "build oracle/_ref first (make -C oracle ref)"
    make_glue(ref)
    if sys.argv[1:] == ["glue"]:
        return
    if sys.argv[1:] == ["backward"]:
        make_backward(ref)
        return
    q = {}
    for name, shape, gen in cases.QUANT_CASES:
        x = gen()
        q[f"{name}/x"] = x
        for scheme in (cases.PER_TENSOR, cases.PER_ROW):
            codes, scales = ref.quantize_int8(x, scheme)
            q[f"{name}/int8_s{scheme}/codes"] = codes.astype(np.int8)
            q[f"{name}/int8_s{scheme}/scales"] = scales
            q[f"{name}/int8_s{scheme}/deq"] = ref.dequantize_int8(codes, scales, scheme)
        for g in cases.INT4_GROUPS:
            codes, scales = ref.quantize_int4(x, g)
            q[f"{name}/int4_g{g}/codes"] = codes.astype(np.int8)
            q[f"{name}/int4_g{g}/packed"] = pack_nibbles(codes)
            q[f"{name}/int4_g{g}/scales"] = scales
            q[f"{name}/int4_g{g}/deq"] = ref.dequantize_int4(codes, scales, g)
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **q)

    f = {}
    for name, M, K, N in cases.FORWARD_CASES:
        for layout in (cases.LAYOUT_KN, cases.LAYOUT_NK):
            x, w, b = cases.forward_inputs(name, M, K, N, layout)
            base = f"{name}/L{layout}"
            if M * K + K * N <= 20000:  # small cases also carry their inputs
                f[f"{base}/x"], f[f"{base}/w"], f[f"{base}/b"] = x, w, b
            for tag, bits, scheme, group in (("int4_g32", 4, 0, 32), ("int4_g16", 4, 0, 16),
                                             ("int8_tensor", 8, cases.PER_TENSOR, 0),
                                             ("int8_row", 8, cases.PER_ROW, 0)):
                lin = ref.linear(w, layout, bits, scheme, group, b)
                f[f"{base}/{tag}/y_bias"] = lin.forward(x, True)
                if tag == "int4_g32":
                    f[f"{base}/{tag}/y_nobias"] = lin.forward(x, False)
                lin.close()
            if layout == cases.LAYOUT_KN:
                # the path a user of the reference takes: nn::Linear -> from_float -> forward
                for tag, bits, group in (("module_int8", 8, 0), ("module_int4_g16", 4, 16), ("module_int4_g32", 4, 32)):
                    lin = ref.linear(w, layout, bits, cases.PER_ROW, group, b, via_module=True)
                    f[f"{base}/{tag}/y"] = lin.forward(x, True)
                    codes, scales = lin.codes()
                    f[f"{base}/{tag}/scales"] = scales
                    f[f"{base}/{tag}/codes_sha256"] = np.frombuffer(sha(codes.astype(np.int8)).encode(), np.uint8)
                    lin.close()
    np.savez_compressed(os.path.join(HERE, "forward.npz"), **f)

    make_backward(ref)

    # benchmark configuration 1 at full size: inputs are re-derivable from the seed; keep digests of the
    # codes and a strided sample of the output.
    x, w, b = cases.config1_inputs()
    c1 = {}
    for tag, scheme in (("tensor", cases.PER_TENSOR), ("row", cases.PER_ROW)):
        lin = ref.linear(w, cases.LAYOUT_KN, 8, scheme, 0, b)
        codes, scales = lin.codes()
        y = lin.forward(x, True)
        c1[f"{tag}/codes_sha256"] = np.frombuffer(sha(codes.astype(np.int8)).encode(), np.uint8)
        c1[f"{tag}/scales"] = scales
        c1[f"{tag}/y_sample"] = y[::8, ::8].copy()
        c1[f"{tag}/y_sha256"] = np.frombuffer(sha(y).encode(), np.uint8)
        lin.close()
    lin = ref.linear(w, cases.LAYOUT_KN, 4, 0, 32, b)
    codes, scales = lin.codes()
    c1["int4/packed_sha256"] = np.frombuffer(sha(pack_nibbles(codes)).encode(), np.uint8)
    c1["int4/scales_sha256"] = np.frombuffer(sha(scales).encode(), np.uint8)
    c1["int4/y_sample"] = lin.forward(x, True)[::8, ::8].copy()
    lin.close()
    np.savez_compressed(os.path.join(HERE, "config1.npz"), **c1)
    for n in ("quantize.npz", "forward.npz", "config1.npz"):
        print(n, os.path.getsize(os.path.join(HERE, n)), "bytes")


if __name__ == "__main__":
    main()
