"""The numpy decoder oracle (oracle/nanollama_oracle.py) against the reference's own operators:
golden outputs recorded from the compiled reference (tests/golden/glue.npz), and the compiled
reference itself when it is present."""
import os

import numpy as np
import pytest

from oracle import nanollama_oracle as no

GOLD = os.path.join(os.path.dirname(__file__), "golden", "glue.npz")
TOL = 2e-6   # float32 reference vs float64 restatement: a few float32 ulps of the largest operand


@pytest.fixture(scope="module")
def g():
    return dict(np.load(GOLD))


def close(a, b, tol=TOL):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    assert np.max(np.abs(a - b)) <= tol * max(1.0, np.max(np.abs(b)))


def test_rms_norm(g):
    close(no.rms_norm(g["rms/x"], g["rms/gamma"], 1e-5), g["rms/y"])


def test_silu(g):
    close(no.silu(g["silu/x"]), g["silu/y"])


def test_softmax(g):
    close(no.softmax(g["softmax/x"]), g["softmax/y"])


def test_rope_tables_and_rotation(g):
    cos, sin = no.rope_tables(128, 640, 10000.0)
    # theta = float32(pos) * inv_freq: one ulp of powf() in inv_freq moves theta by one float32 ulp,
    # which is 6e-5 at |theta| ~ 640; the tables agree to that, not to an ulp of cos/sin
    close(cos[::7], g["rope/cos"], 1e-4)
    close(sin[::7], g["rope/sin"], 1e-4)
    close(no.rope(g["rope/x"], cos, sin, np.arange(40)), g["rope/y"], 1e-5)


def test_swiglu(g):
    x = g["swiglu/x"].astype(np.float64)
    y = (no.silu(x @ g["swiglu/w_gate"]) * (x @ g["swiglu/w_up"])) @ g["swiglu/w_down"]
    close(y, g["swiglu/y"], 1e-5)


def test_live_reference_matches_golden(ref, g):
    if ref is None or not hasattr(ref.L, "sgref_rms_norm"):
        pytest.skip("compiled reference not present")
    np.testing.assert_array_equal(ref.rms_norm(g["rms/x"], g["rms/gamma"], 1e-5), g["rms/y"])
    np.testing.assert_array_equal(ref.rope(g["rope/x"], 640, 10000.0), g["rope/y"])
    np.testing.assert_array_equal(ref.silu(g["silu/x"]), g["silu/y"])


def test_full_forward_is_causal_and_greedy_is_first_max():
    r = np.random.default_rng(0)
    dim, H, hid, V = 32, 2, 48, 50
    layer = lambda: {"wq": r.standard_normal((dim, dim)) * 0.2, "wk": r.standard_normal((dim, dim)) * 0.2,  # noqa: E731
                     "wv": r.standard_normal((dim, dim)) * 0.2, "wo": r.standard_normal((dim, dim)) * 0.2,
                     "w_gate": r.standard_normal((hid, dim)) * 0.2, "w_up": r.standard_normal((hid, dim)) * 0.2,
                     "w_down": r.standard_normal((dim, hid)) * 0.2, "attn_norm": np.ones(dim), "ffn_norm": np.ones(dim)}
    p = {"embed": r.standard_normal((V, dim)), "n_heads": H, "final_norm": np.ones(dim),
         "lm_head": r.standard_normal((V, dim)) * 0.2, "layers": [layer(), layer()]}
    tok = r.integers(0, V, (2, 9))
    full = no.forward_full(p, tok)
    part = no.forward_full(p, tok[:, :5])
    np.testing.assert_allclose(full[:, :5], part, rtol=1e-12, atol=1e-12)   # later tokens do not leak back
    assert no.greedy(np.array([1.0, 3.0, 3.0, 2.0])) == 1
