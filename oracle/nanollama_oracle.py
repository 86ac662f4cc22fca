"""TEST INFRASTRUCTURE — numpy restatement of the decoder the quantized linears sit in.

The reference's own NanoLLaMA (include/sovereigngrad/models.hpp:193-305) has no batch, heads, RoPE
call or KV cache, and its generate() recomputes the whole context for every new token.  The
configuration benchmarked here (dim 2048, 16 layers, 16 heads, SwiGLU 5632, RMSNorm, RoPE 1e4,
vocab 32000) is therefore specified op by op from the reference's operators, each restated below
with the file:line it follows, and the model is evaluated the way generate() does it: one full
causal forward over the whole sequence, no cache.  That makes this file an independent check of the
incremental (KV-cache) product path.

Arithmetic is float64 on float32 inputs unless a function says otherwise; parity with the product
is asserted within the float tolerance of the forward path, never bit for bit.  The per-op
functions are pinned against the compiled reference by tests/test_oracle_glue.py and the golden
file tests/golden/glue.npz.
"""
from __future__ import annotations

import numpy as np


def rms_norm(x, gamma, eps=1e-5):
    """sovereigngrad::rms_norm, src/ops.cpp:1532-1564: x * 1/sqrt(mean(x^2) + eps) * gamma over the last axis."""
    x = np.asarray(x, np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x * inv * np.asarray(gamma, np.float64)


def silu(x):
    """simd::vec_silu, include/sovereigngrad/simd.hpp:103-108: x / (1 + exp(-x))."""
    x = np.asarray(x, np.float64)
    return x / (1.0 + np.exp(-x))


def softmax(x):
    """sovereigngrad::softmax, src/ops.cpp:2101-2150: exp(x - max) / sum over the last axis."""
    x = np.asarray(x, np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def rope_tables(head_dim, max_seq, base=10000.0):
    """nn::RotaryEmbedding, include/sovereigngrad/nn.hpp:583-607: inv_freq[i] = 1 / base^(2i/dim)
    computed in float32, theta = float(pos) * inv_freq[i] in float32, tables [max_seq, dim/2]."""
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base), (np.float32(2.0) * i) / np.float32(head_dim))).astype(np.float32)
    theta = (np.arange(max_seq, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    return np.cos(theta.astype(np.float64)).astype(np.float32), np.sin(theta.astype(np.float64)).astype(np.float32)


def rope(x, cos, sin, positions):
    """sovereigngrad::rotary_embedding, src/ops.cpp:1714-1745: the vector is split in halves and
    element d is paired with element d + half: out[d] = x1*c - x2*s, out[d+half] = x2*c + x1*s.
    x is [..., T, head_dim]; positions [T] selects the table rows (the reference indexes the table
    by the flat vector index, which is the position for a [T, head_dim] input)."""
    x = np.asarray(x, np.float64)
    half = x.shape[-1] // 2
    c = np.asarray(cos, np.float64)[positions]
    s = np.asarray(sin, np.float64)[positions]
    x1, x2 = x[..., :half], x[..., half:]
    return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], axis=-1)


def causal_attention(q, k, v):
    """nn::CausalSelfAttention, include/sovereigngrad/nn.hpp:503-560: scores = q k^T / sqrt(head_dim),
    positions col > row masked (the reference fills -1e9, which softmax turns into exactly 0 in
    float32; -inf here), softmax over keys, times v.  q, k, v are [B, H, T, head_dim]."""
    T, D = q.shape[-2], q.shape[-1]
    scores = np.einsum("bhtd,bhsd->bhts", q, k) / np.sqrt(np.float64(D))
    mask = np.triu(np.ones((T, T), bool), 1)
    scores = np.where(mask, -np.inf, scores)
    return np.einsum("bhts,bhsd->bhtd", softmax(scores), v)


def greedy(logits):
    """NanoLLaMA::generate, include/sovereigngrad/models.hpp:286-298: first index holding the
    strict maximum (the reference compares softmax probabilities; softmax is monotonic)."""
    return np.argmax(np.asarray(logits), axis=-1)


def forward_full(p, tokens):
    """Logits [B, T, vocab] of one causal pass over tokens [B, T].

    p: dict with `embed` [vocab, dim] float32, `n_heads`, `rope_base`, `eps`, `final_norm` [dim],
    `lm_head` [vocab, dim] and `layers`, a list of dicts of DEQUANTIZED float32 weights stored
    [out, in] (`wq wk wv wo w_gate w_up w_down`) plus `attn_norm`, `ffn_norm` [dim].
    Block structure (LLaMA): h += wo(attn(rope(wq n), rope(wk n), wv n)), n = rms_norm(h);
    h += w_down(silu(w_gate n) * w_up n) (nn::SwiGLU, include/sovereigngrad/nn.hpp:138-160)."""
    tokens = np.asarray(tokens)
    B, T = tokens.shape
    H = p["n_heads"]
    h = np.asarray(p["embed"], np.float64)[tokens]                       # embedding lookup, src/ops.cpp:2624
    dim = h.shape[-1]
    hd = dim // H
    cos, sin = rope_tables(hd, T, p.get("rope_base", 10000.0))
    pos = np.arange(T)
    eps = p.get("eps", 1e-5)

    def lin(x, w):
        return x @ np.asarray(w, np.float64).T

    def heads(x):
        return x.reshape(B, T, H, hd).transpose(0, 2, 1, 3)

    for L in p["layers"]:
        n = rms_norm(h, L["attn_norm"], eps)
        q, k, v = heads(lin(n, L["wq"])), heads(lin(n, L["wk"])), heads(lin(n, L["wv"]))
        a = causal_attention(rope(q, cos, sin, pos), rope(k, cos, sin, pos), v)
        h = h + lin(a.transpose(0, 2, 1, 3).reshape(B, T, dim), L["wo"])
        n = rms_norm(h, L["ffn_norm"], eps)
        h = h + lin(silu(lin(n, L["w_gate"])) * lin(n, L["w_up"]), L["w_down"])
    return lin(rms_norm(h, p["final_norm"], eps), p["lm_head"])
