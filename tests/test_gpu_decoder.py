"""Decoder glue (include/sgq_decoder.h) and the NanoLLaMA-INT4 greedy decoder against the numpy
restatement in oracle/nanollama_oracle.py, which evaluates the model the way the reference's
generate() does: one full causal pass over the whole sequence, no KV cache.  Float tolerances:
1e-3 (fp32 paths) and 2e-2 (bf16 tensor-core prefill), relative to the largest reference value."""
import ctypes as C
import importlib

import numpy as np
import pytest
import torch

from oracle import nanollama_oracle as no
from util import TOL_BF16, TOL_FP32, norm_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sgq():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="module")
def nl(sgq):
    return importlib.import_module("sgq_b200.nanollama")


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda()


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("rows,dim,with_delta", [(1, 256, False), (8, 2048, True), (5, 100, True), (300, 513, False)])
def test_add_rmsnorm(sgq, rows, dim, with_delta):
    r = np.random.default_rng(rows * 7 + dim)
    h = r.standard_normal((rows, dim)).astype(np.float32) * 2
    d = r.standard_normal((rows, dim)).astype(np.float32) if with_delta else None
    g = (1 + 0.2 * r.standard_normal(dim)).astype(np.float32)
    ht, dt, gt = dev(h), (dev(d) if with_delta else None), dev(g)
    out = torch.empty_like(ht)
    sgq.check(sgq.lib.sgqd_add_rmsnorm(ptr(ht), ptr(dt), ptr(gt), 1e-5, rows, dim, ptr(out), None, 0, stream()))
    hsum = h.astype(np.float64) + (d if with_delta else 0)
    assert np.max(np.abs(ht.cpu().numpy() - hsum)) <= 1e-6 * np.max(np.abs(hsum))     # residual stream updated in place
    assert norm_err(out.cpu().numpy(), no.rms_norm(hsum.astype(np.float32), g, 1e-5)) <= 5e-6


def test_add_rmsnorm_rejects_alias(sgq):
    h = torch.zeros(2, 64, device="cuda")
    g = torch.ones(64, device="cuda")
    assert sgq.lib.sgqd_add_rmsnorm(ptr(h), None, ptr(g), 1e-5, 2, 64, ptr(h), None, 0, stream()) == 3


@pytest.mark.parametrize("rows,hidden", [(1, 5632), (8, 704), (3, 37)])
def test_silu_mul(sgq, rows, hidden):
    r = np.random.default_rng(hidden)
    gu = (r.standard_normal((rows, 2 * hidden)) * 3).astype(np.float32)
    out = torch.empty(rows, hidden, device="cuda")
    gt = dev(gu)
    sgq.check(sgq.lib.sgqd_silu_mul(ptr(gt), rows, hidden, ptr(out), None, 0, stream()))
    want = no.silu(gu[:, :hidden]) * gu[:, hidden:].astype(np.float64)
    assert norm_err(out.cpu().numpy(), want) <= 2e-6


@pytest.mark.parametrize("M,K,N", [(1, 2048, 512), (5, 256, 48), (8, 2048, 6144), (8, 5632, 2048), (16, 4096, 1024)])
def test_prepared_activations_give_the_decode_kernels_bits(sgq, M, K, N):
    """sgq_prepare_x + sgq_linear_int4_prepared, and the operators that emit the prepared form
    themselves, against sgq_linear_int4 on the same fp32 activations: identical bits."""
    g = torch.Generator(device="cuda").manual_seed(M * K + N)
    x = torch.randn(M, K, device="cuda", generator=g) * 3
    q = sgq.quantize_int4(torch.randn(N, K, device="cuda", generator=g) * 0.05, 32)
    bias = torch.randn(N, device="cuda", generator=g)
    want = sgq.quantized_matmul(x, q, bias, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=sgq.Workspace(x.device))
    nb = sgq.prepared_x_bytes(M, K)
    assert nb > 0 and nb % 256 == 0
    got = sgq.linear_int4_prepared(sgq.prepare_x(x), M, q, bias)
    assert torch.equal(got, want)
    # RMSNorm emitting the prepared form of its output
    h, gamma = x.clone(), 1 + 0.1 * torch.randn(K, device="cuda", generator=g)
    n, planes = torch.empty_like(h), torch.empty(nb, dtype=torch.uint8, device="cuda")
    sgq.check(sgq.lib.sgqd_add_rmsnorm(ptr(h), None, ptr(gamma), 1e-5, M, K, ptr(n), ptr(planes), nb, stream()))
    want_n = sgq.quantized_matmul(n, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=sgq.Workspace(x.device))
    assert torch.equal(sgq.linear_int4_prepared(planes, M, q), want_n)
    # SiLU gate emitting the prepared form of its output
    gu = torch.randn(M, 2 * K, device="cuda", generator=g) * 2
    act = torch.empty(M, K, device="cuda")
    sgq.check(sgq.lib.sgqd_silu_mul(ptr(gu), M, K, ptr(act), ptr(planes), nb, stream()))
    plain = torch.empty(M, K, device="cuda")
    sgq.check(sgq.lib.sgqd_silu_mul(ptr(gu), M, K, ptr(plain), None, 0, stream()))
    assert torch.equal(act, plain)
    want_a = sgq.quantized_matmul(act, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=sgq.Workspace(x.device))
    assert torch.equal(sgq.linear_int4_prepared(planes, M, q), want_a)


def test_prepared_activations_reject_unsupported_shapes(sgq):
    assert sgq.prepared_x_bytes(17, 2048) == 0 and sgq.prepared_x_bytes(4, 300) == 0 and sgq.prepared_x_bytes(0, 2048) == 0
    x = torch.zeros(17, 2048, device="cuda")
    with pytest.raises(sgq.SgqError):
        sgq.prepare_x(x)
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    assert sgq.lib.sgq_prepare_x(ptr(x[:4]), 4, 2048, ptr(buf), buf.numel(), stream()) == 5      # buffer too small
    assert sgq.lib.sgqd_silu_mul(ptr(x), 4, 1024, ptr(x), ptr(buf), buf.numel(), stream()) == 5


@pytest.mark.parametrize("B,T,H,hd,pos0,max_seq", [(2, 1, 2, 128, 0, 16), (2, 1, 3, 64, 9, 16), (2, 5, 2, 128, 3, 16),
                                                   (1, 4, 1, 128, 14, 16)])
def test_rope_kv_store(sgq, B, T, H, hd, pos0, max_seq):
    r = np.random.default_rng(B * 100 + T * 10 + pos0)
    dim = H * hd
    qkv = r.standard_normal((B * T, 3 * dim)).astype(np.float32)
    cos, sin = no.rope_tables(hd, max_seq)
    kc = torch.full((B, H, max_seq, hd), 7.0, device="cuda")
    vc = torch.full((B, H, max_seq, hd), 7.0, device="cuda")
    qt = dev(qkv)
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    ct, st = dev(cos), dev(sin)
    sgq.check(sgq.lib.sgqd_rope_kv_store(ptr(qt), B, T, H, hd, ptr(ct), ptr(st), ptr(pos), ptr(kc), ptr(vc), max_seq, stream()))
    got, kcn, vcn = qt.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy()
    for b in range(B):
        for i in range(T):
            m, p = b * T + i, pos0 + i
            q = qkv[m, :dim].reshape(H, hd)
            k = qkv[m, dim:2 * dim].reshape(H, hd)
            v = qkv[m, 2 * dim:].reshape(H, hd)
            if p >= max_seq:                                   # skipped token: nothing rotated, nothing stored
                np.testing.assert_array_equal(got[m, :dim].reshape(H, hd), q)
                continue
            assert norm_err(got[m, :dim].reshape(H, hd), no.rope(q, cos, sin, [p])) <= 2e-6
            assert norm_err(kcn[b, :, p], no.rope(k, cos, sin, [p])) <= 2e-6
            np.testing.assert_array_equal(vcn[b, :, p], v)
            np.testing.assert_array_equal(got[m, dim:], qkv[m, dim:])          # k and v rows of qkv are left alone
    untouched = np.ones(max_seq, bool)
    untouched[pos0:min(pos0 + T, max_seq)] = False
    assert (kcn[:, :, untouched] == 7.0).all() and (vcn[:, :, untouched] == 7.0).all()


@pytest.mark.parametrize("B,H,hd,length,max_seq", [(1, 1, 128, 1, 8), (2, 2, 128, 7, 64), (8, 16, 128, 130, 640),
                                                   (8, 16, 128, 640, 640), (3, 5, 64, 333, 512), (40, 32, 64, 100, 128),
                                                   (8, 2, 128, 513, 640)])
def test_attn_decode(sgq, B, H, hd, length, max_seq):
    """`length` counts the new token: the cache holds length - 1 rotated keys, the kernel rotates and
    appends the new one at position length - 1 and attends to all of them."""
    r = np.random.default_rng(length * 3 + hd)
    dim, pos0 = H * hd, length - 1
    qkv = r.standard_normal((B, 3 * dim)).astype(np.float32)
    kc = (r.standard_normal((B, H, max_seq, hd)) * 1.5).astype(np.float32)
    vc = r.standard_normal((B, H, max_seq, hd)).astype(np.float32)
    cos, sin = no.rope_tables(hd, max_seq)
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    out = torch.empty(B, dim, device="cuda")
    qt, kt, vt, ct, st = dev(qkv), dev(kc), dev(vc), dev(cos), dev(sin)
    nb = sgq.prepared_x_bytes(B, dim)                         # 0 where (B, dim) has no prepared form
    planes = torch.zeros(max(nb, 1), dtype=torch.uint8, device="cuda")
    for _ in range(2):                                         # a second call over the already appended row changes nothing
        sgq.check(sgq.lib.sgqd_attn_decode(ptr(qt), 3 * dim, B, H, hd, ptr(ct), ptr(st), ptr(kt), ptr(vt), max_seq, ptr(pos), ptr(out),
                                           dim, ptr(planes) if nb else None, nb, stream()))
    if nb:       # the prepared form the kernel emits is the one sgq_prepare_x makes of its fp32 output
        assert torch.equal(planes[:nb], sgq.prepare_x(out, torch.zeros(nb, dtype=torch.uint8, device="cuda"))[:nb])
    q = no.rope(qkv[:, :dim].reshape(B, H, 1, hd), cos, sin, [pos0])
    k_new = no.rope(qkv[:, dim:2 * dim].reshape(B, H, 1, hd), cos, sin, [pos0])
    v_new = qkv[:, 2 * dim:].reshape(B, H, 1, hd)
    k = np.concatenate([kc[:, :, :pos0].astype(np.float64), k_new], axis=2)
    v = np.concatenate([vc[:, :, :pos0].astype(np.float64), v_new], axis=2)
    p = no.softmax(np.einsum("bhqd,bhtd->bhqt", q, k) / np.sqrt(hd))
    want = np.einsum("bhqt,bhtd->bhqd", p, v).reshape(B, dim)
    assert norm_err(out.cpu().numpy(), want) <= 5e-6
    kcn, vcn = kt.cpu().numpy(), vt.cpu().numpy()
    assert norm_err(kcn[:, :, pos0], k_new[:, :, 0]) <= 2e-6                      # appended rows
    np.testing.assert_array_equal(vcn[:, :, pos0], v_new[:, :, 0])
    keep = np.arange(max_seq) != pos0
    np.testing.assert_array_equal(kcn[:, :, keep], kc[:, :, keep])                # everything else untouched
    np.testing.assert_array_equal(vcn[:, :, keep], vc[:, :, keep])
    np.testing.assert_array_equal(qt.cpu().numpy(), qkv)                          # qkv is read only


def test_column_sharded_operators_store_into_every_output(sgq):
    """sgqd_attn_decode_allgather / sgqd_silu_mul_allgather with two output buffers on one GPU standing in for
    two ranks: both receive the slice at the column offset, bit-equal to the plain operators, the columns
    beside it stay untouched; bad arguments are refused."""
    B, H, hd, max_seq, length = 3, 2, 128, 32, 9
    r = np.random.default_rng(21)
    dim, pos0, wide, off = H * hd, length - 1, 3 * H * hd, H * hd
    qkv = dev(r.standard_normal((B, 3 * dim)).astype(np.float32))
    kc0, vc0 = r.standard_normal((B, H, max_seq, hd)).astype(np.float32), r.standard_normal((B, H, max_seq, hd)).astype(np.float32)
    cos, sin = no.rope_tables(hd, max_seq)
    ct, st = dev(cos), dev(sin)
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    ref = torch.empty(B, dim, device="cuda")
    kt, vt = dev(kc0), dev(vc0)
    sgq.check(sgq.lib.sgqd_attn_decode(ptr(qkv), 3 * dim, B, H, hd, ptr(ct), ptr(st), ptr(kt), ptr(vt), max_seq, ptr(pos), ptr(ref),
                                       dim, None, 0, stream()))
    outs = [torch.full((B, wide), 7.0, device="cuda") for _ in range(2)]
    ranks = (C.c_void_p * 2)(*[o.data_ptr() for o in outs])
    kt2, vt2 = dev(kc0), dev(vc0)
    sgq.check(sgq.lib.sgqd_attn_decode_allgather(ptr(qkv), 3 * dim, B, H, hd, ptr(ct), ptr(st), ptr(kt2), ptr(vt2), max_seq, ptr(pos),
                                                 ranks, 2, wide, off, stream()))
    for o in outs:
        assert torch.equal(o[:, off:off + dim], ref)
        assert bool((o[:, :off] == 7.0).all()) and bool((o[:, off + dim:] == 7.0).all())
    assert torch.equal(kt2, kt) and torch.equal(vt2, vt)
    assert sgq.lib.sgqd_attn_decode_allgather(ptr(qkv), 3 * dim, B, H, hd, ptr(ct), ptr(st), ptr(kt2), ptr(vt2), max_seq, ptr(pos),
                                              ranks, 9, wide, off, stream()) == 3
    assert sgq.lib.sgqd_attn_decode_allgather(ptr(qkv), 3 * dim, B, H, hd, ptr(ct), ptr(st), ptr(kt2), ptr(vt2), max_seq, ptr(pos),
                                              ranks, 2, dim, off, stream()) == 2
    rows, hidden = 5, 704
    gu = dev(r.standard_normal((rows, 2 * hidden)).astype(np.float32))
    plain = torch.empty(rows, hidden, device="cuda")
    sgq.check(sgq.lib.sgqd_silu_mul(ptr(gu), rows, hidden, ptr(plain), None, 0, stream()))
    outs = [torch.full((rows, 3 * hidden), 7.0, device="cuda") for _ in range(2)]
    ranks = (C.c_void_p * 2)(*[o.data_ptr() for o in outs])
    sgq.check(sgq.lib.sgqd_silu_mul_allgather(ptr(gu), rows, hidden, ranks, 2, 3 * hidden, 2 * hidden, stream()))
    for o in outs:
        assert torch.equal(o[:, 2 * hidden:], plain)
        assert bool((o[:, :2 * hidden] == 7.0).all())
    assert sgq.lib.sgqd_silu_mul_allgather(ptr(gu), rows, hidden, ranks, 2, hidden, 2 * hidden, stream()) == 2


def test_attn_decode_position_out_of_range_stores_nothing(sgq):
    B, H, hd, max_seq = 2, 2, 128, 16
    r = np.random.default_rng(5)
    qkv, kc, vc = (dev(r.standard_normal(s).astype(np.float32)) for s in ((B, 3 * H * hd), (B, H, max_seq, hd), (B, H, max_seq, hd)))
    cos, sin = (dev(t) for t in no.rope_tables(hd, max_seq))
    k0, v0 = kc.clone(), vc.clone()
    out = torch.empty(B, H * hd, device="cuda")
    pos = torch.tensor([max_seq], dtype=torch.int32, device="cuda")
    sgq.check(sgq.lib.sgqd_attn_decode(ptr(qkv), 3 * H * hd, B, H, hd, ptr(cos), ptr(sin), ptr(kc), ptr(vc), max_seq, ptr(pos), ptr(out),
                                       H * hd, None, 0, stream()))
    torch.cuda.synchronize()
    assert torch.equal(kc, k0) and torch.equal(vc, v0) and torch.isfinite(out).all()


@pytest.mark.parametrize("B,H,hd,T,pos0", [(2, 3, 128, 70, 0), (1, 2, 64, 33, 0), (2, 2, 128, 5, 41), (1, 1, 128, 130, 7)])
def test_attn_prefill(sgq, B, H, hd, T, pos0):
    """Causal attention of a block of new tokens at positions pos0 .. pos0 + T - 1 over a cache that already holds
    them (and pos0 older entries), against the float64 oracle."""
    max_seq = pos0 + T + 3
    r = np.random.default_rng(T * 7 + hd + pos0)
    dim = H * hd
    qkv = r.standard_normal((B * T, 3 * dim)).astype(np.float32)
    kc = (r.standard_normal((B, H, max_seq, hd)) * 1.2).astype(np.float32)
    vc = r.standard_normal((B, H, max_seq, hd)).astype(np.float32)
    out = torch.full((B * T, dim), float("nan"), device="cuda")
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    qt, kt, vt = dev(qkv), dev(kc), dev(vc)
    sgq.check(sgq.lib.sgqd_attn_prefill(ptr(qt), 3 * dim, B, T, H, hd, ptr(kt), ptr(vt), max_seq, ptr(pos), ptr(out), dim, stream()))
    q = qkv[:, :dim].reshape(B, T, H, hd).transpose(0, 2, 1, 3).astype(np.float64)              # [B, H, T, hd]
    S = pos0 + T
    k, v = kc[:, :, :S].astype(np.float64), vc[:, :, :S].astype(np.float64)
    scores = np.einsum("bhtd,bhsd->bhts", q, k) / np.sqrt(hd)
    mask = np.arange(S)[None, :] > (pos0 + np.arange(T))[:, None]
    scores = np.where(mask, -np.inf, scores)
    want = np.einsum("bhts,bhsd->bhtd", no.softmax(scores), v).transpose(0, 2, 1, 3).reshape(B * T, dim)
    assert norm_err(out.cpu().numpy(), want) <= 5e-6
    if hd == 128:       # the tensor-core form of the same attention: operands and weights in bf16, fp32 accumulation and softmax
        out16 = torch.full((B * T, dim), float("nan"), device="cuda")
        sgq.check(sgq.lib.sgqd_attn_prefill_bf16(ptr(qt), 3 * dim, B, T, H, hd, ptr(kt), ptr(vt), max_seq, ptr(pos), ptr(out16), dim, stream()))
        got = out16.cpu().numpy()
        assert np.isfinite(got).all()
        assert norm_err(got, want) <= 2e-2, norm_err(got, want)
    else:
        assert sgq.lib.sgqd_attn_prefill_bf16(ptr(qt), 3 * dim, B, T, H, hd, ptr(kt), ptr(vt), max_seq, ptr(pos), ptr(out), dim, stream()) == 4


def test_embedding_lookup_and_out_of_range_ids(sgq):
    """Rows of the table by index; an id outside [0, vocab) gives zeros as the reference's lookup does."""
    vocab, dim = 37, 260
    r = np.random.default_rng(3)
    table = r.standard_normal((vocab, dim)).astype(np.float32)
    ids = np.array([0, 36, 5, -1, 37, 10 ** 12, 5, -(10 ** 12)], np.int64)
    out = torch.full((len(ids), dim), float("nan"), device="cuda")
    td, idd = dev(table), dev(ids, torch.int64)
    sgq.check(sgq.lib.sgqd_embedding(ptr(td), vocab, dim, ptr(idd), len(ids), ptr(out), stream()))
    want = np.where(((ids >= 0) & (ids < vocab))[:, None], table[np.clip(ids, 0, vocab - 1)], 0.0).astype(np.float32)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    odd = torch.full((2, 7), float("nan"), device="cuda")                   # a width that is not a multiple of 4
    t7 = dev(table[:, :7].copy())
    sgq.check(sgq.lib.sgqd_embedding(ptr(t7), vocab, 7, ptr(idd), 2, ptr(odd), stream()))
    np.testing.assert_array_equal(odd.cpu().numpy(), table[[0, 36], :7])


def test_argmax_rows_first_strict_maximum(sgq):
    """The reference's greedy choice: `if (p > best)` keeps the first of equal candidates."""
    r = np.random.default_rng(4)
    n = 32000
    x = r.standard_normal((6, n)).astype(np.float32)
    x[1, 700] = x[1, 31000] = 9.0                                           # a tie: the first index wins
    x[2, :] = -np.inf
    x[2, 123] = -1e30                                                       # everything else is -inf
    x[3, :] = 0.25                                                          # all equal -> 0
    x[4, 5] = np.nan
    x[4, 6] = 50.0                                                          # NaN never wins
    x[5, :] = -np.inf                                                       # nothing but -inf -> 0
    out = torch.full((6,), -7, dtype=torch.int64, device="cuda")
    xd = dev(x)
    sgq.check(sgq.lib.sgqd_argmax_rows(ptr(xd), 6, n, n, ptr(out), stream()))
    got = out.cpu().numpy()
    assert got.tolist() == [int(np.argmax(x[0])), 700, 123, 0, 6, 0]
    wide = dev(np.concatenate([x, x], axis=1))                              # row stride larger than the row
    sgq.check(sgq.lib.sgqd_argmax_rows(ptr(wide), 6, 100, 2 * n, ptr(out), stream()))
    assert out.cpu().numpy().tolist() == [int(np.nanargmax(x[i, :100])) if i not in (2, 3, 5) else 0 for i in range(6)]


# ---- the whole model ------------------------------------------------------------------------------
def tiny_model(nl, port, *, prompt_len, n_new, prefill_path, seed=3, overlap=True, cfg=None, B=2):
    cfg = cfg or nl.NanoLlamaConfig(dim=256, n_layers=2, n_heads=2, hidden=512, vocab=512, max_seq=64)
    r = np.random.default_rng(seed)
    floats = {}

    def init(name, layer):
        out_f, in_f = nl.weight_shape(cfg, name)
        std = 1.0 if name == "embed" else 2.5 * (2.0 / (in_f + out_f)) ** 0.5     # livelier logits than the default init
        w = (r.standard_normal((out_f, in_f)) * std).astype(np.float32)
        floats[(name, layer)] = w
        return torch.from_numpy(w)

    model = nl.NanoLlamaInt4(cfg, "cuda", B, init=init, prefill_path=prefill_path, overlap=overlap)
    prompt = torch.from_numpy(r.integers(0, cfg.vocab, (B, prompt_len)))
    tokens, logits = model.generate(prompt, n_new, use_graph=False, keep_logits=True)

    def deq(name, layer):
        w = floats[(name, layer)]
        packed, scales = port.quantize_int4(w, 32)
        return port.dequantize_int4(packed, scales, w.shape, 32)

    params = {"embed": floats[("embed", -1)], "n_heads": cfg.n_heads, "rope_base": cfg.rope_base, "eps": cfg.eps,
              "final_norm": np.ones(cfg.dim), "lm_head": deq("lm_head", -1),
              "layers": [dict({n: deq(n, li) for n in nl.LAYER_WEIGHTS}, attn_norm=np.ones(cfg.dim), ffn_norm=np.ones(cfg.dim))
                         for li in range(cfg.n_layers)]}
    seq = np.concatenate([prompt.numpy(), tokens.cpu().numpy()], axis=1)
    want = no.forward_full(params, seq[:, :-1])                  # logits at every position of the final sequence
    return model, prompt, tokens.cpu().numpy(), [l.cpu().numpy() for l in logits], want


# The bf16 prefill rounds activations and dequantized weights to 8 mantissa bits in each of the eight
# chained linears; at this model's K = 256..512 a single such linear already needs the small-K bound
# of the linear tests (4 x TOL_BF16), and that is what the chain is held to.
@pytest.mark.parametrize("prompt_len,n_new,prefill,tol", [(9, 6, "simt", TOL_FP32), (32, 5, "tc_bf16", 4 * TOL_BF16)])
def test_greedy_decode_matches_full_recompute(sgq, nl, port, prompt_len, n_new, prefill, tol):
    path = {"simt": sgq.PATH_SIMT, "tc_bf16": sgq.PATH_TC_BF16}[prefill]
    model, prompt, tokens, logits, want = tiny_model(nl, port, prompt_len=prompt_len, n_new=n_new, prefill_path=path)
    assert len(logits) == n_new
    for s in range(n_new):
        ref = want[:, prompt_len - 1 + s]
        assert norm_err(logits[s], ref) <= tol, f"step {s}"
        top2 = np.sort(ref, axis=-1)[:, -2:]
        decided = (top2[:, 1] - top2[:, 0]) > 4 * tol * np.max(np.abs(ref))
        assert (tokens[decided, s] == no.greedy(ref)[decided]).all(), f"token of step {s}"
    assert sgq.device_status() == 0


@pytest.mark.parametrize("prefill,tol", [("simt", TOL_FP32), ("tc_bf16", TOL_BF16)])
def test_greedy_decode_at_benchmark_dimensions(sgq, nl, port, prefill, tol):
    """The benchmarked model's own dimensions (dim 2048, 16 heads x 128, SwiGLU 5632, vocab 32000, batch 8)
    with one block and a short prompt, so that the full-recompute numpy oracle stays affordable: every
    step's logits within 1e-3 (fp32 prefill) / 2e-2 (bf16 tensor-core prefill) of the oracle."""
    cfg = nl.NanoLlamaConfig(dim=2048, n_layers=1, n_heads=16, hidden=5632, vocab=32000, max_seq=32)
    path = {"simt": sgq.PATH_SIMT, "tc_bf16": sgq.PATH_TC_BF16}[prefill]
    prompt_len, n_new = 8, 3                                   # 8 sequences x 8 tokens = 64 rows: the tensor-core path's minimum
    model, prompt, tokens, logits, want = tiny_model(nl, port, prompt_len=prompt_len, n_new=n_new, prefill_path=path, seed=5,
                                                      cfg=cfg, B=8)
    for s in range(n_new):
        ref = want[:, prompt_len - 1 + s]
        assert norm_err(logits[s], ref) <= tol, (f"step {s}", norm_err(logits[s], ref))
        top2 = np.sort(ref, axis=-1)[:, -2:]
        decided = (top2[:, 1] - top2[:, 0]) > 4 * tol * np.max(np.abs(ref))
        assert (tokens[decided, s] == no.greedy(ref)[decided]).all(), f"token of step {s}"
    assert sgq.device_status() == 0
    del model
    torch.cuda.empty_cache()


def test_overlapped_launches_agree_with_serial_ones(sgq, nl, port):
    """Programmatic dependent launch on (the default of the model) and off: the same bits; with the
    two-CTAs-per-SM form of the decode kernel (mode 2): same tokens, logits equal up to fp32 summation
    order (that form adds its partial sums in a different order)."""
    _, _, tok_on, log_on, _ = tiny_model(nl, port, prompt_len=9, n_new=6, prefill_path=sgq.PATH_SIMT, overlap=1)
    _, _, tok_off, log_off, _ = tiny_model(nl, port, prompt_len=9, n_new=6, prefill_path=sgq.PATH_SIMT, overlap=0)
    _, _, tok_two, log_two, _ = tiny_model(nl, port, prompt_len=9, n_new=6, prefill_path=sgq.PATH_SIMT, overlap=2)
    np.testing.assert_array_equal(tok_on, tok_off)
    np.testing.assert_array_equal(tok_two, tok_off)
    for a, b, c in zip(log_on, log_off, log_two):
        np.testing.assert_array_equal(a, b)
        assert norm_err(c, b) <= 2e-5
    assert sgq.device_status() == 0


@pytest.mark.parametrize("M,K", [(1, 4096), (4, 4096), (8, 2048), (16, 2048), (8, 5632), (3, 256)])
def test_overlap_switch_on_back_to_back_linears(sgq, M, K):
    """A chain of decode forwards whose inputs are the previous outputs, with and without overlap
    (overlapped launches use the two-CTAs-per-SM form of the decode kernel)."""
    g = torch.Generator(device="cuda").manual_seed(11 + M)
    qs = [sgq.quantize_int4(torch.randn(K, K, device="cuda", generator=g) * (1.5 / K ** 0.5), 32) for _ in range(4)]
    x0 = torch.randn(M, K, device="cuda", generator=g)
    torch.cuda.synchronize()

    def chain(keep=None):
        x, ws = x0, sgq.Workspace(x0.device)
        for _ in range(3):
            for q in qs:
                if keep is not None:
                    keep.append(x)
                x = sgq.quantized_matmul(x, q, None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws)
        return x

    prev = sgq.set_stream_overlap(False)
    try:
        inputs = []
        want = chain(inputs)
        outputs = inputs[1:] + [want]
        sgq.set_stream_overlap(1)
        assert torch.equal(chain(), want)                                 # overlapped launches alone change no bit
        sgq.set_stream_overlap(2)                                         # ... the two-CTAs-per-SM form changes the summation order
        got = chain()
        again = chain()
        ws = sgq.Workspace(x0.device)      # every layer on the serial run's input, launched back to back
        singles = [sgq.quantized_matmul(x, qs[i % 4], None, layout=sgq.LAYOUT_NK, path=sgq.PATH_GEMV, workspace=ws)
                   for i, x in enumerate(inputs)]
    finally:
        sgq.set_stream_overlap(prev)
    assert torch.equal(again, got)                                        # run to run: bit-identical
    for y, ref in zip(singles, outputs):                                  # same digits, another order of fp32 partial sums
        assert norm_err(y.cpu().numpy(), ref.cpu().numpy()) <= 2e-5
    assert norm_err(got.cpu().numpy(), want.cpu().numpy()) <= 2e-3        # twelve chained layers amplify that rounding
    assert sgq.device_status() == 0


def test_graph_replay_equals_eager(sgq, nl, port):
    model, prompt, tokens, _, _ = tiny_model(nl, port, prompt_len=9, n_new=6, prefill_path=sgq.PATH_SIMT)
    again = model.generate(prompt, 6, use_graph=True).cpu().numpy()
    np.testing.assert_array_equal(again, tokens)
    third = model.generate(prompt, 6, use_graph=True).cpu().numpy()          # the recorded graph is reused
    np.testing.assert_array_equal(third, tokens)
    assert model.launches_per_decode_step > 0
