/*
 * sgq_decoder.h — the fp32 operators that sit between the quantized linears of a LLaMA-style
 * decoder block (RMSNorm, rotary embedding + KV-cache store, single-query attention over the
 * cache, SiLU gate), exported from the same library as sgq.h.
 *
 * They exist so that a whole greedy-decode step (sixteen blocks, ~200 launches) can be recorded
 * into one CUDA graph and replayed without host work: every quantity that changes from step to
 * step (the position in the cache) is read from DEVICE memory, so the recorded launches stay valid.
 * Arithmetic is fp32 throughout and follows the reference's operators:
 *
 *   sgqd_add_rmsnorm     sovereigngrad::rms_norm            src/ops.cpp:1532-1564
 *   sgqd_rope_kv_store   sovereigngrad::rotary_embedding    src/ops.cpp:1714-1745
 *                        nn::RotaryEmbedding tables         include/sovereigngrad/nn.hpp:583-607
 *   sgqd_attn_decode     nn::CausalSelfAttention            include/sovereigngrad/nn.hpp:503-560
 *                        (last row of the causal softmax(q k^T / sqrt(d)) v; the reference has no
 *                        KV cache and recomputes every row, models.hpp:262-300) + rotary_embedding
 *   sgqd_attn_prefill    causal attention with online softmax  src/cuda_kernels.cu:1323-1394
 *   sgqd_silu_mul        nn::SwiGLU gate                    include/sovereigngrad/nn.hpp:151-156
 *                        simd::vec_silu                     include/sovereigngrad/simd.hpp:103-108
 *   sgqd_embedding       sovereigngrad::embedding           src/ops.cpp:2624-2659
 *   sgqd_argmax_rows     greedy choice in NanoLLaMA::generate  include/sovereigngrad/models.hpp:291-298
 *
 * Conventions are those of sgq.h: device pointers owned by the caller, `stream` is a cudaStream_t
 * passed as void*, calls enqueue and return an sgq_status, nothing is allocated.
 */
#ifndef SGQ_DECODER_H
#define SGQ_DECODER_H

#include "sgq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* h[rows, dim] += delta (skipped when delta is NULL), then out = h * rsqrt(mean(h^2) + eps) * gamma.
 * h is updated in place: it is the residual stream.  out may not alias h.
 * prepared_out (optional, NULL to skip): also writes out in the prepared-activation format of
 * sgq.h (sgq_prepared_x_bytes(rows, dim) bytes, 256-byte aligned) for sgq_linear_int4_prepared. */
SGQ_API int sgqd_add_rmsnorm(float* h, const float* delta, const float* gamma, float eps, int64_t rows, int64_t dim,
                             float* out, void* prepared_out, size_t prepared_bytes, void* stream);

/* qkv[batch * t_new, 3 * n_heads * head_dim] holds, per token, the query, key and value rows of
 * n_heads heads (token m = b * t_new + i is the i-th new token of sequence b, at position
 * *pos0 + i).  Rotates q in place, and stores the rotated k and the v of every new token into
 * k_cache / v_cache[batch, n_heads, max_seq, head_dim].  cos / sin are [max_seq, head_dim / 2]
 * tables (pair (d, d + head_dim/2), angle pos * base^(-2d/head_dim)).  pos0 is a DEVICE int32:
 * the number of tokens already in the cache.  Tokens whose position would be >= max_seq are
 * skipped (nothing is written out of bounds).  head_dim must be a multiple of 8. */
SGQ_API int sgqd_rope_kv_store(float* qkv, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim,
                               const float* cos_table, const float* sin_table, const int32_t* pos0,
                               float* k_cache, float* v_cache, int64_t max_seq, void* stream);

/* One decode step of attention for one NEW token per sequence, fused with that token's rotary
 * embedding and cache append.  qkv[batch, qkv_stride] holds the un-rotated query, key and value of
 * the token at position *pos0 (same layout as above, t_new = 1; qkv is not modified).  The kernel
 * rotates q and k, appends k and v to the caches at position *pos0, and writes
 *   out[b, h*head_dim + d] = sum_{t <= pos0} softmax_t(q . k_t / sqrt(head_dim)) v_t[d].
 * Do not call sgqd_rope_kv_store for the same token.  If *pos0 is outside [0, max_seq) nothing is
 * stored and the query attends to the cache contents only.  head_dim must be 64 or 128.
 * prepared_out (optional, prepared_bytes >= sgq_prepared_x_bytes(batch, n_heads * head_dim)): the rows
 * out[b, 0 .. n_heads*head_dim) additionally in the decode kernel's prepared form, bit-identical to
 * sgq_prepare_x on `out`, so that the linear behind the attention (sgq_linear_int4_prepared) needs no
 * conversion launch. */
SGQ_API int sgqd_attn_decode(float* qkv, int64_t qkv_stride, int64_t batch, int64_t n_heads, int64_t head_dim,
                             const float* cos_table, const float* sin_table, float* k_cache, float* v_cache,
                             int64_t max_seq, const int32_t* pos0, float* out, int64_t out_stride, void* prepared_out,
                             size_t prepared_bytes, void* stream);

/* Causal attention of t_new NEW tokens per sequence (the prompt pass), after sgqd_rope_kv_store has rotated
 * q in place and appended the rotated keys and the values: token i of sequence b (row b * t_new + i of qkv,
 * position *pos0 + i) attends to cache positions 0 .. *pos0 + i,
 *   out[b * t_new + i, h*head_dim + d] = sum_{t <= pos0 + i} softmax_t(q . k_t / sqrt(head_dim)) v_t[d],
 * computed with an online softmax over tiles of 32 keys like the reference's attention
 * (src/cuda_kernels.cu:1323-1394).  head_dim must be 64 or 128; batch * n_heads <= 65535. */
SGQ_API int sgqd_attn_prefill(const float* qkv, int64_t qkv_stride, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim,
                              const float* k_cache, const float* v_cache, int64_t max_seq, const int32_t* pos0, float* out,
                              int64_t out_stride, void* stream);

/* The same attention on the tensor cores, for prompt passes whose linears run on the bf16 tensor-core path anyway
 * (SGQ_PATH_TC_BF16): q, k, v and the softmax weights are rounded to bf16, the products accumulate in fp32, the
 * softmax is fp32.  Within 2e-2 of the largest output of sgqd_attn_prefill (measured ~3e-3).  head_dim must be 128.
 * (No counterpart in the reference, whose attention is fp32.) */
SGQ_API int sgqd_attn_prefill_bf16(const float* qkv, int64_t qkv_stride, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim,
                              const float* k_cache, const float* v_cache, int64_t max_seq, const int32_t* pos0, float* out,
                              int64_t out_stride, void* stream);

/* gate_up[rows, 2 * hidden] = [gate | up] per row; out[rows, hidden] = gate / (1 + exp(-gate)) * up.
 * prepared_out: as for sgqd_add_rmsnorm, the prepared form of out[rows, hidden]. */
SGQ_API int sgqd_silu_mul(const float* gate_up, int64_t rows, int64_t hidden, float* out, void* prepared_out,
                          size_t prepared_bytes, void* stream);

/* Column-sharded forms of the two operators whose output is a column slice per GPU (the heads of this rank, the
 * SwiGLU columns of this rank): the result goes straight into the full-width buffer of EVERY rank,
 * out_ranks[r][row * stride + col_offset + c] (plain peer stores; out_ranks is a HOST array of `world` device
 * pointers, as for sgq_linear_int4_allgather), so no copy kernel stands between the operator and sgq_peer_barrier.
 * Otherwise as sgqd_attn_decode (without the prepared form) and sgqd_silu_mul. */
SGQ_API int sgqd_attn_decode_allgather(float* qkv, int64_t qkv_stride, int64_t batch, int64_t n_heads, int64_t head_dim,
                                       const float* cos_table, const float* sin_table, float* k_cache, float* v_cache,
                                       int64_t max_seq, const int32_t* pos0, float* const* out_ranks, int world,
                                       int64_t out_stride, int64_t col_offset, void* stream);
SGQ_API int sgqd_silu_mul_allgather(const float* gate_up, int64_t rows, int64_t hidden, float* const* out_ranks, int world,
                                    int64_t ld, int64_t col_offset, void* stream);

/* out[i, :] = table[ids[i], :] for rows indices (ids: DEVICE int64).  An id outside [0, vocab) gives a row
 * of zeros, as in the reference (src/ops.cpp:2643-2649); the table is never read out of bounds. */
SGQ_API int sgqd_embedding(const float* table, int64_t vocab, int64_t dim, const int64_t* ids, int64_t rows, float* out,
                           void* stream);

/* out[r] = first index of the strict maximum of x[r, 0..n) (row stride ld), a DEVICE int64 per row: the
 * reference's greedy choice keeps the first of equal candidates (models.hpp:291-298).  NaN never wins;
 * a row of NaNs (or n == 0) gives 0. */
SGQ_API int sgqd_argmax_rows(const float* x, int64_t rows, int64_t n, int64_t ld, int64_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SGQ_DECODER_H */
