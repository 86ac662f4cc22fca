/* sgq.h — C ABI of the B200 (sm_100a) SovereignGrad quantization hot path.
 *
 * Drop-in boundary: each entry point replaces one function of the reference's
 * `sovereigngrad::quantization` namespace (file:line of what it replaces is given per
 * function; paths are relative to the reference checkout).  Plain pointers and sizes only.
 *
 * Conventions
 *  - Every data pointer is a DEVICE pointer owned by the caller; the library allocates no
 *    device memory.  Scratch, where a function needs it, is the caller's `workspace`.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream, which is what
 *    the reference uses throughout).  Calls are asynchronous: they enqueue work and return.
 *  - Return value: sgq_status (0 = ok).  Nothing throws, aborts or synchronises the device.
 *    `sgq_last_error()` gives a thread-local detail string for the last non-zero status.
 *  - Entry points are re-entrant; concurrent calls must not share output or workspace buffers.
 *
 * Data layout (the reference keeps integer codes in an fp32 tensor,
 * src/quantization.cpp:32-38,127-153, and defines no bytes; this is the packed form):
 *  - INT8 codes: one two's-complement int8 per element, flat row-major order.
 *  - INT4 codes: two two's-complement nibbles per byte, element 2i in the LOW nibble and
 *    element 2i+1 in the HIGH nibble, flat row-major order, ceil(numel/2) bytes; the high
 *    nibble of an odd tail byte is 0.
 *  - scales: fp32, in the reference's order — [1] per tensor, [rows] per row of the stored
 *    tensor, [ceil(numel/group)] for INT4 where group g covers flat elements
 *    [g*group, min(numel,(g+1)*group)).
 *  - weight `layout`: SGQ_LAYOUT_KN = stored as [K=in, N=out], y = x*W (the reference module's
 *    native form, include/sovereigngrad/nn.hpp:935-958); SGQ_LAYOUT_NK = stored as [N, K],
 *    y = x*W^T.  Because INT4 groups run over the flat index they lie along N for KN and
 *    along K for NK.
 */
#ifndef SGQ_H
#define SGQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGQ_ABI_VERSION 1

#if defined(__GNUC__)
#define SGQ_API __attribute__((visibility("default")))
#else
#define SGQ_API
#endif

typedef enum sgq_status {
    SGQ_OK = 0,
    SGQ_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
    SGQ_ERR_BAD_SHAPE = 2,      /* negative size, inner dimensions that do not match, ldy < N */
    SGQ_ERR_BAD_ARGUMENT = 3,   /* unknown layout / scheme / path value */
    SGQ_ERR_UNSUPPORTED = 4,    /* the requested `path` cannot run this shape (never silently rerouted) */
    SGQ_ERR_WORKSPACE = 5,      /* workspace missing, too small or not 256-byte aligned */
    SGQ_ERR_ALIGNMENT = 6,      /* a pointer breaks the alignment the requested path needs */
    SGQ_ERR_CUDA = 7,           /* a CUDA call or launch failed; see sgq_last_error() */
    SGQ_ERR_DEVICE = 8,         /* current device is not compute capability 10.x */
    SGQ_ERR_TIMEOUT = 9         /* a bounded device-side wait gave up (read back from the status word) */
} sgq_status;

enum { SGQ_LAYOUT_KN = 0, SGQ_LAYOUT_NK = 1 };
enum { SGQ_PER_TENSOR = 0, SGQ_PER_ROW = 1 };

/* Which kernel family runs a forward.  AUTO picks by shape; the others force one family and
 * return SGQ_ERR_UNSUPPORTED when it cannot take the shape. */
enum {
    SGQ_PATH_AUTO = 0,
    SGQ_PATH_SIMT = 1,    /* tiled fp32 SIMT kernel, any shape; one fused-multiply-add chain per
                             output in ascending k, i.e. the reference CPU rounding */
    SGQ_PATH_GEMV = 2,    /* decode (M <= 16): weight-streaming kernels.  [N,K] (INT4 g=32, INT8): exact integer
                             tensor-core dot products of the codes with fixed-point activations (24 bits below the
                             absmax of every 32 k of a row; from three rows on the last 8 bits only where one value
                             dominates its 32), fp32 scaling and accumulation; any activation distribution stays
                             within ~1e-4 of the reference's fp32 forward (bound 1e-3); a row with a
                             NaN or Inf activation yields a NaN output row.  [K,N] (the reference module's layout):
                             fp32 throughout */
    SGQ_PATH_TC_BF16 = 3, /* prefill: tcgen05 kind::f16 on bf16 activations and bf16 weights (INT4 with any group that is a
                             multiple of 8, or INT8; K % 64 == 0).
                             With the scratch sgq_linear_workspace_bytes() asks for, a launch in front expands the weight
                             to bf16 [N,K] (INT4: code * scale in fp32, rounded once; INT8 stored [N,K]: the exact codes,
                             scale applied in fp32 afterwards) and both operands reach the tensor cores by TMA; weights
                             stored [K,N] (N % 32 == 0) are transposed by that launch.  For weights stored [N,K] and
                             with sgq_set_stream_overlap on, the GEMM starts while that launch is still running: the
                             expansion goes slice of K by slice of K and counts finished slices in the last 256 bytes of
                             the scratch, which the GEMM's loads wait on (bounded).  With scratch for the activations
                             only (M * K * 2 bytes, rounded up to 256), INT4 g=32 and INT8 weights stored [N,K] are dequantized tile by tile in
                             shared memory instead (slower).  Bound 2e-2 of the largest output. */
    SGQ_PATH_TC_I8 = 4    /* prefill, INT8 weights only: activations quantized per row, tcgen05 kind::i8 */
};

SGQ_API const char* sgq_status_string(int status);
SGQ_API const char* sgq_last_error(void);
SGQ_API int sgq_abi_version(void);

/* Overlap of consecutive kernels in a stream (programmatic dependent launch; process-wide switch,
 * off by default, returns the previous setting; no counterpart in the reference).  With 1, every
 * kernel of this library is launched so that it may start while the kernel before it in the same
 * stream is still finishing: its set-up, and for the decode kernel the first tiles of WEIGHTS and
 * SCALES, are fetched early; activations, workspaces and outputs are touched only after the
 * earlier kernel has completed, so results are the same bits as without overlap.  With 2 the INT4
 * decode kernel additionally runs as two smaller CTAs per SM, so that the next forward's CTA can sit
 * beside the running one; that form adds its fp32 partial sums in another order (results equal to
 * fp32 rounding, bit-identical run to run) and measured no faster than 1 on B200.  The one rule
 * the switch adds: a weight, scale or bias buffer must not be the output of the kernel launched
 * immediately before the linear that reads it in the same stream (quantize, then run something
 * else or synchronise, then multiply).  It pays in launch-bound sequences: a decode step is ~130
 * kernels of 3-17 us. */
SGQ_API int sgq_set_stream_overlap(int enabled);

/* Kernels that wait on hardware barriers (TMA / tensor-core pipelines) bound every wait; one that
 * runs out writes a code into a device status word instead of hanging.  This call SYNCHRONISES
 * with the device (a blocking copy), returns SGQ_ERR_TIMEOUT if the word is non-zero, stores it
 * in *word (may be NULL) and clears it when `clear` is non-zero.  Meant for tests and for error
 * paths, not for the hot loop.  No counterpart in the reference, whose launches are unchecked. */
SGQ_API int sgq_device_status(unsigned int* word, int clear);

/* ---- quantize / pack ---------------------------------------------------------------- */

/* Replaces quantization::quantize_int8 (src/quantization.cpp:11-78).
 * x: rows*cols fp32.  scheme SGQ_PER_TENSOR: absmax over everything, 1 scale (:22-41);
 * SGQ_PER_ROW: one scale per row (:42-75).  max_abs starts at 1e-8f, scale = max_abs/127,
 * code = clamp(round_half_away(x * (127/max_abs)), -127, 127).  Bit-exact with the reference.
 * Per tensor, scales[0] transiently holds the running absmax while the call executes. */
SGQ_API int sgq_quantize_int8(const float* x, int64_t rows, int64_t cols, int scheme, int8_t* codes, float* scales,
                      void* stream);

/* Replaces quantization::quantize_int4 (src/quantization.cpp:113-159).  group <= 0 means 32
 * (:118).  scale = max_abs/7, code = clamp(round_half_away(x * (7/max_abs)), -8, 7), packed two
 * per byte.  packed: ceil(numel/2) bytes; scales: ceil(numel/group) floats.  Bit-exact. */
SGQ_API int sgq_quantize_int4(const float* x, int64_t numel, int64_t group, uint8_t* packed, float* scales, void* stream);

/* Replaces quantization::dequantize_int8 (src/quantization.cpp:80-111): out = code * scale. */
SGQ_API int sgq_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme, float* out,
                        void* stream);
/* Replaces quantization::dequantize_int4 (src/quantization.cpp:161-187). */
SGQ_API int sgq_dequantize_int4(const uint8_t* packed, const float* scales, int64_t numel, int64_t group, float* out,
                        void* stream);

/* The reference's `QuantizedTensor::qdata` view (include/sovereigngrad/quantization.hpp:18):
 * integer codes held as fp32, and back.  Used to exchange tensors with reference checkpoints,
 * which store qdata as fp32 (src/module.cpp:94-112). */
SGQ_API int sgq_codes_to_f32_int8(const int8_t* codes, int64_t numel, float* out, void* stream);
SGQ_API int sgq_codes_to_f32_int4(const uint8_t* packed, int64_t numel, float* out, void* stream);
SGQ_API int sgq_codes_from_f32_int8(const float* codes_f32, int64_t numel, int8_t* codes, void* stream);
SGQ_API int sgq_codes_from_f32_int4(const float* codes_f32, int64_t numel, uint8_t* packed, void* stream);

/* ---- forward -------------------------------------------------------------------------- */

/* Bytes of scratch the forward wants for this shape and path (0 = none).  bits is 4 or 8.  With SGQ_PATH_AUTO:
 * enough for whichever path AUTO takes - the decode kernels up to 16 rows, blocks of 16 rows on the decode kernels
 * up to 63 rows (the blocks share the scratch), the tensor-core path from 64 rows on. */
SGQ_API size_t sgq_linear_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int path);

/* Replaces quantization::quantized_matmul_int4 (src/quantization.cpp:199-206), i.e.
 * dequantize_int4 + matmul (src/ops.cpp:378-455) + broadcast add (src/ops.cpp:132-171) in one
 * launch: y[m, n] = sum_k x[m,k] * code(k,n) * scale(k,n) + bias[n].
 * x: [M,K] fp32 row-major.  y: [M,N] fp32 with row stride ldy >= N (ldy lets a rank write its
 * column slice into a wider buffer).  bias: N floats or NULL (= the reference's undefined
 * bias, :202).  workspace: NULL or >= sgq_linear_workspace_bytes(...) bytes, 256-byte aligned. */
SGQ_API int sgq_linear_int4(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed, const float* scales,
                    int layout, int64_t group, const float* bias, float* y, int64_t ldy, int path, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Replaces quantization::quantized_matmul_int8 (src/quantization.cpp:189-197).  scheme
 * SGQ_PER_ROW scales follow the rows of the STORED tensor: index k for KN, n for NK. */
SGQ_API int sgq_linear_int8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                    int layout, int scheme, const float* bias, float* y, int64_t ldy, int path, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Gradient with respect to the activations of a frozen quantized layer.  The reference attaches a
 * MatmulNode when x requires a gradient (src/ops.cpp:451-453), so it can backpropagate through
 * quantized_matmul_int4 / _int8 (src/quantization.cpp:189-206) into x; its backward is
 * grad_output.matmul(deq(W)^T contiguous) (src/ops.cpp:367-370).  These entry points compute the same:
 *   layout KN (y = x * W):    dx[m,k] = sum_n dy[m,n] * code(k,n) * scale(k,n)
 *   layout NK (y = x * W^T):  dx[m,k] = sum_n dy[m,n] * code(n,k) * scale(n,k)
 * dy: [M,N] fp32 row-major, dx: [M,K] with row stride ldx >= K; packed/codes/scales, group and scheme
 * are the forward's own.  It is the forward of the same stored tensor read with the other layout flag,
 * so every path of the forward is available (SGQ_PATH_SIMT reproduces the reference's fp32 chain;
 * workspace as sgq_linear_backward_x_workspace_bytes says).  Weights get no gradient: they are codes. */
SGQ_API int sgq_linear_int4_backward_x(const float* dy, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                                       const float* scales, int layout, int64_t group, float* dx, int64_t ldx, int path,
                                       void* workspace, size_t workspace_bytes, void* stream);
SGQ_API int sgq_linear_int8_backward_x(const float* dy, int64_t M, int64_t K, int64_t N, const int8_t* codes,
                                       const float* scales, int layout, int scheme, float* dx, int64_t ldx, int path,
                                       void* workspace, size_t workspace_bytes, void* stream);
SGQ_API size_t sgq_linear_backward_x_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int path);

/* Dynamic quantization of activations: one scale per row (token) of x[M,K], the reference's per-channel
 * quantizer applied to x (src/quantization.cpp:42-75): sx[m] = max(|x[m,:]|, 1e-8) / 127,
 * xq = clamp(round_half_away(x * (127 / max)), -127, 127).  Bit-exact with the reference.  The same
 * codes feed sgq_linear_w8a8. */
SGQ_API int sgq_quantize_activations_int8(const float* x, int64_t M, int64_t K, int8_t* xq, float* sx, void* stream);

/* Prepared activations: the decode kernel's own operand format (int8 digit planes of the
 * activations with one power-of-two scale per row).  (No counterpart in the reference.)  A decode
 * forward normally converts x on the fly; a caller that runs several linears on the same x, or
 * whose previous operator can emit the format directly (sgq_decoder.h), converts once and calls
 * sgq_linear_int4_prepared, which computes exactly what sgq_linear_int4(..., SGQ_LAYOUT_NK,
 * group 32, SGQ_PATH_GEMV) computes for that x.  The format is opaque, depends on (M, K) and is
 * only valid for the library build that wrote it.
 *   sgq_prepared_x_bytes  bytes of the prepared form of x[M, K]; 0 when there is none (it needs
 *                         1 <= M <= 16 and K % 256 == 0)
 *   sgq_prepare_x         x[M, K] fp32 (16-byte aligned) -> prepared (256-byte aligned) */
SGQ_API size_t sgq_prepared_x_bytes(int64_t M, int64_t K);
SGQ_API int sgq_prepare_x(const float* x, int64_t M, int64_t K, void* prepared, size_t prepared_bytes, void* stream);
SGQ_API int sgq_linear_int4_prepared(const void* prepared, size_t prepared_bytes, int64_t M, int64_t K, int64_t N,
                                     const uint8_t* packed, const float* scales, const float* bias, float* y,
                                     int64_t ldy, void* stream);

/* Fused all-gather for a decode forward whose output features are split over the GPUs of one box
 * (rank q owns rows [n_offset, n_offset + N_local) of the [N_total, K] weight).  (No counterpart in
 * the reference, which is single-device.)  The decode kernel stores its [M, N_local] slice straight
 * into the full-width output y_ranks[r][m * ldy + n_offset + n] of EVERY rank r (plain peer stores
 * over NVLink; y_ranks is a HOST array of `world` device pointers, entry `rank` being this GPU's own
 * buffer, the others peer-mapped).  Same shapes as SGQ_PATH_GEMV (M <= 16, INT4 g=32, [N,K]).
 * The outputs are whole once every rank has passed a barrier: either pass `signals`, `rank` and
 * `local_state` (as for sgq_peer_barrier below; local_state = 16 zero-initialised bytes of this GPU's
 * memory, 8-byte aligned, shared by all calls that use the same signals) and the barrier runs in the
 * tail of the kernel itself, or pass signals = NULL and call sgq_peer_barrier afterwards.  Alternate
 * between two sets of output buffers from one forward to the next: a rank that runs ahead then
 * writes the other set while a slower rank still reads this one.
 * Prefill-sized batches (M >= 64, K % 64 == 0, workspace of sgq_linear_workspace_bytes(4, M, K, N_local,
 * SGQ_LAYOUT_NK, SGQ_PATH_TC_BF16) bytes) take the tcgen05 GEMM of SGQ_PATH_TC_BF16 instead, whose epilogue
 * stores every output tile into all ranks' outputs in the same way (bound 2e-2, bit-equal to the single-GPU
 * result of that path); with `signals` the barrier kernel is launched behind the GEMM by this call. */
SGQ_API int sgq_linear_int4_allgather(const float* x, int64_t M, int64_t K, int64_t N_local, const uint8_t* packed,
                                      const float* scales, const float* bias, float* const* y_ranks, int world,
                                      int64_t ldy, int64_t n_offset, void* workspace, size_t workspace_bytes,
                                      void* const* signals, int rank, void* local_state, void* stream);

/* The same forward with the wait taken out of the producer.  The kernel stores its slices into every
 * rank's output and only SIGNALS: every thread block, when its own slices are out, adds one to this
 * rank's slot on every rank (a system-scope release reduction: no separate fence, no election of a
 * last block), so the slots count arrivals and local_state counts what this rank has sent; it does
 * not wait for the other ranks.  (Every rank must therefore run the same sequence of launches on the
 * same signals, as for the barrier.)  Instead every kernel launched through this entry point first waits, in its
 * prologue, until all ranks have signalled the exchanges this GPU has already finished — one NVLink
 * round trip that overlaps the kernel's own start-up and weight prefetch, and no extra launch.
 * Consequences for the caller:
 *  - the outputs of call i are whole on this GPU once a LATER call on the same signals (this entry
 *    point or sgq_peer_barrier) has been enqueued behind it and has run; end a sequence with
 *    sgq_peer_barrier before reading the last outputs;
 *  - as with the other form, alternate between two sets of output buffers;
 *  - signals, rank and local_state are required (same objects as for sgq_peer_barrier);
 *  - decode batches only (M <= 16): SGQ_ERR_UNSUPPORTED for the prefill-sized batches of the other form. */
SGQ_API int sgq_linear_int4_allgather_deferred(const float* x, int64_t M, int64_t K, int64_t N_local, const uint8_t* packed,
                                               const float* scales, const float* bias, float* const* y_ranks, int world,
                                               int64_t ldy, int64_t n_offset, void* workspace, size_t workspace_bytes,
                                               void* const* signals, int rank, void* local_state, void* stream);

/* The same exchange for a slice that some other kernel produced: src[M, n_local] (this GPU) is
 * stored into y_ranks[r][m * ldy + n_offset + n] of every rank r.  Follow with sgq_peer_barrier. */
SGQ_API int sgq_peer_scatter(const float* src, int64_t M, int64_t n_local, float* const* y_ranks, int world, int64_t ldy,
                             int64_t n_offset, void* stream);

/* Barrier between the GPUs of one box, in stream order, no host involvement.  signals: HOST array of
 * `world` device pointers, signals[r] = rank r's array of `world` 64-bit slots (zero-initialised,
 * writable by every rank: symmetric / peer-mapped memory).  local_epoch: one zero-initialised 64-bit
 * counter in this GPU's own memory.  Every rank must call it the same number of times.  All peer
 * stores this GPU issued before the barrier are visible on their targets once the targets' barriers
 * return.  The wait is bounded (about half a second by default, see
 * sgq_set_peer_wait_budget): if a rank never arrives the kernel gives up, returns, and
 * sgq_device_status() reports SGQ_ERR_TIMEOUT; the outputs of that exchange are then incomplete and
 * must not be used. */
SGQ_API int sgq_peer_barrier(void* const* signals, int rank, int world, void* local_epoch, void* stream);

/* Number of polls a device-side wait for another GPU spends before it gives up (process-wide, applies
 * to launches made afterwards; returns the previous value; no counterpart in the reference).  A poll
 * costs 0.1-0.4 us once a wait has lasted more than a few microseconds; the default 2^21 is about half
 * a second.  Smaller values make a missing rank show up sooner (and let a test make a wait run out). */
SGQ_API unsigned int sgq_set_peer_wait_budget(unsigned int polls);

/* Decode forward for callers that cannot allocate device memory.  (No counterpart in the
 * reference: there every call allocates its temporaries through MemoryAllocator.)
 *
 * Who needs it: code that runs inside someone else's memory budget — a plugin whose host owns all
 * device allocations, a process whose pool was sized and frozen at start-up, a token loop that
 * must stay clear of the allocator and its locks.  Such callers can pass inputs and outputs they
 * already own, but have nowhere to get the scratch that sgq_linear_int4 wants for batches of
 * more than 4 rows (the activation planes of the decode kernel).
 *
 * Same computation and results as sgq_linear_int4(..., SGQ_LAYOUT_NK, group 32, SGQ_PATH_GEMV),
 * but the scratch is a fixed array inside the library's device image: 448 KiB on every GPU that
 * loads the library, held until the process exits.  Limits and rules:
 *  - shapes the decode kernel takes (M <= 16, K % 256 == 0, 16-byte aligned x/packed/scales) whose
 *    prepared activations, sgq_prepared_x_bytes(M, K), are at most 448 KiB (e.g. K = 8192 at
 *    M = 16); anything larger returns SGQ_ERR_WORKSPACE;
 *  - the first call on each device looks up the array's device address (a runtime query, no
 *    allocation); make that first call outside any stream capture;
 *  - all calls on a device share the one array, whose contents are simply overwritten by the next
 *    call: two calls that may overlap on the GPU (different streams, no ordering) race.  Nothing
 *    in it has to be cleared between calls;
 *  - no cudaMalloc, cudaFree or other allocating routine is called. */
SGQ_API int sgq_linear_int4_decode_noalloc(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                                           const float* scales, const float* bias, float* y, int64_t ldy, void* stream);

/* Integer sub-path behind SGQ_PATH_TC_I8, exposed so its exact parts can be checked: x is
 * quantized per row with the rule of sgq_quantize_int8(SGQ_PER_ROW) into xq/sx, acc is the exact
 * int32 product of the codes, y = ((float)acc * sx[m]) * sw + bias.  xq_out [M,K], sx_out [M]
 * and acc_out [M,N] may each be NULL (then they live in the workspace, or are not materialised).
 * The reference has no counterpart: it never quantizes activations.  Layout must be NK. */
SGQ_API int sgq_linear_w8a8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                    int scheme, const float* bias, float* y, int64_t ldy, int8_t* xq_out, float* sx_out,
                    int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream);
SGQ_API size_t sgq_linear_w8a8_workspace_bytes(int64_t M, int64_t K, int64_t N);

/* Copies column slices gathered rank-major, src[r][m][n_local] (the order an all-gather leaves
 * them in), into row-major dst[m][r*n_local + n_local...] with row stride ldd. */
SGQ_API int sgq_interleave_slices(const float* src, int64_t world, int64_t M, int64_t n_local, float* dst, int64_t ldd,
                          void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SGQ_H */
