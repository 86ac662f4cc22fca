// Quantize / pack / dequantize kernels (HBM-bound integer and byte work).
//
// Arithmetic is the reference's, bit for bit (src/quantization.cpp:22-75,113-159): running
// absmax from 1e-8f, scale = max/qmax and inv = qmax/max as two IEEE divisions, code =
// clamp(round_half_away(x * inv)).  No fast-math: `/` is div.rn, products are __fmul_rn.
#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {
namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------------------------------------
// INT4, group = 32, the hot case.  A lane owns 8 consecutive floats (two 128-bit loads, one
// 32-bit packed store); four neighbouring lanes own one group and share its absmax through
// two xor-shuffles.  A warp covers 256 contiguous floats (1 KiB) per step; UNROLL steps are
// loaded before the first is used so that several KiB per warp are in flight.
// Algorithmic bytes per element: 4 read + 0.5 + 0.125 written.
// ------------------------------------------------------------------------------------------
template <int UNROLL>
__global__ void __launch_bounds__(kThreads) quantize_int4_g32_kernel(const float4* __restrict__ x,
                                                                     uint32_t* __restrict__ packed,
                                                                     float* __restrict__ scales, int64_t n8) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
    for (int64_t base = warp * 32 * UNROLL; base < n8; base += nwarps * 32 * UNROLL) {
        float4 a[UNROLL], b[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int64_t i = base + u * 32 + lane;
            if (i < n8) {
                a[u] = __ldcs(x + 2 * i);
                b[u] = __ldcs(x + 2 * i + 1);
            } else {
                a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                b[u] = a[u];
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int64_t i = base + u * 32 + lane;
            float m = 1e-8f;
            m = absmax_step(m, a[u].x); m = absmax_step(m, a[u].y); m = absmax_step(m, a[u].z); m = absmax_step(m, a[u].w);
            m = absmax_step(m, b[u].x); m = absmax_step(m, b[u].y); m = absmax_step(m, b[u].z); m = absmax_step(m, b[u].w);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            const float inv = 7.0f / m;
            uint32_t w = 0;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(a[u].x, inv) & 0xF);
            w |= static_cast<uint32_t>(quantize_code<7, -8>(a[u].y, inv) & 0xF) << 4;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(a[u].z, inv) & 0xF) << 8;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(a[u].w, inv) & 0xF) << 12;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(b[u].x, inv) & 0xF) << 16;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(b[u].y, inv) & 0xF) << 20;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(b[u].z, inv) & 0xF) << 24;
            w |= static_cast<uint32_t>(quantize_code<7, -8>(b[u].w, inv) & 0xF) << 28;
            if (i < n8) {
                __stcs(packed + i, w);
                if ((lane & 3) == 0) __stcs(scales + (i >> 2), m / 7.0f);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// INT4, any group size, any element count (groups may straddle rows, the last may be short,
// a byte may hold nibbles of two groups).  Three steps on the same stream:
//   A: scales[g] <- absmax of group g (one warp per group)
//   B: one thread per output byte: inv = 7 / absmax of each element's group, code, pack
//   C: scales[g] <- scales[g] / 7
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) group_absmax_kernel(const float* __restrict__ x, float* __restrict__ scales,
                                                                int64_t n, int64_t group, int64_t ngroups) {
    const int lane = threadIdx.x & 31;
    int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
    for (; warp < ngroups; warp += nwarps) {
        const int64_t beg = warp * group;
        const int64_t end = (beg + group < n) ? beg + group : n;
        float m = 1e-8f;
        for (int64_t i = beg + lane; i < end; i += 32) m = absmax_step(m, x[i]);
        m = warp_max(m);
        if (lane == 0) scales[warp] = m;
    }
}

__global__ void __launch_bounds__(kThreads) pack_int4_generic_kernel(const float* __restrict__ x,
                                                                     const float* __restrict__ absmax,
                                                                     uint8_t* __restrict__ packed, int64_t n,
                                                                     int64_t group, int64_t nbytes) {
    int64_t b = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; b < nbytes; b += stride) {
        const int64_t e0 = 2 * b, e1 = 2 * b + 1;
        const int64_t g0 = e0 / group;
        const float inv0 = 7.0f / absmax[g0];
        uint32_t v = static_cast<uint32_t>(quantize_code<7, -8>(x[e0], inv0) & 0xF);
        if (e1 < n) {
            const int64_t g1 = e1 / group;
            const float inv1 = (g1 == g0) ? inv0 : 7.0f / absmax[g1];
            v |= static_cast<uint32_t>(quantize_code<7, -8>(x[e1], inv1) & 0xF) << 4;
        }
        packed[b] = static_cast<uint8_t>(v);
    }
}

__global__ void __launch_bounds__(kThreads) scale_from_absmax_kernel(float* __restrict__ scales, int64_t n, float qmax) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < n; i += stride) scales[i] = scales[i] / qmax;
}

__global__ void __launch_bounds__(kThreads) scale_from_absmax_pdl_kernel(float* __restrict__ scales, int64_t n, float qmax) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < n; i += stride) scales[i] = scales[i] / qmax;
}

// ------------------------------------------------------------------------------------------
// INT8 per row: one CTA per row.  VEC path (cols % 4 == 0, 16-byte aligned rows): the row is
// read once into registers when it fits (<= CACHE float4 per thread), else read twice (the
// second read comes from L2).  Bytes per element: 4 read + 1 written.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_max(float m, float* red) {
    m = warp_max(m);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) red[w] = m;
    __syncthreads();
    float r = (lane < (kThreads >> 5)) ? red[lane] : 1e-8f;
    r = warp_max(r);
    __syncthreads();
    return r;
}

__device__ __forceinline__ uint32_t pack4_int8(float4 v, float inv) {
    uint32_t w = static_cast<uint32_t>(quantize_code<127, -127>(v.x, inv) & 0xFF);
    w |= static_cast<uint32_t>(quantize_code<127, -127>(v.y, inv) & 0xFF) << 8;
    w |= static_cast<uint32_t>(quantize_code<127, -127>(v.z, inv) & 0xFF) << 16;
    w |= static_cast<uint32_t>(quantize_code<127, -127>(v.w, inv) & 0xFF) << 24;
    return w;
}

template <int CACHE>
__global__ void __launch_bounds__(kThreads) quantize_int8_rows_vec_kernel(const float* __restrict__ x,
                                                                         int8_t* __restrict__ codes,
                                                                         float* __restrict__ scales, int64_t rows,
                                                                         int64_t cols) {
    __shared__ float red[kThreads / 32];
    const int64_t c4 = cols >> 2;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
        uint32_t* qr = reinterpret_cast<uint32_t*>(codes + r * cols);
        float m = 1e-8f;
        if (c4 <= static_cast<int64_t>(CACHE) * kThreads) {
            float4 v[CACHE];
#pragma unroll
            for (int u = 0; u < CACHE; ++u) {
                int64_t i = threadIdx.x + static_cast<int64_t>(u) * kThreads;
                v[u] = (i < c4) ? __ldcs(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < CACHE; ++u) {
                m = absmax_step(m, v[u].x); m = absmax_step(m, v[u].y); m = absmax_step(m, v[u].z); m = absmax_step(m, v[u].w);
            }
            m = block_max(m, red);
            const float inv = 127.0f / m;
#pragma unroll
            for (int u = 0; u < CACHE; ++u) {
                int64_t i = threadIdx.x + static_cast<int64_t>(u) * kThreads;
                if (i < c4) qr[i] = pack4_int8(v[u], inv);
            }
        } else {
            for (int64_t i = threadIdx.x; i < c4; i += kThreads) {
                float4 v = xr[i];
                m = absmax_step(m, v.x); m = absmax_step(m, v.y); m = absmax_step(m, v.z); m = absmax_step(m, v.w);
            }
            m = block_max(m, red);
            const float inv = 127.0f / m;
            for (int64_t i = threadIdx.x; i < c4; i += kThreads) qr[i] = pack4_int8(xr[i], inv);
        }
        if (threadIdx.x == 0) scales[r] = m / 127.0f;
    }
}

__global__ void __launch_bounds__(kThreads) quantize_int8_rows_scalar_kernel(const float* __restrict__ x,
                                                                            int8_t* __restrict__ codes,
                                                                            float* __restrict__ scales, int64_t rows,
                                                                            int64_t cols) {
    __shared__ float red[kThreads / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + r * cols;
        float m = 1e-8f;
        for (int64_t i = threadIdx.x; i < cols; i += kThreads) m = absmax_step(m, xr[i]);
        m = block_max(m, red);
        const float inv = 127.0f / m;
        for (int64_t i = threadIdx.x; i < cols; i += kThreads)
            codes[r * cols + i] = static_cast<int8_t>(quantize_code<127, -127>(xr[i], inv));
        if (threadIdx.x == 0) scales[r] = m / 127.0f;
    }
}

// ------------------------------------------------------------------------------------------
// INT8 per tensor: a grid-wide absmax has to finish before the first code can be written.
//   1: *cell <- 1e-8f            2: atomicMax of the bit pattern (non-negative floats order
//   like their bits)             3: codes, walking the tensor BACKWARDS so that the part step 2
//   touched last is still in the 126 MB L2      4: *cell <- *cell / 127
// Compulsory bytes per element: 4 read + 1 written; 8 read + 1 written when the tensor does
// not stay in L2 between steps 2 and 3.
// ------------------------------------------------------------------------------------------
// The four kernels of this path are launched with programmatic stream serialization when overlap is on: each lets
// the next one start its launch and waits for the one before it before it touches the cell or the tensor.
__global__ void set_f32_kernel(float* p, float v) {
    pdl_launch_dependents();
    pdl_wait();
    *p = v;
}

__global__ void __launch_bounds__(kThreads) tensor_absmax_kernel(const float* __restrict__ x, int64_t n,
                                                                 float* __restrict__ cell) {
    __shared__ float red[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    float m = 1e-8f;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const int64_t n4 = vec ? (n >> 2) : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    int64_t i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {
        float4 a = x4[i], b = x4[i + stride], c = x4[i + 2 * stride], d = x4[i + 3 * stride];
        m = absmax_step(m, a.x); m = absmax_step(m, a.y); m = absmax_step(m, a.z); m = absmax_step(m, a.w);
        m = absmax_step(m, b.x); m = absmax_step(m, b.y); m = absmax_step(m, b.z); m = absmax_step(m, b.w);
        m = absmax_step(m, c.x); m = absmax_step(m, c.y); m = absmax_step(m, c.z); m = absmax_step(m, c.w);
        m = absmax_step(m, d.x); m = absmax_step(m, d.y); m = absmax_step(m, d.z); m = absmax_step(m, d.w);
    }
    for (; i < n4; i += stride) {
        float4 a = x4[i];
        m = absmax_step(m, a.x); m = absmax_step(m, a.y); m = absmax_step(m, a.z); m = absmax_step(m, a.w);
    }
    for (int64_t j = 4 * n4 + tid; j < n; j += stride) m = absmax_step(m, x[j]);
    m = block_max(m, red);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(cell), __float_as_uint(m));
}

__global__ void __launch_bounds__(kThreads) quantize_int8_tensor_kernel(const float* __restrict__ x, int64_t n,
                                                                        const float* __restrict__ cell,
                                                                        int8_t* __restrict__ codes) {
    pdl_launch_dependents();
    pdl_wait();
    const float inv = 127.0f / *cell;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(codes) & 3) == 0);
    const int64_t n4 = vec ? (n >> 2) : 0;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint32_t* q4 = reinterpret_cast<uint32_t*>(codes);
    for (int64_t j = 4 * n4 + tid; j < n; j += stride) codes[j] = static_cast<int8_t>(quantize_code<127, -127>(x[j], inv));
    int64_t i = tid;
    for (; i + 3 * stride < n4; i += 4 * stride) {
        const int64_t r0 = n4 - 1 - i, r1 = r0 - stride, r2 = r1 - stride, r3 = r2 - stride;
        float4 a = x4[r0], b = x4[r1], c = x4[r2], d = x4[r3];
        __stcs(q4 + r0, pack4_int8(a, inv));
        __stcs(q4 + r1, pack4_int8(b, inv));
        __stcs(q4 + r2, pack4_int8(c, inv));
        __stcs(q4 + r3, pack4_int8(d, inv));
    }
    for (; i < n4; i += stride) {
        const int64_t r0 = n4 - 1 - i;
        __stcs(q4 + r0, pack4_int8(x4[r0], inv));
    }
}

// ------------------------------------------------------------------------------------------
// dequantize and code-view kernels (elementwise)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) dequantize_int8_kernel(const int8_t* __restrict__ codes,
                                                                   const float* __restrict__ scales, int64_t n,
                                                                   int64_t cols, int per_row, float* __restrict__ out) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < n; i += stride) {
        const float s = per_row ? scales[i / cols] : scales[0];
        out[i] = __fmul_rn(static_cast<float>(codes[i]), s);
    }
}

__global__ void __launch_bounds__(kThreads) dequantize_int4_kernel(const uint8_t* __restrict__ packed,
                                                                   const float* __restrict__ scales, int64_t n,
                                                                   int64_t group, float* __restrict__ out) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < n; i += stride) out[i] = __fmul_rn(static_cast<float>(load_code_int4(packed, i)), scales[i / group]);
}

__global__ void __launch_bounds__(kThreads) codes_to_f32_kernel(int bits, const void* __restrict__ codes, int64_t n,
                                                                float* __restrict__ out) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < n; i += stride)
        out[i] = (bits == 8) ? static_cast<float>(static_cast<const int8_t*>(codes)[i])
                             : static_cast<float>(load_code_int4(static_cast<const uint8_t*>(codes), i));
}

__global__ void __launch_bounds__(kThreads) codes_from_f32_kernel(int bits, const float* __restrict__ src, int64_t n,
                                                                  void* __restrict__ codes) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    if (bits == 8) {
        for (; i < n; i += stride) static_cast<int8_t*>(codes)[i] = static_cast<int8_t>(static_cast<int>(src[i]));
    } else {
        const int64_t nbytes = (n + 1) >> 1;
        for (; i < nbytes; i += stride) {
            uint32_t v = static_cast<uint32_t>(static_cast<int>(src[2 * i])) & 0xF;
            if (2 * i + 1 < n) v |= (static_cast<uint32_t>(static_cast<int>(src[2 * i + 1])) & 0xF) << 4;
            static_cast<uint8_t*>(codes)[i] = static_cast<uint8_t>(v);
        }
    }
}

__global__ void __launch_bounds__(kThreads) interleave_kernel(const float* __restrict__ src, int64_t world, int64_t M,
                                                              int64_t n_local, float* __restrict__ dst, int64_t ldd) {
    const int64_t total = world * M * n_local;
    int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (; i < total; i += stride) {
        const int64_t n = i % n_local;
        const int64_t m = (i / n_local) % M;
        const int64_t r = i / (n_local * M);
        dst[m * ldd + r * n_local + n] = src[i];
    }
}

int grid_for(int64_t work_items, int per_block, int waves = 8) {
    int64_t blocks = ceil_div(work_items, per_block);
    int64_t cap = static_cast<int64_t>(sm_count()) * waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace

int launch_quantize_int4(const float* x, int64_t n, int64_t group, uint8_t* packed, float* scales, cudaStream_t s) {
    if (n == 0) return SGQ_OK;
    int64_t done = 0;  // elements handled by the group-of-32 kernel
    if (group == 32 && aligned(x, 16) && aligned(packed, 4)) {
        const int64_t full_groups = n / 32;
        if (full_groups > 0) {
            const int64_t n8 = full_groups * 4;
            constexpr int UNROLL = 4;
            // one warp step = 32*UNROLL chunks; grid sized in multiples of the SM count
            const int grid = grid_for(n8, kThreads * UNROLL, 16);
            quantize_int4_g32_kernel<UNROLL><<<grid, kThreads, 0, s>>>(reinterpret_cast<const float4*>(x),
                                                                        reinterpret_cast<uint32_t*>(packed), scales, n8);
            SGQ_LAUNCH_CHECK("quantize_int4_g32_kernel");
            done = full_groups * 32;
        }
    }
    if (done < n) {
        // remainder (or everything, for other group sizes); `done` is a multiple of 32, so the
        // remainder starts on a byte and on a group boundary.
        const float* xr = x + done;
        uint8_t* pr = packed + done / 2;
        float* sr = scales + done / group;
        const int64_t nr = n - done;
        const int64_t ngroups = ceil_div(nr, group);
        const int64_t nbytes = (nr + 1) / 2;
        group_absmax_kernel<<<grid_for(ngroups, kThreads / 32), kThreads, 0, s>>>(xr, sr, nr, group, ngroups);
        SGQ_LAUNCH_CHECK("group_absmax_kernel");
        pack_int4_generic_kernel<<<grid_for(nbytes, kThreads), kThreads, 0, s>>>(xr, sr, pr, nr, group, nbytes);
        SGQ_LAUNCH_CHECK("pack_int4_generic_kernel");
        scale_from_absmax_kernel<<<grid_for(ngroups, kThreads), kThreads, 0, s>>>(sr, ngroups, 7.0f);
        SGQ_LAUNCH_CHECK("scale_from_absmax_kernel");
    }
    return SGQ_OK;
}

int launch_quantize_int8(const float* x, int64_t rows, int64_t cols, int scheme, int8_t* codes, float* scales,
                         cudaStream_t s) {
    const int64_t n = rows * cols;
    if (scheme == SGQ_PER_TENSOR) {
        const bool ov = stream_overlap_enabled();
        SGQ_CUDA_TRY(launch_kernel(set_f32_kernel, dim3(1), dim3(1), 0, s, ov, scales, 1e-8f));
        if (n > 0) {
            const int grid = grid_for(n, kThreads * 16, 8);
            SGQ_CUDA_TRY(launch_kernel(tensor_absmax_kernel, dim3(grid), dim3(kThreads), 0, s, ov, x, n, scales));
            SGQ_CUDA_TRY(launch_kernel(quantize_int8_tensor_kernel, dim3(grid), dim3(kThreads), 0, s, ov, x, n,
                                       static_cast<const float*>(scales), codes));
        }
        SGQ_CUDA_TRY(launch_kernel(scale_from_absmax_pdl_kernel, dim3(1), dim3(kThreads), 0, s, ov, scales, static_cast<int64_t>(1), 127.0f));
        return SGQ_OK;
    }
    if (rows == 0) return SGQ_OK;
    const int grid = static_cast<int>(rows < 65535LL * 16 ? rows : 65535LL * 16);
    if (cols > 0 && (cols & 3) == 0 && aligned(x, 16) && aligned(codes, 4)) {
        quantize_int8_rows_vec_kernel<8><<<grid, kThreads, 0, s>>>(x, codes, scales, rows, cols);
        SGQ_LAUNCH_CHECK("quantize_int8_rows_vec_kernel");
    } else {
        quantize_int8_rows_scalar_kernel<<<grid, kThreads, 0, s>>>(x, codes, scales, rows, cols);
        SGQ_LAUNCH_CHECK("quantize_int8_rows_scalar_kernel");
    }
    return SGQ_OK;
}

int launch_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme,
                           float* out, cudaStream_t s) {
    const int64_t n = rows * cols;
    if (n == 0) return SGQ_OK;
    dequantize_int8_kernel<<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(codes, scales, n, cols,
                                                                           scheme == SGQ_PER_ROW ? 1 : 0, out);
    SGQ_LAUNCH_CHECK("dequantize_int8_kernel");
    return SGQ_OK;
}

int launch_dequantize_int4(const uint8_t* packed, const float* scales, int64_t n, int64_t group, float* out,
                           cudaStream_t s) {
    if (n == 0) return SGQ_OK;
    dequantize_int4_kernel<<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(packed, scales, n, group, out);
    SGQ_LAUNCH_CHECK("dequantize_int4_kernel");
    return SGQ_OK;
}

int launch_codes_to_f32(int bits, const void* codes, int64_t n, float* out, cudaStream_t s) {
    if (n == 0) return SGQ_OK;
    codes_to_f32_kernel<<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(bits, codes, n, out);
    SGQ_LAUNCH_CHECK("codes_to_f32_kernel");
    return SGQ_OK;
}

int launch_codes_from_f32(int bits, const float* codes_f32, int64_t n, void* codes, cudaStream_t s) {
    if (n == 0) return SGQ_OK;
    codes_from_f32_kernel<<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(bits, codes_f32, n, codes);
    SGQ_LAUNCH_CHECK("codes_from_f32_kernel");
    return SGQ_OK;
}

int launch_interleave(const float* src, int64_t world, int64_t M, int64_t n_local, float* dst, int64_t ldd,
                      cudaStream_t s) {
    const int64_t total = world * M * n_local;
    if (total == 0) return SGQ_OK;
    interleave_kernel<<<grid_for(total, kThreads * 4), kThreads, 0, s>>>(src, world, M, n_local, dst, ldd);
    SGQ_LAUNCH_CHECK("interleave_kernel");
    return SGQ_OK;
}

}  // namespace sgq
