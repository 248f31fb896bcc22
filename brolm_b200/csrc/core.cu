// Row-wise kernels of the decoder step: embedding, norms with the residual
// sum, rotary position encoding with the write into the paged cache, the
// gated activation and the soft-cap of the logits.  Each kernel runs one
// block per token row; statistics and sums are float whatever the element
// type.  Compiled for sm_100a only.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding gather with scale:  h[t, :] = float(table[ids[t], :]) * scale
// (wlejon/brolm src/gemma2.cpp:283-285 and :340-343, fused).
// ---------------------------------------------------------------------------
template <typename W>
__global__ void embed_scale_kernel(const int32_t* __restrict__ ids, const W* __restrict__ table,
                                   float scale, float* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    const W* row = table + (size_t)ids[t] * hidden;
    float* dst = out + (size_t)t * hidden;
#pragma unroll 4
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(row[i]) * scale;
}

BROLM_API int brolm_embed_scale(const void* ids, const void* table, int table_dtype, float scale,
                                void* out, int tokens, int hidden, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (table_dtype == BROLM_F32)
        embed_scale_kernel<float><<<tokens, 256, 0, stream>>>((const int32_t*)ids, (const float*)table, scale,
                                                              (float*)out, hidden);
    else if (table_dtype == BROLM_BF16)
        embed_scale_kernel<bf16><<<tokens, 256, 0, stream>>>((const int32_t*)ids, (const bf16*)table, scale,
                                                             (float*)out, hidden);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm:  y = x * rsqrt(mean(x^2) + eps) * (offset + w)
// (src/gemma2.cpp:349; the reference folds the +1 into w at load, :154-175).
// `rows` (optional) picks the input rows, so that only wanted rows of the
// final norm are computed.
//
// One block per row.  When the width is a multiple of 4 and at most
// 256 * 4 * MAXC, every thread keeps its share of the row in registers: all
// loads of the row and of the gain are issued before the first use, so a row
// costs one trip to memory instead of one per element (a decode step has only
// a handful of rows, and latency is all there is).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
    uint2 t;
    *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
}

// MAXC = 0: any width, plain loops.
template <typename X, typename W, typename O, int MAXC>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const X* __restrict__ x, const int32_t* __restrict__ rows,
                                                      const W* __restrict__ w, float eps, float offset,
                                                      O* __restrict__ out, int hidden) {
    __shared__ float scratch[64];
    const int r = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const X* src = x + (size_t)(rows ? rows[r] : r) * hidden;
    O* dst = out + (size_t)r * hidden;
    if (MAXC == 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_float(src[i]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            dst[i] = from_float<O>(to_float(src[i]) * inv * (offset + to_float(w[i])));
        return;
    }
    constexpr int C = MAXC > 0 ? MAXC : 1;
    float v[C][4], g[C][4];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        if (i < hidden) { load4(src + i, v[c]); load4(w + i, g[c]); }
        else { v[c][0] = v[c][1] = v[c][2] = v[c][3] = 0.0f; g[c][0] = g[c][1] = g[c][2] = g[c][3] = 0.0f; }
    }
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) ss += v[c][0] * v[c][0] + v[c][1] * v[c][1] + v[c][2] * v[c][2] + v[c][3] * v[c][3];
    ss = block_sum_once(ss, scratch, 0);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = v[c][e] * inv * (offset + g[c][e]);
            store4(dst + i, o);
        }
    }
}

static int vec_chunks(int hidden, const void* a, const void* b, const void* c, const void* d) {
    const uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d;
    if (hidden % 4 != 0 || (bits & 15)) return 0;
    if (hidden <= 1024) return 1;
    if (hidden <= 2048) return 2;
    if (hidden <= 3072) return 3;
    if (hidden <= 4096) return 4;
    if (hidden <= 8192) return 8;
    return 0;
}

template <typename X, typename W, typename O>
static int rmsnorm_launch(const void* x, const void* rows, const void* w, float eps, float offset, void* out, int n,
                          int hidden, cudaStream_t s) {
    const int c = vec_chunks(hidden, x, w, out, nullptr);
#define BROLM_RMS(C) launch_pdl(rmsnorm_kernel<X, W, O, C>, dim3(n), dim3(256), 0, s, (const X*)x, (const int32_t*)rows, \
                                (const W*)w, eps, offset, (O*)out, hidden)
    if (c == 1) return BROLM_RMS(1);
    if (c == 2) return BROLM_RMS(2);
    if (c == 3) return BROLM_RMS(3);
    if (c == 4) return BROLM_RMS(4);
    if (c == 8) return BROLM_RMS(8);
    return BROLM_RMS(0);
#undef BROLM_RMS
}

template <typename X, typename W>
static int rmsnorm_out(const void* x, const void* rows, const void* w, float eps, float offset, void* out,
                       int out_dtype, int n, int hidden, cudaStream_t s) {
    if (out_dtype == BROLM_F32) return rmsnorm_launch<X, W, float>(x, rows, w, eps, offset, out, n, hidden, s);
    if (out_dtype == BROLM_BF16) return rmsnorm_launch<X, W, bf16>(x, rows, w, eps, offset, out, n, hidden, s);
    return BROLM_ERR_BAD_DTYPE;
}

BROLM_API int brolm_rmsnorm(const void* x, int x_dtype, const void* rows, const void* w, int w_dtype, float eps,
                            float offset, void* out, int out_dtype, int n, int hidden, cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_F32)
        return rmsnorm_out<float, float>(x, rows, w, eps, offset, out, out_dtype, n, hidden, stream);
    if (x_dtype == BROLM_F32 && w_dtype == BROLM_BF16)
        return rmsnorm_out<float, bf16>(x, rows, w, eps, offset, out, out_dtype, n, hidden, stream);
    if (x_dtype == BROLM_BF16 && w_dtype == BROLM_F32)
        return rmsnorm_out<bf16, float>(x, rows, w, eps, offset, out, out_dtype, n, hidden, stream);
    if (x_dtype == BROLM_BF16 && w_dtype == BROLM_BF16)
        return rmsnorm_out<bf16, bf16>(x, rows, w, eps, offset, out, out_dtype, n, hidden, stream);
    return BROLM_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// Residual sum with the norms around it, one pass over the row:
//     h += post ? rmsnorm(y; w_post) : y          (src/gemma2.cpp:372-373, 385-386)
//     out = rmsnorm(h; w_next)   if w_next        (src/gemma2.cpp:376, :349 of the next layer)
// h is the float residual stream.  Same register scheme as above.
// ---------------------------------------------------------------------------
// y may come as n_parts partial sums, part_stride elements apart (the slices
// of a product that was cut along K); they are added in order while loading.
template <typename Y, typename W, typename O, int MAXC>
__global__ void __launch_bounds__(256, (MAXC >= 1 && MAXC <= 3) ? 4 : 1) residual_rmsnorm_kernel(float* __restrict__ h, const Y* __restrict__ y,
                                                               int n_parts, long long part_stride,
                                                               const W* __restrict__ w_post, float eps_post,
                                                               float off_post, const W* __restrict__ w_next,
                                                               float eps_next, float off_next, O* __restrict__ out,
                                                               int hidden) {
    __shared__ float scratch[64];
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * hidden;
    const Y* yr = y + (size_t)r * hidden;
    O* dst = out + (size_t)r * hidden;
    pdl_trigger();
    if (MAXC == 0) {
        pdl_wait();
        auto y_at = [&](int i) {
            float v = to_float(yr[i]);
            for (int s = 1; s < n_parts; ++s) v += to_float(yr[(size_t)s * part_stride + i]);
            return v;
        };
        float inv_post = 1.0f;
        if (w_post) {
            float ss = 0.0f;
            for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
                const float v = y_at(i);
                ss += v * v;
            }
            ss = block_sum(ss, scratch);
            inv_post = rsqrtf(ss / (float)hidden + eps_post);
        }
        float ss2 = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = y_at(i);
            if (w_post) v = v * inv_post * (off_post + to_float(w_post[i]));
            const float s = hr[i] + v;
            hr[i] = s;
            ss2 += s * s;
        }
        if (!w_next) return;
        ss2 = block_sum(ss2, scratch);
        const float inv_next = rsqrtf(ss2 / (float)hidden + eps_next);
        // every thread reads back only what it wrote itself
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            dst[i] = from_float<O>(hr[i] * inv_next * (off_next + to_float(w_next[i])));
        return;
    }
    constexpr int C = MAXC > 0 ? MAXC : 1;
    float v[C][4], res[C][4];
    // The gains are weights: brought into the L1 while the kernel before this one finishes, and read where
    // they are used, so that they hold no registers meanwhile (with many rows the number of blocks that fit
    // an SM, and with it the bytes in flight, is set by the registers).
    {
        const size_t line = (size_t)threadIdx.x * 128;
        if (line < (size_t)hidden * sizeof(W)) {
            if (w_post) prefetch_l1(reinterpret_cast<const char*>(w_post) + line);
            if (w_next) prefetch_l1(reinterpret_cast<const char*>(w_next) + line);
        }
    }
    pdl_wait();
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c][e] = res[c][e] = 0.0f;
        if (i < hidden) {
            // every slice's load goes out before the first is added: one round trip to the L2, not one per slice
            constexpr int AT_ONCE = 4;
            load4(hr + i, res[c]);
            for (int s0 = 0; s0 < n_parts; s0 += AT_ONCE) {
                float t[AT_ONCE][4];
#pragma unroll
                for (int s = 0; s < AT_ONCE; ++s)
                    if (s0 + s < n_parts) load4(yr + (size_t)(s0 + s) * part_stride + i, t[s]);
#pragma unroll
                for (int s = 0; s < AT_ONCE; ++s)
                    if (s0 + s < n_parts) {                  // added in the order of the slices
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[c][e] += t[s][e];
                    }
            }
        }
    }
    if (w_post) {
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) ss += v[c][0] * v[c][0] + v[c][1] * v[c][1] + v[c][2] * v[c][2] + v[c][3] * v[c][3];
        ss = block_sum_once(ss, scratch, 0);
        const float inv_post = rsqrtf(ss / (float)hidden + eps_post);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int i = (c * 256 + threadIdx.x) * 4;
            float g[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (i < hidden) load4(w_post + i, g);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[c][e] = v[c][e] * inv_post * (off_post + g[e]);
        }
    }
    float ss2 = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            res[c][e] += v[c][e];
            ss2 += res[c][e] * res[c][e];
        }
        if (i < hidden) store4(hr + i, res[c]);
    }
    if (!w_next) return;
    ss2 = block_sum_once(ss2, scratch, 1);
    const float inv_next = rsqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            float g[4], o[4];
            load4(w_next + i, g);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = res[c][e] * inv_next * (off_next + g[e]);
            store4(dst + i, o);
        }
    }
}

// The same for y in one part, with the row in shared memory instead of registers: cp.async brings y and the
// residual straight into the block's own copy, every thread reads back only the elements it copied itself
// (the mapping of elements to threads and the order of every sum are those of the kernel above), and with
// about 32 registers eight blocks fit an SM, which is what keeps enough bytes in flight when there are
// thousands of rows.  Dynamic shared memory: C * 1024 elements of Y, then C * 1024 floats.
__device__ __forceinline__ void copy_async(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async(bf16* dst, const bf16* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
template <typename Y, typename W, typename O, int C>
__global__ void __launch_bounds__(256, 8) residual_rmsnorm_rows_kernel(float* __restrict__ h, const Y* __restrict__ y,
                                                                       const W* __restrict__ w_post, float eps_post,
                                                                       float off_post, const W* __restrict__ w_next,
                                                                       float eps_next, float off_next,
                                                                       O* __restrict__ out, int hidden) {
    __shared__ float scratch[64];
    extern __shared__ __align__(16) unsigned char row_raw[];
    Y* sy = reinterpret_cast<Y*>(row_raw);
    float* sh = reinterpret_cast<float*>(row_raw + (size_t)C * 1024 * sizeof(Y));
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * hidden;
    const Y* yr = y + (size_t)r * hidden;
    O* dst = out + (size_t)r * hidden;
    pdl_trigger();
    {
        const size_t line = (size_t)threadIdx.x * 128;
        if (line < (size_t)hidden * sizeof(W)) {
            if (w_post) prefetch_l1(reinterpret_cast<const char*>(w_post) + line);
            if (w_next) prefetch_l1(reinterpret_cast<const char*>(w_next) + line);
        }
    }
    pdl_wait();
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            copy_async(sh + i, hr + i);
            copy_async(sy + i, yr + i);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float inv_post = 1.0f;
    if (w_post) {
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int i = (c * 256 + threadIdx.x) * 4;
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (i < hidden) load4(sy + i, v);
            ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
        ss = block_sum_once(ss, scratch, 0);
        inv_post = rsqrtf(ss / (float)hidden + eps_post);
    }
    float ss2 = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f}, res[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (i < hidden) {
            load4(sy + i, v);
            load4(sh + i, res);
            if (w_post) {
                float g[4];
                load4(w_post + i, g);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = v[e] * inv_post * (off_post + g[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            res[e] += v[e];
            ss2 += res[e] * res[e];
        }
        if (i < hidden) {
            store4(hr + i, res);
            if (w_next) store4(sh + i, res);
        }
    }
    if (!w_next) return;
    ss2 = block_sum_once(ss2, scratch, 1);
    const float inv_next = rsqrtf(ss2 / (float)hidden + eps_next);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            float res[4], g[4], o[4];
            load4(sh + i, res);
            load4(w_next + i, g);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = res[e] * inv_next * (off_next + g[e]);
            store4(dst + i, o);
        }
    }
}

template <typename Y, typename W, typename O>
static int residual_launch(void* h, const void* y, int n_parts, long long part_stride, const void* w_post, float eps_post, float off_post,
                           const void* w_next, float eps_next, float off_next, void* out, int n, int hidden,
                           cudaStream_t s) {
    int c = vec_chunks(hidden, h, y, w_post, w_next);
    if (c && (((uintptr_t)out & 15) || part_stride % 4 != 0)) c = 0;
    if (n_parts == 1 && c >= 1 && c <= 4) {
        // one part: the row in shared memory (whatever the number of rows, so that a row's bits do not
        // depend on how many rows the launch has)
#define BROLM_ROWS(C) launch_pdl(residual_rmsnorm_rows_kernel<Y, W, O, C>, dim3(n), dim3(256), \
        (size_t)C * 1024 * (sizeof(Y) + sizeof(float)), s, (float*)h, (const Y*)y, (const W*)w_post, eps_post, off_post, \
        (const W*)w_next, eps_next, off_next, (O*)out, hidden)
        if (c == 1) return BROLM_ROWS(1);
        if (c == 2) return BROLM_ROWS(2);
        if (c == 3) return BROLM_ROWS(3);
        return BROLM_ROWS(4);
#undef BROLM_ROWS
    }
#define BROLM_RES(C) launch_pdl(residual_rmsnorm_kernel<Y, W, O, C>, dim3(n), dim3(256), 0, s, (float*)h, (const Y*)y, \
        n_parts, part_stride, (const W*)w_post, eps_post, off_post, (const W*)w_next, eps_next, off_next, (O*)out, hidden)
    if (c == 1) return BROLM_RES(1);
    if (c == 2) return BROLM_RES(2);
    if (c == 3) return BROLM_RES(3);
    if (c == 4) return BROLM_RES(4);
    if (c == 8) return BROLM_RES(8);
    return BROLM_RES(0);
#undef BROLM_RES
}

template <typename Y, typename W>
static int residual_out(void* h, const void* y, int n_parts, long long part_stride, const void* w_post, float eps_post, float off_post,
                        const void* w_next, float eps_next, float off_next, void* out, int out_dtype, int n,
                        int hidden, cudaStream_t s) {
    if (out_dtype == BROLM_F32)
        return residual_launch<Y, W, float>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out, n, hidden, s);
    if (out_dtype == BROLM_BF16)
        return residual_launch<Y, W, bf16>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out, n, hidden, s);
    return BROLM_ERR_BAD_DTYPE;
}

// w_post and w_next share one element type (w_dtype); either may be null.
BROLM_API int brolm_residual_rmsnorm(void* h, const void* y, int y_dtype, int n_parts, long long part_stride,
                                     const void* w_post, float eps_post,
                                     float off_post, const void* w_next, float eps_next, float off_next,
                                     int w_dtype, void* out, int out_dtype, int n, int hidden,
                                     cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    if (n_parts < 1) return BROLM_ERR_BAD_SIZE;
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_F32)
        return residual_out<float, float>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                          out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_BF16)
        return residual_out<float, bf16>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                         out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_F32)
        return residual_out<bf16, float>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                         out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_BF16)
        return residual_out<bf16, bf16>(h, y, n_parts, part_stride, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                        out_dtype, n, hidden, stream);
    return BROLM_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// Rotary position encoding of q and k in the fused projection output, and the
// write of k (rotated) and v into the paged cache.
//
// qkv row t: [ q: n_q*hd | k: n_kv*hd | v: n_kv*hd ].  The pair is
// (i, i + rot/2) inside the first `rot` elements of a head, the angle
// pos * theta^(-2i/rot) comes from a table of (cos, sin) built on the host in
// double (src/gemma2.cpp:355-356; pairing as stored in the checkpoint, which
// include/brolm/detail/weights.h:106-127 permutes instead).
//
// A negative position marks a padding row, which is left untouched.  The cache
// of this layer is k_pages/v_pages [page][kv_head][page_size][hd];
// cache_rows[t] = page * page_size + place says where token t goes, a negative
// value that it is not kept (a later position of the same step owns its place
// in the ring).  One block per (token, head), one pair of elements per thread:
// every load of a token is issued at once.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const float2* __restrict__ cos_sin, int n_q, int n_kv, int hd, int rot,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int32_t* __restrict__ cache_rows, int page_size) {
    const int t = blockIdx.x, head = blockIdx.y;          // head: q heads, then k heads, then v heads
    const int pos = positions[t];
    if (pos < 0) return;
    const bool is_v = head >= n_q + n_kv, is_k = !is_v && head >= n_q;
    const bool rotate = !is_v && cos_sin != nullptr;
    if (!rotate && !((is_k || is_v) && k_pages)) return;  // nothing to do for this head
    const int crow = (k_pages && (is_k || is_v)) ? cache_rows[t] : -1;
    if (is_v && crow < 0) return;
    T* p = qkv + (size_t)t * (n_q + 2 * n_kv) * hd + (size_t)head * hd;
    T* dst = nullptr;
    if (crow >= 0) {
        const int g = is_k ? head - n_q : head - n_q - n_kv;
        T* pages = is_k ? k_pages : v_pages;
        dst = pages + (((size_t)(crow / page_size) * n_kv + g) * page_size + crow % page_size) * hd;
    }
    const int half = rot >> 1;
    for (int j = threadIdx.x; j < (hd >> 1); j += blockDim.x) {
        // the two elements of this thread: a rotated pair, or two elements past the rotated part
        const bool in_rot = j < half;
        const int e0 = in_rot ? j : rot + 2 * (j - half), e1 = in_rot ? j + half : e0 + 1;
        T a = p[e0], b = p[e1];
        if (rotate && in_rot) {
            const float2 c = cos_sin[(size_t)pos * half + j];
            const float fa = to_float(a), fb = to_float(b);
            a = from_float<T>(fa * c.x - fb * c.y);
            b = from_float<T>(fa * c.y + fb * c.x);
            p[e0] = a;
            p[e1] = b;
        }
        if (dst) { dst[e0] = a; dst[e1] = b; }
    }
}

// bfloat16, rot == hd, hd a multiple of 16: eight pairs per thread with 16-byte
// accesses; one block per token, items = heads * hd/16.
__global__ void __launch_bounds__(256) rope_kv_write_vec_kernel(bf16* __restrict__ qkv,
                                                                const int32_t* __restrict__ positions,
                                                                const float2* __restrict__ cos_sin, int n_q, int n_kv,
                                                                int hd, bf16* __restrict__ k_pages,
                                                                bf16* __restrict__ v_pages,
                                                                const int32_t* __restrict__ cache_rows,
                                                                int page_size) {
    const int t = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int pos = positions[t];
    if (pos < 0) return;
    const int half = hd >> 1, per_head = half >> 3;
    const int heads = n_q + 2 * n_kv;
    const int crow = k_pages ? cache_rows[t] : -1;
    bf16* row = qkv + (size_t)t * heads * hd;
    for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
        const int head = item / per_head, i0 = (item - head * per_head) << 3;
        const bool is_v = head >= n_q + n_kv, is_k = !is_v && head >= n_q;
        const bool rotate = !is_v && cos_sin != nullptr;
        const bool keep = crow >= 0 && (is_k || is_v);
        if (!rotate && !keep) continue;
        bf16* p = row + (size_t)head * hd;
        uint4 ra = *reinterpret_cast<const uint4*>(p + i0), rb = *reinterpret_cast<const uint4*>(p + half + i0);
        if (rotate) {
            const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * half + i0);
            __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&ra);
            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 c = cs[j];                       // (cos, sin) of pairs 2j and 2j + 1
                const float2 fa = __bfloat1622float2(a2[j]), fb = __bfloat1622float2(b2[j]);
                a2[j] = __floats2bfloat162_rn(fa.x * c.x - fb.x * c.y, fa.y * c.z - fb.y * c.w);
                b2[j] = __floats2bfloat162_rn(fa.x * c.y + fb.x * c.x, fa.y * c.w + fb.y * c.z);
            }
            *reinterpret_cast<uint4*>(p + i0) = ra;
            *reinterpret_cast<uint4*>(p + half + i0) = rb;
        }
        if (keep) {
            const int g = is_k ? head - n_q : head - n_q - n_kv;
            bf16* dst = (is_k ? k_pages : v_pages) +
                        (((size_t)(crow / page_size) * n_kv + g) * page_size + crow % page_size) * hd;
            *reinterpret_cast<uint4*>(dst + i0) = ra;
            *reinterpret_cast<uint4*>(dst + half + i0) = rb;
        }
    }
}

// The same for a q/k/v projection that arrives as float partial sums of K slices (the few-token tcgen05
// product cut along K so that every SM streams weights): the slices are added in order, q and k rotated,
// and everything rounded to bfloat16 once, into the packed q/k/v row and into the cache pages.
// rot == hd (or no rotation), hd a multiple of 16; one block per token, eight pairs per thread and item.
__global__ void __launch_bounds__(256) rope_kv_write_parts_kernel(const float* __restrict__ parts, int n_parts,
                                                                  long long part_stride, bf16* __restrict__ qkv,
                                                                  int ld_out, const int32_t* __restrict__ positions,
                                                                  const float2* __restrict__ cos_sin, int n_q,
                                                                  int n_kv, int hd, bf16* __restrict__ k_pages,
                                                                  bf16* __restrict__ v_pages,
                                                                  const int32_t* __restrict__ cache_rows,
                                                                  int page_size) {
    const int t = blockIdx.x;
    const int pos = positions[t];                 // (the host's, written before the step's first kernel)
    const int crow = (k_pages && pos >= 0) ? cache_rows[t] : -1;
    pdl_trigger();
    pdl_wait();
    if (pos < 0) return;
    const int half = hd >> 1, per_head = half >> 3;
    const int heads = n_q + 2 * n_kv, width = heads * hd;
    const float* src = parts + (size_t)t * width;
    bf16* row = qkv + (size_t)t * ld_out;
    for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
        const int head = item / per_head, i0 = (item - head * per_head) << 3;
        const bool is_v = head >= n_q + n_kv, is_k = !is_v && head >= n_q;
        const bool rotate = !is_v && cos_sin != nullptr;
        float a[8], b[8];
        load8(src + (size_t)head * hd + i0, a);
        load8(src + (size_t)head * hd + half + i0, b);
        for (int s = 1; s < n_parts; ++s) {                    // added in the order of the slices
            float ta[8], tb[8];
            load8(src + (size_t)s * part_stride + (size_t)head * hd + i0, ta);
            load8(src + (size_t)s * part_stride + (size_t)head * hd + half + i0, tb);
#pragma unroll
            for (int j = 0; j < 8; ++j) { a[j] += ta[j]; b[j] += tb[j]; }
        }
        if (rotate) {
            const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * half + i0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 c = cs[j];                       // (cos, sin) of pairs 2j and 2j + 1
                const float a0 = a[2 * j], a1 = a[2 * j + 1], b0 = b[2 * j], b1 = b[2 * j + 1];
                a[2 * j] = a0 * c.x - b0 * c.y;
                b[2 * j] = a0 * c.y + b0 * c.x;
                a[2 * j + 1] = a1 * c.z - b1 * c.w;
                b[2 * j + 1] = a1 * c.w + b1 * c.z;
            }
        }
        uint4 ra, rb;
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&ra);
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            a2[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
            b2[j] = __floats2bfloat162_rn(b[2 * j], b[2 * j + 1]);
        }
        bf16* p = row + (size_t)head * hd;
        *reinterpret_cast<uint4*>(p + i0) = ra;
        *reinterpret_cast<uint4*>(p + half + i0) = rb;
        if (crow >= 0 && (is_k || is_v)) {
            const int g = is_k ? head - n_q : head - n_q - n_kv;
            bf16* dst = (is_k ? k_pages : v_pages) +
                        (((size_t)(crow / page_size) * n_kv + g) * page_size + crow % page_size) * hd;
            *reinterpret_cast<uint4*>(dst + i0) = ra;
            *reinterpret_cast<uint4*>(dst + half + i0) = rb;
        }
    }
}

// parts: [n_parts] float slices of (tokens, (n_q + 2 n_kv) * hd), part_stride elements apart; qkv: bfloat16 rows of
// ld_out elements.  The rotation covers the whole head (cos_sin [position][hd / 2], null: none).
BROLM_API int brolm_rope_kv_write_parts(const void* parts, int n_parts, long long part_stride, void* qkv, int ld_out,
                                        const void* positions, const void* cos_sin, int n_q, int n_kv, int hd,
                                        void* k_pages, void* v_pages, const void* cache_rows, int page_size,
                                        int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (n_parts < 1 || hd <= 0 || hd % 16 != 0 || page_size <= 0 || n_q <= 0 || n_kv <= 0) return BROLM_ERR_BAD_SIZE;
    if (k_pages && (!v_pages || !cache_rows)) return BROLM_ERR_BAD_SIZE;
    if (((uintptr_t)parts & 15) || ((uintptr_t)qkv & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
        ((uintptr_t)cos_sin & 15) || ld_out % 8 != 0 || part_stride % 4 != 0)
        return BROLM_ERR_ALIGNMENT;
    int items = (n_q + 2 * n_kv) * (hd >> 4);
    int th = (items + 31) / 32 * 32;
    if (th > 256) th = 256;
    return launch_pdl(rope_kv_write_parts_kernel, dim3(tokens), dim3(th), 0, stream, (const float*)parts, n_parts,
                      part_stride, (bf16*)qkv, ld_out, (const int32_t*)positions, (const float2*)cos_sin, n_q, n_kv, hd,
                      (bf16*)k_pages, (bf16*)v_pages, (const int32_t*)cache_rows, page_size);
}

BROLM_API int brolm_rope_kv_write(void* qkv, int dtype, const void* positions, const void* cos_sin, int n_q, int n_kv,
                                  int hd, int rot, void* k_pages, void* v_pages, const void* cache_rows,
                                  int page_size, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (rot > hd || (rot & 1) || (hd & 1) || page_size <= 0) return BROLM_ERR_BAD_SIZE;
    if (n_q + 2 * n_kv > 65535) return BROLM_ERR_TOO_LARGE;
    if (dtype == BROLM_BF16 && (rot == hd || !cos_sin) && hd % 16 == 0 && ((uintptr_t)qkv & 15) == 0 &&
        ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0 && ((uintptr_t)cos_sin & 15) == 0) {
        int items = (n_q + 2 * n_kv) * (hd >> 4);
        int th = (items + 31) / 32 * 32;
        if (th > 256) th = 256;
        return launch_pdl(rope_kv_write_vec_kernel, dim3(tokens), dim3(th), 0, stream, (bf16*)qkv,
                          (const int32_t*)positions, (const float2*)cos_sin, n_q, n_kv, hd, (bf16*)k_pages,
                          (bf16*)v_pages, (const int32_t*)cache_rows, page_size);
    }
    dim3 grid(tokens, n_q + 2 * n_kv);
    int threads = ((hd >> 1) + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    if (dtype == BROLM_F32)
        rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>(
            (float*)qkv, (const int32_t*)positions, (const float2*)cos_sin, n_q, n_kv, hd, rot, (float*)k_pages,
            (float*)v_pages, (const int32_t*)cache_rows, page_size);
    else if (dtype == BROLM_BF16)
        rope_kv_write_kernel<bf16><<<grid, threads, 0, stream>>>(
            (bf16*)qkv, (const int32_t*)positions, (const float2*)cos_sin, n_q, n_kv, hd, rot, (bf16*)k_pages,
            (bf16*)v_pages, (const int32_t*)cache_rows, page_size);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}

// ---------------------------------------------------------------------------
// Gated activation on the fused [gate | up] projection:
//     out[t, j] = act(gate[t, j]) * up[t, j]        (src/gemma2.cpp:380-381)
// act 0: gelu, tanh form  0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// act 1: silu             z / (1 + exp(-z))
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_apply(float z, int act) {
    if (act == 0) {
        const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
        return 0.5f * z * (1.0f + tanhf(u));
    }
    return z / (1.0f + expf(-z));
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int act) {
    const size_t t = blockIdx.x;
    const T* g = gate_up + t * 2 * (size_t)inter;
    const T* u = g + inter;
    T* o = out + t * (size_t)inter;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < inter; j += gridDim.y * blockDim.x)
        o[j] = from_float<T>(act_apply(to_float(g[j]), act) * to_float(u[j]));
}

// bfloat16 with inter a multiple of 8: eight elements per thread, 16-byte accesses.
__global__ void __launch_bounds__(256) gated_act_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out,
                                                            int inter, int act) {
    const size_t t = blockIdx.x;
    const bf16* g = gate_up + t * 2 * (size_t)inter;
    const bf16* u = g + inter;
    bf16* o = out + t * (size_t)inter;
    for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * 8; j < inter; j += gridDim.y * blockDim.x * 8) {
        float gv[8], uv[8];
        load8(g + j, gv);
        load8(u + j, uv);
        uint4 r;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            r2[e] = __floats2bfloat162_rn(act_apply(gv[2 * e], act) * uv[2 * e], act_apply(gv[2 * e + 1], act) * uv[2 * e + 1]);
        *reinterpret_cast<uint4*>(o + j) = r;
    }
}

BROLM_API int brolm_gated_act(const void* gate_up, void* out, int dtype, int tokens, int inter, int act,
                              cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (act < 0 || act > 1) return BROLM_ERR_BAD_SIZE;
    if (dtype == BROLM_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        int by = (inter / 8 + 255) / 256;
        if (by > 65535) by = 65535;
        gated_act_vec_kernel<<<dim3(tokens, by), 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, inter, act);
        return launch_status();
    }
    int by = (inter + 1023) / 1024;
    if (by > 65535) by = 65535;
    dim3 grid(tokens, by);
    if (dtype == BROLM_F32)
        gated_act_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, act);
    else if (dtype == BROLM_BF16)
        gated_act_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, inter, act);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}

// ---------------------------------------------------------------------------
// Logits to float with the final soft-cap:  out = cap * tanh(x / cap)
// (src/gemma2.cpp:406-412, one pass instead of three).  In and out may be the
// same float buffer.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ x, float* __restrict__ out, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = soft_cap(to_float(x[i]), cap);
}

BROLM_API int brolm_softcap(const void* x, int dtype, void* out, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    long long blocks = (n + 255) / 256;
    if (blocks > device_sm_count() * 32) blocks = device_sm_count() * 32;
    if (dtype == BROLM_F32)
        softcap_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (float*)out, (size_t)n, cap);
    else if (dtype == BROLM_BF16)
        softcap_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((const bf16*)x, (float*)out, (size_t)n, cap);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}
