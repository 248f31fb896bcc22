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
// ---------------------------------------------------------------------------
template <typename X, typename W, typename O>
__global__ void rmsnorm_kernel(const X* __restrict__ x, const int32_t* __restrict__ rows, const W* __restrict__ w,
                               float eps, float offset, O* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const X* src = x + (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_float(src[i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    O* dst = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = from_float<O>(to_float(src[i]) * inv * (offset + to_float(w[i])));
}

template <typename X, typename W>
static int rmsnorm_out(const void* x, const void* rows, const void* w, float eps, float offset, void* out,
                       int out_dtype, int n, int hidden, cudaStream_t s) {
    if (out_dtype == BROLM_F32)
        rmsnorm_kernel<X, W, float><<<n, 256, 0, s>>>((const X*)x, (const int32_t*)rows, (const W*)w, eps, offset,
                                                      (float*)out, hidden);
    else if (out_dtype == BROLM_BF16)
        rmsnorm_kernel<X, W, bf16><<<n, 256, 0, s>>>((const X*)x, (const int32_t*)rows, (const W*)w, eps, offset,
                                                     (bf16*)out, hidden);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
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
// h is the float residual stream.
// ---------------------------------------------------------------------------
template <typename Y, typename W, typename O>
__global__ void residual_rmsnorm_kernel(float* __restrict__ h, const Y* __restrict__ y, const W* __restrict__ w_post,
                                        float eps_post, float off_post, const W* __restrict__ w_next, float eps_next,
                                        float off_next, O* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * hidden;
    const Y* yr = y + (size_t)r * hidden;
    float inv_post = 1.0f;
    if (w_post) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_float(yr[i]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        inv_post = rsqrtf(ss / (float)hidden + eps_post);
    }
    float ss2 = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_float(yr[i]);
        if (w_post) v = v * inv_post * (off_post + to_float(w_post[i]));
        const float s = hr[i] + v;
        hr[i] = s;
        ss2 += s * s;
    }
    if (!w_next) return;
    ss2 = block_sum(ss2, scratch);
    const float inv_next = rsqrtf(ss2 / (float)hidden + eps_next);
    O* dst = out + (size_t)r * hidden;
    // every thread reads back only what it wrote itself
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        dst[i] = from_float<O>(hr[i] * inv_next * (off_next + to_float(w_next[i])));
}

template <typename Y, typename W>
static int residual_out(void* h, const void* y, const void* w_post, float eps_post, float off_post,
                        const void* w_next, float eps_next, float off_next, void* out, int out_dtype, int n,
                        int hidden, cudaStream_t s) {
    if (out_dtype == BROLM_F32)
        residual_rmsnorm_kernel<Y, W, float><<<n, 256, 0, s>>>((float*)h, (const Y*)y, (const W*)w_post, eps_post,
                                                               off_post, (const W*)w_next, eps_next, off_next,
                                                               (float*)out, hidden);
    else if (out_dtype == BROLM_BF16)
        residual_rmsnorm_kernel<Y, W, bf16><<<n, 256, 0, s>>>((float*)h, (const Y*)y, (const W*)w_post, eps_post,
                                                              off_post, (const W*)w_next, eps_next, off_next,
                                                              (bf16*)out, hidden);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}

// w_post and w_next share one element type (w_dtype); either may be null.
BROLM_API int brolm_residual_rmsnorm(void* h, const void* y, int y_dtype, const void* w_post, float eps_post,
                                     float off_post, const void* w_next, float eps_next, float off_next,
                                     int w_dtype, void* out, int out_dtype, int n, int hidden,
                                     cudaStream_t stream) {
    if (n <= 0) return BROLM_OK;
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_F32)
        return residual_out<float, float>(h, y, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                          out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_F32 && w_dtype == BROLM_BF16)
        return residual_out<float, bf16>(h, y, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                         out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_F32)
        return residual_out<bf16, float>(h, y, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
                                         out_dtype, n, hidden, stream);
    if (y_dtype == BROLM_BF16 && w_dtype == BROLM_BF16)
        return residual_out<bf16, bf16>(h, y, w_post, eps_post, off_post, w_next, eps_next, off_next, out,
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
// Token t belongs to batch row tok_seq[t] and stands at positions[t]; a
// negative position marks a padding row, which is left untouched.  The cache
// of this layer is k_pages/v_pages [page][kv_head][page_size][hd]; position p
// lives at ring index p % ring in page page_table[row][(p % ring)/page_size].
// Positions older than kv_len[row] - ring are not written: a later position of
// the same step owns their place.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const int32_t* __restrict__ tok_seq, const float2* __restrict__ cos_sin,
                                     int n_q, int n_kv, int hd, int rot, T* __restrict__ k_pages,
                                     T* __restrict__ v_pages, const int32_t* __restrict__ page_table, int pt_stride,
                                     const int32_t* __restrict__ kv_len, int ring, int page_size) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos < 0) return;
    const int row_stride = (n_q + 2 * n_kv) * hd;
    T* row = qkv + (size_t)t * row_stride;
    const int half = rot >> 1;

    if (cos_sin) {
        const float2* cs = cos_sin + (size_t)pos * half;
        const int pairs = (n_q + n_kv) * half;
        for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
            const int head = idx / half, i = idx - head * half;
            T* p = row + head * hd;
            const float a = to_float(p[i]), b = to_float(p[i + half]);
            const float2 c = cs[i];
            p[i] = from_float<T>(a * c.x - b * c.y);
            p[i + half] = from_float<T>(a * c.y + b * c.x);
        }
    }
    if (!k_pages) return;
    const int b = tok_seq[t];
    if (pos < kv_len[b] - ring) return;
    __syncthreads();   // the rotated k of this row is complete
    const int ridx = pos % ring;
    const int page = page_table[(size_t)b * pt_stride + ridx / page_size];
    const int off = ridx % page_size;
    const T* ksrc = row + n_q * hd;
    const T* vsrc = ksrc + n_kv * hd;
    for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx - g * hd;
        const size_t dst = (((size_t)page * n_kv + g) * page_size + off) * hd + d;
        k_pages[dst] = ksrc[idx];
        v_pages[dst] = vsrc[idx];
    }
}

BROLM_API int brolm_rope_kv_write(void* qkv, int dtype, const void* positions, const void* tok_seq,
                                  const void* cos_sin, int n_q, int n_kv, int hd, int rot, void* k_pages,
                                  void* v_pages, const void* page_table, int pt_stride, const void* kv_len, int ring,
                                  int page_size, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (rot > hd || (rot & 1) || ring <= 0 || page_size <= 0 || ring % page_size != 0) return BROLM_ERR_BAD_SIZE;
    if (dtype == BROLM_F32)
        rope_kv_write_kernel<float><<<tokens, 256, 0, stream>>>(
            (float*)qkv, (const int32_t*)positions, (const int32_t*)tok_seq, (const float2*)cos_sin, n_q, n_kv, hd,
            rot, (float*)k_pages, (float*)v_pages, (const int32_t*)page_table, pt_stride, (const int32_t*)kv_len,
            ring, page_size);
    else if (dtype == BROLM_BF16)
        rope_kv_write_kernel<bf16><<<tokens, 256, 0, stream>>>(
            (bf16*)qkv, (const int32_t*)positions, (const int32_t*)tok_seq, (const float2*)cos_sin, n_q, n_kv, hd,
            rot, (bf16*)k_pages, (bf16*)v_pages, (const int32_t*)page_table, pt_stride, (const int32_t*)kv_len, ring,
            page_size);
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

BROLM_API int brolm_gated_act(const void* gate_up, void* out, int dtype, int tokens, int inter, int act,
                              cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (act < 0 || act > 1) return BROLM_ERR_BAD_SIZE;
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
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == BROLM_F32)
        softcap_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (float*)out, (size_t)n, cap);
    else if (dtype == BROLM_BF16)
        softcap_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((const bf16*)x, (float*)out, (size_t)n, cap);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}
