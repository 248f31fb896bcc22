// Soft-capped, windowed, causal grouped-query attention on CUDA cores, for
// float and bfloat16 elements, with every product, score and sum in float.
//
// This is the exact path: the float model uses it for prompts and for
// decoding, and it is the reference the tensor-core kernels are checked
// against.  One block handles one (sequence, kv head) and a tile of 32
// "rows"; a row is a (query token, query head of the group) pair, so all
// query heads that share a kv head reuse the same staged keys and values.
//
// Keys come either from the packed projection output of this step
// (prompts: sequence b owns rows cu_q[b] .. cu_q[b+1]) or from the paged
// cache (decoding).  The key loop walks tiles of 32 keys anchored at
// multiples of 32 of the absolute position, and folds them in ascending
// order with one online-softmax update per tile.  The order of operations for
// one query therefore does not depend on how the tokens were cut into steps
// or on what else is in the batch: a prompt pass and a decode pass give the
// same bits for the same inputs.
//
// Scores follow wlejon/brolm src/gemma2.cpp:360-367: s = (q.k) * scale, then
// cap * tanh(s / cap), then the mask, then softmax.  Key j is visible from a
// query at position p iff 0 <= p - j < window (window <= 0: no window).
#include "common.cuh"

namespace {

constexpr int ROWS = 32;         // rows per block
constexpr int KT = 32;           // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int RPW = ROWS / WARPS;  // rows per warp

struct AttnArgs {
    const void* q;            // [tokens, q_stride] elements; head h at h*hd
    void* out;                // [tokens, out_stride]
    int q_stride, out_stride;
    const int32_t* cu_q;      // [B+1] first packed row of each sequence
    const int32_t* kv_len;    // [B] keys of each sequence after this step
    // packed source
    const void* k;            // [tokens, kv_stride]; kv head g at g*hd
    const void* v;
    int kv_stride;
    // paged source
    const void* k_pages;      // [page][n_kv][page_size][hd]
    const void* v_pages;
    const int32_t* page_table;
    int pt_stride, ring, page_size;
    int n_kv, group, hd;
    float scale, cap;
    int window;
};

// DPL: output dims per lane = ceil(hd / 32) rounded up to the instantiated size.
template <typename T, int DPL, bool PAGED>
__global__ void __launch_bounds__(WARPS * 32) attn_simt_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int hd = a.hd;
    const int qs = hd + 4;                 // padded stride of q and k rows (floats)
    float* Qs = smem;                      // [ROWS][qs]
    float* Ks = Qs + ROWS * qs;            // [KT][qs]
    float* Vs = Ks + KT * qs;              // [KT][hd]

    const int b = blockIdx.z, g = blockIdx.y;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int kv_len = a.kv_len[b];
    const int n_rows = q_len * a.group;
    const int row0 = blockIdx.x * ROWS;
    if (row0 >= n_rows || kv_len <= 0) return;
    const int rows_here = min(ROWS, n_rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int first_pos = kv_len - q_len;            // position of the sequence's first query
    const int window = a.window > 0 ? a.window : 0x3fffffff;

    // stage the queries of this tile as floats
    const T* qg = (const T*)a.q;
    for (int idx = threadIdx.x; idx < ROWS * (hd / 8); idx += blockDim.x) {
        const int r = idx / (hd / 8), c = (idx - r * (hd / 8)) * 8;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (r < rows_here) {
            const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
            load8(qg + (size_t)(q0 + tok) * a.q_stride + head * hd + c, v);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) Qs[r * qs + c + i] = v[i];
    }

    // key range of the whole tile
    const int tok_lo = row0 / a.group, tok_hi = (row0 + rows_here - 1) / a.group;
    const int pos_lo = first_pos + tok_lo, pos_hi = first_pos + tok_hi;
    const int key_lo = max(0, pos_lo - window + 1), key_hi = pos_hi;   // inclusive

    // per-row state of this warp
    int rpos[RPW];
    float m[RPW], l[RPW], acc[RPW][DPL];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        rpos[i] = r < rows_here ? first_pos + (row0 + r) / a.group : -1;
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[i][d] = 0.0f;
    }

    for (int t0 = (key_lo / KT) * KT; t0 <= key_hi; t0 += KT) {
        __syncthreads();   // the tile before this one is consumed (and Qs is written, first time)
        // stage keys and values t0 .. t0+KT-1; places outside [key_lo, key_hi] read as zero
        for (int idx = threadIdx.x; idx < KT * (hd / 8); idx += blockDim.x) {
            const int j = idx / (hd / 8), c = (idx - j * (hd / 8)) * 8;
            const int kp = t0 + j;
            float kv[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (kp >= key_lo && kp <= key_hi) {
                if (PAGED) {
                    const int ridx = kp % a.ring;
                    const int page = a.page_table[(size_t)b * a.pt_stride + ridx / a.page_size];
                    const size_t off = (((size_t)page * a.n_kv + g) * a.page_size + ridx % a.page_size) * hd + c;
                    load8((const T*)a.k_pages + off, kv);
                    load8((const T*)a.v_pages + off, vv);
                } else {
                    const size_t off = (size_t)(q0 + kp) * a.kv_stride + g * hd + c;
                    load8((const T*)a.k + off, kv);
                    load8((const T*)a.v + off, vv);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                Ks[j * qs + c + i] = kv[i];
                Vs[j * hd + c + i] = vv[i];
            }
        }
        __syncthreads();

        // scores: lane j holds key t0 + j
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.0f;
        const float* kr = Ks + lane * qs;
        for (int c = 0; c < hd; c += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(kr + c);
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(Qs + (warp * RPW + i) * qs + c);
                s[i] = fmaf(qq.x, kk.x, s[i]);
                s[i] = fmaf(qq.y, kk.y, s[i]);
                s[i] = fmaf(qq.z, kk.z, s[i]);
                s[i] = fmaf(qq.w, kk.w, s[i]);
            }
        }
        const int kp = t0 + lane;
        float p[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const bool visible = rpos[i] >= 0 && kp <= rpos[i] && rpos[i] - kp < window;
            const float sc = visible ? soft_cap(s[i] * a.scale, a.cap) : -INFINITY;
            const float tile_max = warp_max(sc);
            const float m_new = fmaxf(m[i], tile_max);
            float corr = 1.0f;
            p[i] = 0.0f;
            if (m_new > -INFINITY) {
                corr = expf(m[i] - m_new);           // m[i] = -inf gives 0
                p[i] = visible ? expf(sc - m_new) : 0.0f;
            }
            l[i] = l[i] * corr + warp_sum(p[i]);
            m[i] = m_new;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[i][d] *= corr;
        }
        // acc[row][d] += sum_j p[row][j] * V[j][d], keys in ascending order
        for (int j = 0; j < KT; ++j) {
            float vj[DPL];
#pragma unroll
            for (int d = 0; d < DPL; ++d) {
                const int dim = lane + 32 * d;
                vj[d] = dim < hd ? Vs[j * hd + dim] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const float pj = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[i][d] = fmaf(pj, vj[d], acc[i][d]);
            }
        }
    }

    T* og = (T*)a.out;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp * RPW + i;
        if (r >= rows_here) continue;
        const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
        const float inv = l[i] > 0.0f ? 1.0f / l[i] : 0.0f;
        T* dst = og + (size_t)(q0 + tok) * a.out_stride + head * hd;
#pragma unroll
        for (int d = 0; d < DPL; ++d) {
            const int dim = lane + 32 * d;
            if (dim < hd) dst[dim] = from_float<T>(acc[i][d] * inv);
        }
    }
}

template <typename T, int DPL>
int launch(const AttnArgs& a, bool paged, int batch, int max_q_len, cudaStream_t stream) {
    const size_t smem = (size_t)((ROWS + KT) * (a.hd + 4) + KT * a.hd) * sizeof(float);
    if (smem > 227 * 1024) return BROLM_ERR_TOO_LARGE;
    dim3 grid((max_q_len * a.group + ROWS - 1) / ROWS, a.n_kv, batch);
    static size_t allowed[2] = {0, 0};        // raised once per size, not at every launch
    if (smem > allowed[paged]) {
        cudaError_t e = paged ? cudaFuncSetAttribute(attn_simt_kernel<T, DPL, true>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                              : cudaFuncSetAttribute(attn_simt_kernel<T, DPL, false>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed[paged] = smem;
    }
    if (paged)
        attn_simt_kernel<T, DPL, true><<<grid, WARPS * 32, smem, stream>>>(a);
    else
        attn_simt_kernel<T, DPL, false><<<grid, WARPS * 32, smem, stream>>>(a);
    return launch_status();
}

template <typename T>
int dispatch(const AttnArgs& a, bool paged, int batch, int max_q_len, cudaStream_t stream) {
    const int dpl = (a.hd + 31) / 32;
    if (dpl <= 1) return launch<T, 1>(a, paged, batch, max_q_len, stream);
    if (dpl <= 2) return launch<T, 2>(a, paged, batch, max_q_len, stream);
    if (dpl <= 4) return launch<T, 4>(a, paged, batch, max_q_len, stream);
    if (dpl <= 8) return launch<T, 8>(a, paged, batch, max_q_len, stream);
    if (dpl <= 16) return launch<T, 16>(a, paged, batch, max_q_len, stream);
    return BROLM_ERR_TOO_LARGE;
}

}  // namespace

// head_dim must be a multiple of 8 and at most 512; strides and the offsets of
// heads must keep 8 elements in one aligned 16-byte (bf16) or 32-byte (float)
// span, which holds when every stride is a multiple of 8.
BROLM_API int brolm_attn_simt(int dtype, const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                              const void* kv_len, const void* k, const void* v, int kv_stride, const void* k_pages,
                              const void* v_pages, const void* page_table, int pt_stride, int ring, int page_size,
                              int n_kv, int group, int hd, float scale, float cap, int window, int batch,
                              int max_q_len, cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    if (hd <= 0 || hd % 8 != 0 || hd > 512 || group <= 0 || n_kv <= 0) return BROLM_ERR_BAD_SIZE;
    if (q_stride % 8 != 0 || out_stride % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (batch > 65535 || n_kv > 65535) return BROLM_ERR_TOO_LARGE;
    const bool paged = k_pages != nullptr;
    if (paged) {
        if (ring <= 0 || page_size <= 0 || page_size % KT != 0 || ring % page_size != 0) return BROLM_ERR_BAD_SIZE;
    } else {
        if (!k || !v || kv_stride % 8 != 0) return BROLM_ERR_ALIGNMENT;
    }
    AttnArgs a;
    a.q = q; a.out = out; a.q_stride = q_stride; a.out_stride = out_stride;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len;
    a.k = k; a.v = v; a.kv_stride = kv_stride;
    a.k_pages = k_pages; a.v_pages = v_pages; a.page_table = (const int32_t*)page_table;
    a.pt_stride = pt_stride; a.ring = ring; a.page_size = page_size;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window;
    if (dtype == BROLM_F32) return dispatch<float>(a, paged, batch, max_q_len, stream);
    if (dtype == BROLM_BF16) return dispatch<bf16>(a, paged, batch, max_q_len, stream);
    return BROLM_ERR_BAD_DTYPE;
}
