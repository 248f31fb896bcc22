// Matrix product for a handful of tokens:  Y[M,N] = X[M,K] * W[N,K]^T with
// M <= 16, bfloat16 operands, float accumulation (decode steps).
//
// With so few tokens the product only has to stream W from memory once, so
// the kernel is built around that stream.  The roles of the operands are
// swapped for the tensor cores: 16 rows of W fill the M side of an
// mma.sync m16n8k16, 8 tokens fill the N side.  Every thread fetches its own
// fragments in 16-byte pieces: the four lanes of a quad read 8 consecutive k
// each (32 k in all), which is two k16 steps of the instruction under a fixed
// permutation of k that X is loaded with as well, so no ldmatrix and no
// exchange between threads is needed on the way in.
//
// A block owns a few 16-row tiles of W over the whole of K; its 8 warps take
// interleaved 64-wide blocks of K.  The weights of the next DEPTH blocks of a
// warp are in flight at any time: cp.async copies each thread's pieces into a
// slot of shared memory that only this thread reads back (a queue per thread,
// no barrier), which is what it takes to keep the memory busy at the latency
// it has.  The warps add their partial sums in shared memory in warp order (the result does not
// depend on scheduling).  Epilogues: plain store (bfloat16 or float), the
// gated activation act(gate) * up for W = [Wg; Wu] (wlejon/brolm
// src/gemma2.cpp:378-381), cap * tanh(y / cap) into float logits
// (src/gemma2.cpp:406-412), or, for the fused q/k/v projection, the rotary
// position encoding of q and k with the write of k and v into the paged cache
// (src/gemma2.cpp:355-356): a tile then holds eight (i, i + hd/2) pairs of one
// head, rows i in its first eight rows and rows i + hd/2 in the other eight,
// so that both elements of a pair meet in one thread.
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int KB = 64;     // k per warp iteration
// Blocks of K whose weights a warp has in flight; the queue has one slot more.  A slot of a block is
// MT * 16 KB: three blocks of 64 KB (MT 1) or two of 96 KB (MT 2) share an SM, one of 192 KB (MT 4) has it alone.
template <int MT> __host__ __device__ constexpr int depth() { return MT == 1 ? 3 : 2; }
template <int MT> __host__ __device__ constexpr size_t queue_bytes() { return (size_t)(depth<MT>() + 1) * WARPS * (4 * MT) * 32 * 16; }

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes from global memory into this thread's slot of the queue (zeros when !ok)
__device__ __forceinline__ void copy16(uint32_t dst, const bf16* p, bool ok) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(p), "r"(ok ? 16 : 0) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg16_cached(const bf16* p, bool ok) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ok) v = *reinterpret_cast<const uint4*>(p);
    return v;
}

__device__ __forceinline__ float act_apply(float z, int act) {
    if (act == 0) {
        const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
        return 0.5f * z * (1.0f + tanhf(u));
    }
    return z / (1.0f + expf(-z));
}

enum : int { EPI_STORE = 0, EPI_GATED = 1, EPI_SOFTCAP = 2, EPI_ROPE = 3 };

struct SkinnyArgs {
    const bf16* x;
    const bf16* w;
    void* y;
    int ldx, ldw, ldy;
    int M, N, K;          // N: rows of W used as outputs (EPI_GATED: W has 2N rows, gate then up)
    int out_f32;
    int act;
    float cap;
    int ksplit;           // blocks along K; > 1: block (x, s) writes float partial sums to y + s * part_stride
    long long part_stride;
    // EPI_ROPE: W = [Wq; Wk; Wv], heads of hd rows; y is the bfloat16 q/k/v row of a token
    const int32_t* positions;     // < 0: a padding row, nothing is written for it
    const float2* cos_sin;        // [position][hd / 2] (cos, sin); null: no rotation
    int n_q, n_kv, hd;
    bf16* k_pages;                // [page][kv head][page_size][hd]; null: nothing is kept
    bf16* v_pages;
    const int32_t* cache_rows;    // page * page_size + place of a token, < 0: not kept
    int page_size;
};

// MT: 16-row tiles of W per block.  NT: 8-token tiles.
template <int MT, int NT, int EPI>
__global__ void __launch_bounds__(WARPS * 32) skinny_kernel(SkinnyArgs a) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int q = lane & 3, r = lane >> 2;
    constexpr int OUT_TILES = EPI == EPI_GATED ? MT / 2 : MT;      // 16-column tiles of Y per block
    const int n0 = blockIdx.x * OUT_TILES * 16;

    // first row of W of each tile
    // (EPI_ROPE: tile t of the grid is pairs 8j .. 8j + 7 of head h, t = h * (hd / 16) + j; its rows
    // 8 .. 15 are the partners hd / 2 further on)
    int wrow[MT];
    const int half = EPI == EPI_ROPE ? a.hd >> 1 : 8;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        if (EPI == EPI_ROPE) {
            const int t = blockIdx.x * MT + i, per_head = a.hd >> 4;
            wrow[i] = (t / per_head) * a.hd + (t % per_head) * 8;
        } else {
            wrow[i] = EPI == EPI_GATED ? ((i & 1) ? a.N : 0) + n0 + 16 * (i >> 1) : n0 + 16 * i;
        }
    }
    const int w_rows = EPI == EPI_GATED ? 2 * a.N : a.N;
    const int n_limit = a.N;                                       // output columns that exist

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

    const int nkb_all = (a.K + KB - 1) / KB;
    const int per = (nkb_all + a.ksplit - 1) / a.ksplit;
    const int kb_first = blockIdx.y * per, nkb = min(nkb_all, kb_first + per);
    uint4 xc[2][NT];                                               // [half of the block][token tile]
    extern __shared__ __align__(16) uint8_t queue_raw[];
    constexpr int DEPTH = depth<MT>();
    constexpr int PIECES = 4 * MT;                                 // 16-byte pieces of a thread per block of K
    const uint32_t queue = (uint32_t)__cvta_generic_to_shared(queue_raw) + (warp * PIECES * 32 + lane) * 16;
    auto slot_of = [&](int n) { return queue + (uint32_t)(n % (DEPTH + 1)) * (WARPS * PIECES * 32 * 16); };

    // asks for the weights of the warp's n-th block of K (block kb); pieces: [half][tile][row r / its partner]
    auto fetch_w = [&](int kb, int n) {
        const uint32_t dst = slot_of(n);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = kb * KB + h * 32 + q * 8;
            const bool kok = kb < nkb && kk < a.K;                  // K is a multiple of 8
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const int col = (EPI == EPI_GATED ? wrow[i] - ((i & 1) ? a.N : 0) : wrow[i]) + r;   // output column of row r
                const bool ok0 = kok && col < n_limit, ok1 = kok && col + half < n_limit;
                copy16(dst + ((h * MT + i) * 2) * 512, a.w + (ok0 ? (size_t)(wrow[i] + r) * a.ldw + kk : 0), ok0);
                copy16(dst + ((h * MT + i) * 2 + 1) * 512, a.w + (ok1 ? (size_t)(wrow[i] + r + half) * a.ldw + kk : 0), ok1);
            }
        }
    };
    auto load_x = [&](int kb, uint4 (&xv)[2][NT]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = kb * KB + h * 32 + q * 8;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int tok = j * 8 + r;
                xv[h][j] = ldg16_cached(a.x + (size_t)tok * a.ldx + kk, kk < a.K && tok < a.M);
            }
        }
    };
    (void)w_rows;

    // EPI_ROPE: what this thread's (pair, token) of the epilogue needs from memory — the token's position and
    // place in the cache (written by the host for this step, not by the kernel before) and the pair's
    // (cos, sin) — is fetched now, so that the epilogue waits for nothing.
    constexpr int ROPE_PAIRS = MT * NT * 2 * 32;
    static_assert(EPI != EPI_ROPE || ROPE_PAIRS <= WARPS * 32, "one (pair, token) per thread");
    int rope_pos = -1, rope_crow = -1;
    float2 rope_cs = make_float2(1.0f, 0.0f);
    if constexpr (EPI == EPI_ROPE) {
        if ((int)threadIdx.x < ROPE_PAIRS) {
            const int idx = threadIdx.x;
            const int ln = idx & 31, e = (idx >> 5) & 1, j = (idx >> 6) % NT, i = (idx >> 6) / NT;
            const int tok = j * 8 + (ln & 3) * 2 + e, col = wrow[i] + (ln >> 2);
            if (tok < a.M && col < n_limit) {
                rope_pos = a.positions[tok];
                if (rope_pos >= 0) {
                    const int head = col / a.hd, within = col - head * a.hd;
                    const bool is_v = head >= a.n_q + a.n_kv;
                    if (!is_v && a.cos_sin) rope_cs = a.cos_sin[(size_t)rope_pos * half + within];
                    if (head >= a.n_q && a.k_pages) rope_crow = a.cache_rows[tok];
                }
            }
        }
    }

    // The weights depend on nothing that ran before: the first DEPTH blocks are asked for while the
    // kernel before this one is still finishing; X is its output and has to wait.
    const int kb0 = kb_first + warp;
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
        fetch_w(kb0 + d * WARPS, d);
        copy_commit();
    }
    pdl_wait();
    if (kb0 < nkb) load_x(kb0, xc);
    int n = 0;
    for (int kb = kb0; kb < nkb; kb += WARPS, ++n) {
        uint4 xn[2][NT];
        const bool more = kb + WARPS < nkb;
        if (more) load_x(kb + WARPS, xn);
        // block n + DEPTH goes into the slot that block n - 1 was read from
        fetch_w(kb + DEPTH * WARPS, n + DEPTH);
        copy_commit();
        copy_wait<DEPTH>();                                         // block n has landed
        const uint32_t src = slot_of(n);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const uint4 w0 = lds16(src + ((h * MT + i) * 2) * 512), w1 = lds16(src + ((h * MT + i) * 2 + 1) * 512);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16(acc[i][j], w0.x, w1.x, w0.y, w1.y, xc[h][j].x, xc[h][j].y);
                    mma_bf16(acc[i][j], w0.z, w1.z, w0.w, w1.w, xc[h][j].z, xc[h][j].w);
                }
            }
        }
        if (more) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < NT; ++j) xc[h][j] = xn[h][j];
        }
    }
    copy_wait<0>();

    // The stream of weights is over: the next kernel may take its place on the SMs now.  (Letting it in
    // earlier packs its blocks onto the few SMs that happen to have room, and they then run unevenly.)
    pdl_trigger();

    // partial sums of the warps -> shared memory (the queue is drained and free), then summed in warp order
    static_assert(sizeof(float) * WARPS * MT * NT * 4 * 32 <= queue_bytes<MT>(), "the sums fit where the queue was");
    float (*red)[MT * NT * 4][32] = reinterpret_cast<float (*)[MT * NT * 4][32]>(queue_raw);
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[warp][(i * NT + j) * 4 + e][lane] = acc[i][j][e];
    __syncthreads();

    if (EPI == EPI_ROPE) {
        // one (pair, token) per thread: e & 1 picks the token, rows r and r + 8 are the pair
        if ((int)threadIdx.x < ROPE_PAIRS && rope_pos >= 0) {
            const int idx = threadIdx.x;
            const int ln = idx & 31, e = (idx >> 5) & 1, j = (idx >> 6) % NT, i = (idx >> 6) / NT;
            const int tok = j * 8 + (ln & 3) * 2 + e;
            const int col = wrow[i] + (ln >> 2);                    // first element of the pair in the q/k/v row
            float va = 0.0f, vb = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                va += red[w][(i * NT + j) * 4 + e][ln];
                vb += red[w][(i * NT + j) * 4 + e + 2][ln];
            }
            const int head = col / a.hd, within = col - head * a.hd;
            const bool is_v = head >= a.n_q + a.n_kv, is_k = !is_v && head >= a.n_q;
            if (!is_v && a.cos_sin) {
                const float ra = va * rope_cs.x - vb * rope_cs.y, rb = va * rope_cs.y + vb * rope_cs.x;
                va = ra;
                vb = rb;
            }
            const bf16 qa = __float2bfloat16_rn(va), qb = __float2bfloat16_rn(vb);
            bf16* y = reinterpret_cast<bf16*>(a.y) + (size_t)tok * a.ldy + col;
            y[0] = qa;
            y[half] = qb;
            if (rope_crow >= 0) {
                const int kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
                bf16* dst = (is_k ? a.k_pages : a.v_pages) +
                            (((size_t)(rope_crow / a.page_size) * a.n_kv + kvh) * a.page_size + rope_crow % a.page_size) * a.hd +
                            within;
                dst[0] = qa;
                dst[half] = qb;
            }
        }
        return;
    }

    constexpr int OUT_ELEMS = OUT_TILES * NT * 4 * 32;
    for (int idx = threadIdx.x; idx < OUT_ELEMS; idx += WARPS * 32) {
        const int ln = idx & 31, e = (idx >> 5) & 3, j = (idx >> 7) % NT, ot = (idx >> 7) / NT;
        const int col = n0 + ot * 16 + (ln >> 2) + ((e >> 1) << 3);
        const int tok = j * 8 + (ln & 3) * 2 + (e & 1);
        float v;
        if (EPI == EPI_GATED) {
            float gsum = 0.0f, usum = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                gsum += red[w][((2 * ot) * NT + j) * 4 + e][ln];
                usum += red[w][((2 * ot + 1) * NT + j) * 4 + e][ln];
            }
            v = act_apply(gsum, a.act) * usum;
        } else {
            v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += red[w][(ot * NT + j) * 4 + e][ln];
            if (EPI == EPI_SOFTCAP) v = soft_cap(v, a.cap);
        }
        if (col < n_limit && tok < a.M) {
            if (a.ksplit > 1) reinterpret_cast<float*>(a.y)[blockIdx.y * a.part_stride + (size_t)tok * a.ldy + col] = v;
            else if (a.out_f32) reinterpret_cast<float*>(a.y)[(size_t)tok * a.ldy + col] = v;
            else reinterpret_cast<bf16*>(a.y)[(size_t)tok * a.ldy + col] = __float2bfloat16_rn(v);
        }
    }
}

template <int MT, int NT, int EPI>
int launch(const SkinnyArgs& a, cudaStream_t stream) {
    constexpr int cols = (EPI == EPI_GATED ? MT / 2 : MT) * 16;
    dim3 blocks((a.N + cols - 1) / cols, a.ksplit);        // (EPI_ROPE: hd is a multiple of 16, so N is too)
    constexpr size_t smem = queue_bytes<MT>();
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(skinny_kernel<MT, NT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return launch_pdl(skinny_kernel<MT, NT, EPI>, blocks, dim3(WARPS * 32), smem, stream, a);
}

template <int EPI>
int dispatch(const SkinnyArgs& a, int mt, cudaStream_t stream) {
    const int nt = (a.M + 7) / 8;
    if constexpr (EPI == EPI_GATED) {
        // (a gate and an up tile per block; blocks of two pairs measured slower at every size)
        if (nt == 1) return launch<2, 1, EPI>(a, stream);
        return launch<2, 2, EPI>(a, stream);
    } else if constexpr (EPI == EPI_ROPE) {
        if (nt == 1) return mt >= 2 && (a.N / 16) % 2 == 0 ? launch<2, 1, EPI>(a, stream) : launch<1, 1, EPI>(a, stream);
        return mt >= 2 && (a.N / 16) % 2 == 0 ? launch<2, 2, EPI>(a, stream) : launch<1, 2, EPI>(a, stream);
    } else {
        if (nt == 1) return mt >= 4 ? launch<4, 1, EPI>(a, stream) : mt >= 2 ? launch<2, 1, EPI>(a, stream) : launch<1, 1, EPI>(a, stream);
        return mt >= 4 ? launch<4, 2, EPI>(a, stream) : mt >= 2 ? launch<2, 2, EPI>(a, stream) : launch<1, 2, EPI>(a, stream);
    }
}

}  // namespace

// epilogue 0: Y = X W^T (bfloat16, or float when out_f32); 1: Y = act(X Wg^T) * (X Wu^T) with
// W = [Wg; Wu] of 2N rows; 2: Y = cap * tanh(X W^T / cap), float.  M <= 16; K a multiple of 8;
// rows of X and W 16-byte aligned.  tiles: 16-row tiles of W per block (1, 2 or 4; epilogue 1 always takes 2).
// ksplit > 1 (epilogue 0 only): K is cut into ksplit slices, slice s writes its float partial
// sums at y + s * part_stride (elements); the reader adds the slices in order.
// The fused q/k/v projection of at most 16 tokens with the rotary position encoding and the write of
// k and v into the paged cache as its epilogue.  W = [Wq; Wk; Wv] ((n_q + 2 n_kv) * hd rows, hd a
// multiple of 16), y the bfloat16 q/k/v rows.  The rotation covers the whole head (pairs i, i + hd/2);
// cos_sin null: no rotation; k_pages null: nothing is kept.
BROLM_API int brolm_skinny_qkv_rope(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int K,
                                    const void* positions, const void* cos_sin, int n_q, int n_kv, int hd,
                                    void* k_pages, void* v_pages, const void* cache_rows, int page_size, int tiles,
                                    cudaStream_t stream) {
    if (M <= 0) return BROLM_OK;
    if (M > 16) return BROLM_ERR_TOO_LARGE;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return BROLM_ERR_ALIGNMENT;
    if (hd <= 0 || hd % 16 != 0 || n_q <= 0 || n_kv <= 0 || page_size <= 0) return BROLM_ERR_BAD_SIZE;
    if (k_pages && (!v_pages || !cache_rows)) return BROLM_ERR_BAD_SIZE;
    SkinnyArgs a;
    a.x = (const bf16*)x; a.w = (const bf16*)w; a.y = y; a.ldx = ldx; a.ldw = ldw; a.ldy = ldy;
    a.M = M; a.N = (n_q + 2 * n_kv) * hd; a.K = K; a.out_f32 = 0; a.act = 0; a.cap = 0.0f;
    a.ksplit = 1; a.part_stride = 0;
    a.positions = (const int32_t*)positions; a.cos_sin = (const float2*)cos_sin;
    a.n_q = n_q; a.n_kv = n_kv; a.hd = hd;
    a.k_pages = (bf16*)k_pages; a.v_pages = (bf16*)v_pages; a.cache_rows = (const int32_t*)cache_rows;
    a.page_size = page_size;
    return dispatch<EPI_ROPE>(a, tiles, stream);
}

BROLM_API int brolm_skinny_gemm(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
                                int epilogue, int out_f32, int act, float cap, int tiles, int ksplit,
                                long long part_stride, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BROLM_OK;
    if (M > 16) return BROLM_ERR_TOO_LARGE;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return BROLM_ERR_ALIGNMENT;
    if (epilogue == EPI_GATED && (act < 0 || act > 1)) return BROLM_ERR_BAD_SIZE;
    SkinnyArgs a;
    a.x = (const bf16*)x; a.w = (const bf16*)w; a.y = y; a.ldx = ldx; a.ldw = ldw; a.ldy = ldy;
    a.M = M; a.N = N; a.K = K; a.out_f32 = out_f32; a.act = act; a.cap = cap;
    if (ksplit < 1 || ksplit > 64 || (ksplit > 1 && epilogue != EPI_STORE)) return BROLM_ERR_BAD_SIZE;
    a.ksplit = ksplit; a.part_stride = part_stride;
    a.positions = nullptr; a.cos_sin = nullptr; a.n_q = a.n_kv = a.hd = 0; a.k_pages = a.v_pages = nullptr;
    a.cache_rows = nullptr; a.page_size = 0;
    if (epilogue == EPI_STORE) return dispatch<EPI_STORE>(a, tiles, stream);
    if (epilogue == EPI_GATED) return dispatch<EPI_GATED>(a, tiles, stream);
    if (epilogue == EPI_SOFTCAP) { a.out_f32 = 1; return dispatch<EPI_SOFTCAP>(a, tiles, stream); }
    return BROLM_ERR_BAD_SIZE;
}
