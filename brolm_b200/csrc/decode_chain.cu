// A decode step as chains of operations inside one persistent kernel (sm_100a).
//
// With a handful of tokens every matrix product of a layer is a stream of
// weights from memory, and what a kernel boundary costs (the stream drains, the
// next kernel ramps up) is of the order of the products themselves.  This
// kernel runs a LIST of operations with one block per SM and keeps the weight
// stream going across them:
//
//   GEMM   Y = X W^T on tcgen05 with the operands swapped (128 rows of W fill
//          the M side, up to 16 tokens the N side), W and X tiles through a
//          ring of TMA stages, accumulators in tensor memory.  Results: float
//          partial sums of K slices, the gated activation act(X Wg^T) * (X Wu^T)
//          in bfloat16, or float with the tanh soft-cap.
//   NORM   h += rmsnorm(sum of partial sums; w_post);  out = rmsnorm(h; w_next)
//          on the float residual stream (wlejon/brolm src/gemma2.cpp:372-376,
//          385-386, :349 of the next layer); block r does row r.
//   ROPE   adds the partial sums of the fused q/k/v product, rotates q and k
//          (src/gemma2.cpp:355-356), writes all three in bfloat16 and k, v into
//          the paged cache.
//
// Between two operations the blocks meet at a barrier in global memory.  The
// warp that loads W does not take part in it: weights depend on nothing, so it
// runs ahead through the whole list as far as the ring has room, and the next
// product's weights are in shared memory when the barrier opens.
//
//   warp 0     one thread: TMA loads of W tiles (128 x 64), all operations ahead
//   warp 1     one thread: tcgen05.mma into one of two accumulators
//   warp 2     one thread: TMA loads of the X tiles (16 x 64) of an operation,
//              once the barrier before that operation has opened
//   warps 3-6  epilogues of GEMM items, NORM and ROPE work, and the barrier
//
// Every wait is bounded: mbarrier waits by tc::mbar_wait, the barrier between
// operations by the same clock limit.  A wait that runs out raises the block's
// give-up flag and a flag in global memory that the other blocks poll; every
// role then leaves its loops, the loaders let their copies land, the tensor
// memory is freed and the kernel returns with an error word set.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BR = 128, BK = 64, BT = 16;
constexpr int W_BYTES = BR * BK * 2, X_BYTES = BT * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int STAGES = 11;
constexpr int THREADS = 224, VEC0 = 96, VEC = 128;
constexpr int TMEM_COLS = 32;
constexpr int MAX_PARTS = 8;            // K slices whose partial sums a NORM or ROPE operation adds
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 64 + 64 * BT * 4;

enum : int { OP_GEMM = 0, OP_NORM = 1, OP_ROPE = 2 };
enum : int { EPI_PARTS = 0, EPI_GATED = 1, EPI_SOFTCAP = 2 };

// One operation: 32 eight-byte fields (integers as they are, floats as doubles,
// pointers as addresses), written by the host once per model and cache.
enum : int {
    F_KIND = 0, F_EPI, F_ACT, F_MAP_W, F_MAP_X, F_N, F_K, F_KSPLIT, F_PER, F_ROW_TILES, F_ITEMS, F_LDY,
    F_PART_STRIDE, F_Y, F_CAP,
    F_H, F_PARTS, F_N_PARTS, F_IN_STRIDE, F_HIDDEN, F_W_POST, F_EPS_POST, F_OFF_POST, F_W_NEXT, F_EPS_NEXT,
    F_OFF_NEXT, F_OUT,
    F_COS_SIN, F_K_PAGES, F_V_PAGES, F_HEADS, F_ROPE,        // F_HEADS: n_q | n_kv << 16 | hd << 32; F_ROPE: rot | page << 16 | group << 32
    F_COUNT
};
static_assert(F_COUNT == 32, "an operation has 32 fields");
struct ChainOp { long long f[32]; };

struct ChainArgs {
    const CUtensorMap* maps;
    const ChainOp* ops;
    int first, count, M;
    const int* positions;
    const int* cache_rows[4];
    unsigned* sync;            // [0]: arrivals at the barrier, [1]: a block gave up, [2]: blocks that are through
    long long* trace;          // when given: nanosecond stamps, eight per (block, operation)
};

__device__ __forceinline__ void stamp(const ChainArgs& g, int o, int k) {
    if (g.trace) {
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g.trace[((size_t)blockIdx.x * g.count + o) * 8 + k] = t;
    }
}

__device__ int g_chain_error;

__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_chain_error, code);
}
// after giving up: let a copy in flight land, but do not wait long for one that was never issued
__device__ inline void wait_briefly(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try(bar, parity) && clock64() - t0 < 20000000ll) {}
}
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void vec_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ double as_double(long long v) { return __longlong_as_double(v); }

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// Sum over the 128 threads of warps 3-6, in a fixed order.
__device__ __forceinline__ float vec_sum(float v, float* scratch, int vt) {
    v = warp_sum(v);
    vec_sync();
    if ((vt & 31) == 0) scratch[vt >> 5] = v;
    vec_sync();
    return (scratch[0] + scratch[1]) + (scratch[2] + scratch[3]);
}

__device__ __forceinline__ void gains4(const uint2 r, float off, float (&g)[4]) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    g[0] = off + a.x; g[1] = off + a.y; g[2] = off + b.x; g[3] = off + b.y;
}

// NORM for one row by 128 threads; the row lives in registers (C * 512 >= hidden).
template <int C>
__device__ void norm_row(const ChainOp& op, int row, int vt, float* scratch) {
    const int hidden = (int)op.f[F_HIDDEN], n_parts = (int)op.f[F_N_PARTS];
    const long long in_stride = op.f[F_IN_STRIDE];
    float* h = reinterpret_cast<float*>(op.f[F_H]) + (size_t)row * hidden;
    const float* y = reinterpret_cast<const float*>(op.f[F_PARTS]) + (size_t)row * hidden;
    const bf16* w_post = reinterpret_cast<const bf16*>(op.f[F_W_POST]);
    const bf16* w_next = reinterpret_cast<const bf16*>(op.f[F_W_NEXT]);
    bf16* out = reinterpret_cast<bf16*>(op.f[F_OUT]) + (size_t)row * hidden;
    float v[C][4], res[C][4];
    // the gains are weights and come from memory: ask for them first, packed, so that they are there
    // when the statistics are
    uint2 gp[C], gn[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * VEC + vt) * 4;
        gp[c] = gn[c] = make_uint2(0u, 0u);
        if (i < hidden) {
            if (w_post) gp[c] = *reinterpret_cast<const uint2*>(w_post + i);
            if (w_next) gn[c] = *reinterpret_cast<const uint2*>(w_next + i);
        }
    }
    // every load of a chunk is issued before the first is used: the row comes in a few round trips to the L2
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * VEC + vt) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c][e] = res[c][e] = 0.0f;
        if (i < hidden) {
            float4 t[MAX_PARTS];
#pragma unroll
            for (int s = 0; s < MAX_PARTS; ++s)
                if (s < n_parts) t[s] = ldcg4(y + (size_t)s * in_stride + i);
            const float4 r = ldcg4(h + i);
            res[c][0] = r.x; res[c][1] = r.y; res[c][2] = r.z; res[c][3] = r.w;
#pragma unroll
            for (int s = 0; s < MAX_PARTS; ++s)
                if (s < n_parts) {                            // added in the order of the slices
                    v[c][0] += t[s].x; v[c][1] += t[s].y; v[c][2] += t[s].z; v[c][3] += t[s].w;
                }
        }
    }
    if (w_post && n_parts > 0) {
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) ss += v[c][0] * v[c][0] + v[c][1] * v[c][1] + v[c][2] * v[c][2] + v[c][3] * v[c][3];
        ss = vec_sum(ss, scratch, vt);
        const float inv = rsqrtf(ss / (float)hidden + (float)as_double(op.f[F_EPS_POST]));
        const float off = (float)as_double(op.f[F_OFF_POST]);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int i = (c * VEC + vt) * 4;
            if (i < hidden) {
                float g[4];
                gains4(gp[c], off, g);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[c][e] = v[c][e] * inv * g[e];
            }
        }
    }
    float ss2 = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * VEC + vt) * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            res[c][e] += v[c][e];
            ss2 += res[c][e] * res[c][e];
        }
        if (i < hidden && n_parts > 0) *reinterpret_cast<float4*>(h + i) = make_float4(res[c][0], res[c][1], res[c][2], res[c][3]);
    }
    if (!w_next) return;
    ss2 = vec_sum(ss2, scratch, vt);
    const float inv = rsqrtf(ss2 / (float)hidden + (float)as_double(op.f[F_EPS_NEXT]));
    const float off = (float)as_double(op.f[F_OFF_NEXT]);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (c * VEC + vt) * 4;
        if (i < hidden) {
            float g[4];
            gains4(gn[c], off, g);
            const __nv_bfloat162 lo = __floats2bfloat162_rn(res[c][0] * inv * g[0], res[c][1] * inv * g[1]);
            const __nv_bfloat162 hi = __floats2bfloat162_rn(res[c][2] * inv * g[2], res[c][3] * inv * g[3]);
            uint2 pack;
            pack.x = *reinterpret_cast<const uint32_t*>(&lo);
            pack.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(out + i) = pack;
        }
    }
}

// ROPE for one (token, head) by 128 threads.
__device__ void rope_head(const ChainOp& op, const ChainArgs& g, int t, int head, int vt) {
    const int pos = g.positions[t];
    if (pos < 0) return;                                   // a padding row
    const long long heads = op.f[F_HEADS], rope = op.f[F_ROPE];
    const int n_q = (int)(heads & 0xffff), n_kv = (int)((heads >> 16) & 0xffff), hd = (int)(heads >> 32);
    const int rot = (int)(rope & 0xffff), page = (int)((rope >> 16) & 0xffff), group = (int)(rope >> 32);
    const int width = (n_q + 2 * n_kv) * hd;
    const int n_parts = (int)op.f[F_N_PARTS];
    const long long in_stride = op.f[F_IN_STRIDE];
    const float* src = reinterpret_cast<const float*>(op.f[F_PARTS]) + (size_t)t * width + (size_t)head * hd;
    bf16* dst = reinterpret_cast<bf16*>(op.f[F_OUT]) + (size_t)t * width + (size_t)head * hd;
    const float2* cos_sin = reinterpret_cast<const float2*>(op.f[F_COS_SIN]);
    const bool is_v = head >= n_q + n_kv, is_k = !is_v && head >= n_q;
    const bool rotate = !is_v && cos_sin != nullptr;
    bf16* kept = nullptr;
    if (is_k || is_v) {
        bf16* pages = reinterpret_cast<bf16*>(is_k ? op.f[F_K_PAGES] : op.f[F_V_PAGES]);
        const int crow = pages ? g.cache_rows[group][t] : -1;
        if (crow >= 0) {
            const int kvh = is_k ? head - n_q : head - n_q - n_kv;
            kept = pages + (((size_t)(crow / page) * n_kv + kvh) * page + crow % page) * hd;
        }
    }
    const int half = rot >> 1;
    for (int j = vt; j < (hd >> 1); j += VEC) {
        const bool in_rot = j < half;
        const int e0 = in_rot ? j : rot + 2 * (j - half), e1 = in_rot ? j + half : e0 + 1;
        float pa[MAX_PARTS], pb[MAX_PARTS];
#pragma unroll
        for (int s = 0; s < MAX_PARTS; ++s)
            if (s < n_parts) {
                pa[s] = __ldcg(src + (size_t)s * in_stride + e0);
                pb[s] = __ldcg(src + (size_t)s * in_stride + e1);
            }
        float2 c = make_float2(1.0f, 0.0f);
        if (rotate && in_rot) c = cos_sin[(size_t)pos * half + j];
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_PARTS; ++s)
            if (s < n_parts) {
                a += pa[s];
                b += pb[s];
            }
        if (rotate && in_rot) {
            const float ra = a * c.x - b * c.y, rb = a * c.y + b * c.x;
            a = ra;
            b = rb;
        }
        const bf16 qa = __float2bfloat16_rn(a), qb = __float2bfloat16_rn(b);
        dst[e0] = qa;
        dst[e1] = qb;
        if (kept) {
            kept[e0] = qa;
            kept[e1] = qb;
        }
    }
}

__global__ void __launch_bounds__(THREADS, 1) decode_chain_kernel(const ChainArgs g) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {                      // never seen; refuse rather than compute wrongly
        if (threadIdx.x == 0) atomicCAS(&g_chain_error, 0, 13);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);      // [0] stop, [1] scratch for the drain
    volatile int* phase = reinterpret_cast<volatile int*>(tmem_slot + 3);        // barriers this block has passed
    float* scratch = reinterpret_cast<float*>(tmem_slot + 4);                    // 4 floats
    volatile int* decision = reinterpret_cast<volatile int*>(tmem_slot + 8);     // the vector warps stop together
    float* upx = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tmem_slot) + 64);   // gated: up values, 64 x BT
    const uint32_t stage0 = smem_u32(base);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                   acc_empty0 = acc_full0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 2);                      // the W loader and the X loader
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8 * s, 1);
            mbar_init(acc_empty0 + 8 * s, 4);
        }
        give_up[0] = 0;
        give_up[1] = 0;
        phase[0] = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int G = gridDim.x;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int o = 0; o < g.count && ok; ++o) {
                const ChainOp& op = g.ops[g.first + o];
                if ((int)op.f[F_KIND] != OP_GEMM) continue;
                const CUtensorMap* map = g.maps + op.f[F_MAP_W];
                const int items = (int)op.f[F_ITEMS], row_tiles = (int)op.f[F_ROW_TILES], per = (int)op.f[F_PER];
                const int nkb = ((int)op.f[F_K] + BK - 1) / BK, N = (int)op.f[F_N];
                const bool gated = (int)op.f[F_EPI] == EPI_GATED;
                for (int item = blockIdx.x; item < items && ok; item += G) {
                    const int rt = item % row_tiles, lo = (item / row_tiles) * per, hi = min(nkb, lo + per);
                    for (int kb = lo; kb < hi; ++kb, ++it) {
                        const int s = it % STAGES;
                        ok = wait_on(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 1);
                        if (!ok) break;
                        const uint32_t full = full0 + 8 * s, dst = stage0 + s * STAGE_BYTES;
                        mbar_expect_tx(full, W_BYTES);
                        if (gated) {
                            tma_load_2d(dst, map, kb * BK, rt * 64, full);                     // 64 gate rows
                            tma_load_2d(dst + W_BYTES / 2, map, kb * BK, N + rt * 64, full);   // their 64 up rows
                        } else {
                            tma_load_2d(dst, map, kb * BK, rt * BR, full);
                        }
                    }
                }
            }
            pdl_trigger();                                    // all weights are asked for: the next kernel may move in
            if (*give_up)
                for (int j = max(0, it - STAGES); j < it; ++j) wait_briefly(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
        }
    } else if (warp == 2) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            pdl_wait();
            for (int o = 0; o < g.count && ok; ++o) {
                const ChainOp& op = g.ops[g.first + o];
                if ((int)op.f[F_KIND] != OP_GEMM) continue;
                // X is what the operations before this one wrote: wait for the barrier after them
                const long long t0 = clock64();
                while (phase[0] < o) {
                    if (*give_up) { ok = false; break; }
                    if (clock64() - t0 > WAIT_CYCLES) {
                        *give_up = 1;
                        atomicCAS(&g_chain_error, 0, 6);
                        ok = false;
                        break;
                    }
                }
                if (!ok) break;
                proxy_fence();
                const CUtensorMap* map = g.maps + op.f[F_MAP_X];
                const int items = (int)op.f[F_ITEMS], row_tiles = (int)op.f[F_ROW_TILES], per = (int)op.f[F_PER];
                const int nkb = ((int)op.f[F_K] + BK - 1) / BK;
                for (int item = blockIdx.x; item < items && ok; item += G) {
                    const int lo = (item / row_tiles) * per, hi = min(nkb, lo + per);
                    for (int kb = lo; kb < hi; ++kb, ++it) {
                        const int s = it % STAGES;
                        ok = wait_on(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 7);
                        if (!ok) break;
                        const uint32_t full = full0 + 8 * s;
                        mbar_expect_tx(full, X_BYTES);
                        tma_load_2d(stage0 + s * STAGE_BYTES + W_BYTES, map, kb * BK, 0, full);
                    }
                }
            }
            if (*give_up)
                for (int j = max(0, it - STAGES); j < it; ++j) wait_briefly(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id = idesc_bf16(BR, BT);
            int it = 0, local = 0;
            bool ok = true;
            for (int o = 0; o < g.count && ok; ++o) {
                const ChainOp& op = g.ops[g.first + o];
                if ((int)op.f[F_KIND] != OP_GEMM) continue;
                const int items = (int)op.f[F_ITEMS], row_tiles = (int)op.f[F_ROW_TILES], per = (int)op.f[F_PER];
                const int nkb = ((int)op.f[F_K] + BK - 1) / BK;
                for (int item = blockIdx.x; item < items && ok; item += G, ++local) {
                    const int as = local & 1;
                    ok = wait_on(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, give_up, 5);
                    if (!ok) break;
                    fence_after_sync();
                    const uint32_t acc = tmem + as * BT;
                    const int lo = (item / row_tiles) * per, hi = min(nkb, lo + per);
                    for (int kb = lo; kb < hi; ++kb, ++it) {
                        const int s = it % STAGES;
                        ok = wait_on(full0 + 8 * s, (it / STAGES) & 1, give_up, 2);
                        if (!ok) break;
                        if (kb == lo && item == (int)blockIdx.x) stamp(g, o, 3);
                        fence_after_sync();
                        const uint64_t a = desc_kmajor(stage0 + s * STAGE_BYTES),
                                       b = desc_kmajor(stage0 + s * STAGE_BYTES + W_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) umma(acc, a + 2 * k, b + 2 * k, id, (kb > lo) | (k > 0));
                        umma_commit(empty0 + 8 * s);
                    }
                    if (ok) umma_commit(acc_full0 + 8 * as);
                    stamp(g, o, 4);
                }
            }
        }
    } else if (warp >= 3) {
        // The four warps share named barrier 2, so they must agree on every step that uses it: a warp whose
        // wait ran out keeps walking its items (without waiting or storing) to the end of the operation, and
        // whether to go on is decided once per operation, by one thread, for all four.
        const int vt = threadIdx.x - VEC0;
        const int quarter = warp & 3;
        const int lrow = quarter * 32 + lane;                       // row of a tile = lane of tensor memory
        int local = 0;
        bool failed = false;
        bool stopped = false;
        pdl_wait();
        for (int o = 0; o < g.count; ++o) {
            const ChainOp& op = g.ops[g.first + o];
            const int kind = (int)op.f[F_KIND];
            if (vt == 0) stamp(g, o, 0);
            if (kind == OP_GEMM) {
                const int items = (int)op.f[F_ITEMS], row_tiles = (int)op.f[F_ROW_TILES], epi = (int)op.f[F_EPI];
                const int N = (int)op.f[F_N], ldy = (int)op.f[F_LDY], act = (int)op.f[F_ACT];
                const long long part_stride = op.f[F_PART_STRIDE];
                const float cap = (float)as_double(op.f[F_CAP]);
                for (int item = blockIdx.x; item < items; item += G, ++local) {
                    const int rt = item % row_tiles, ks = item / row_tiles;
                    const int as = local & 1;
                    bool live = false;
                    if (!failed) {
                        live = __all_sync(0xffffffffu, wait_on(acc_full0 + 8 * as, (local >> 1) & 1, give_up, 3));
                        failed = !live;
                    }
                    float r[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = 0.0f;
                    if (live) {
                        fence_after_sync();
                        uint32_t v[16];
                        tmem_ld16(tmem + as * BT + ((uint32_t)(quarter * 32) << 16), v);
                        tmem_wait_ld();
                        fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty0 + 8 * as);
#pragma unroll
                        for (int i = 0; i < 16; ++i) r[i] = __uint_as_float(v[i]);
                    }
                    if (epi == EPI_GATED) {
                        // lanes 0-63 hold the gate values of 64 outputs, lanes 64-127 their up values
                        const int col = rt * 64 + (lrow & 63);
                        if (lrow >= 64) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) upx[(lrow - 64) * BT + i] = r[i];
                        }
                        vec_sync();
                        if (live && lrow < 64 && col < N) {
                            bf16* y = reinterpret_cast<bf16*>(op.f[F_Y]);
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < g.M)
                                    y[(size_t)i * ldy + col] =
                                        __float2bfloat16_rn(fast_gate_act(r[i], act) * upx[lrow * BT + i]);
                        }
                        vec_sync();                                 // upx may be written again
                    } else {
                        const int col = rt * BR + lrow;
                        if (live && col < N) {
                            float* y = reinterpret_cast<float*>(op.f[F_Y]) + (size_t)ks * part_stride;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < g.M) y[(size_t)i * ldy + col] = epi == EPI_SOFTCAP ? soft_cap(r[i], cap) : r[i];
                        }
                    }
                }
            } else if (kind == OP_NORM) {
                if ((int)blockIdx.x < g.M) {
                    const int hidden = (int)op.f[F_HIDDEN];
                    if (hidden <= 2 * VEC * 4) norm_row<2>(op, blockIdx.x, vt, scratch);
                    else if (hidden <= 5 * VEC * 4) norm_row<5>(op, blockIdx.x, vt, scratch);
                    else norm_row<9>(op, blockIdx.x, vt, scratch);       // up to 4608; the host refuses wider rows
                }
            } else {
                const long long heads = op.f[F_HEADS];
                const int n_heads = (int)(heads & 0xffff) + 2 * (int)((heads >> 16) & 0xffff);
                for (int i = blockIdx.x; i < g.M * n_heads; i += G) rope_head(op, g, i / n_heads, i % n_heads, vt);
            }
            if (vt == 0) stamp(g, o, 1);
            if (o + 1 == g.count) break;
            // ---- the barrier between two operations.  One thread arrives with release and polls with acquire
            // for the block: what the other threads wrote is ordered before its arrival by the named barrier.
            proxy_fence();
            vec_sync();
            if (vt == 0) {
                if (!*give_up) {
                    const unsigned target = (unsigned)(o + 1) * (unsigned)G;
                    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(g.sync) : "memory");
                    const long long t0 = clock64();
                    unsigned spins = 0;
                    while (load_acquire(g.sync) < target) {
                        if ((++spins & 63u) == 0) {
                            if (*give_up || load_acquire(g.sync + 1)) { *give_up = 1; break; }
                            if (clock64() - t0 > WAIT_CYCLES) {
                                *give_up = 1;
                                atomicCAS(&g_chain_error, 0, 8);
                                break;
                            }
                        }
                    }
                    proxy_fence();
                    stamp(g, o, 2);
                }
                if (*give_up) atomicExch(g.sync + 1, 1u);           // the other blocks need not wait their full time
                decision[0] = *give_up;
                if (!*give_up) phase[0] = o + 1;
            }
            vec_sync();
            if (decision[0]) { stopped = true; break; }
        }
        // the last block to leave zeroes the barrier's count for the next launch
        if (vt == 0 && !stopped && !*give_up && g.count > 1) {
            __threadfence();
            if (atomicAdd(g.sync + 2, 1u) == (unsigned)G - 1) {
                g.sync[0] = 0;
                g.sync[2] = 0;
                __threadfence();
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

bool g_smem_raised = false;
int g_coop_pdl = 1;             // whether the cooperative and the programmatic attribute go together

}  // namespace

// Writes the 128-byte tensor map of a row-major bfloat16 matrix (rows x cols, ld elements between rows)
// with boxes of box_rows x 64 to host memory; the caller copies it into its device array of maps.
BROLM_API int brolm_chain_make_map(void* dst, const void* ptr, long long rows, long long cols, long long ld,
                                   int box_rows) {
    if (cols <= 0 || rows <= 0 || cols % 8 != 0 || ld % 8 != 0 || ((uintptr_t)ptr & 15)) return BROLM_ERR_ALIGNMENT;
    if (box_rows < 1 || box_rows > 256) return BROLM_ERR_BAD_SIZE;
    CUtensorMap map;
    const int st = tc::make_map_2d(&map, ptr, rows, cols, ld, box_rows);
    if (st) return st;
    memcpy(dst, &map, sizeof(map));
    return BROLM_OK;
}

BROLM_API int brolm_chain_limits(int* max_tokens, int* op_bytes, int* map_bytes) {
    *max_tokens = BT;
    *op_bytes = (int)sizeof(ChainOp);
    *map_bytes = (int)sizeof(CUtensorMap);
    return BROLM_OK;
}

// Runs operations [first, first + count) of `ops` for M tokens.  `sync` points at four words of device
// memory that were zero before the first launch; a launch that ends without an error leaves them zero.
// `trace` (may be null): int64 [blocks][count][8] that receives nanosecond stamps of every block and
// operation: 0 start, 1 work done, 2 barrier passed, 3 first tile multiplied, 4 last tile issued.
BROLM_API int brolm_decode_chain(const void* maps, const void* ops, int first, int count, int M, const void* positions,
                                 const void* rows0, const void* rows1, const void* rows2, const void* rows3,
                                 void* sync, void* trace, cudaStream_t stream) {
    if (count <= 0 || M <= 0) return BROLM_OK;
    if (M > BT) return BROLM_ERR_TOO_LARGE;
    if (((uintptr_t)maps & 63) || ((uintptr_t)ops & 7)) return BROLM_ERR_ALIGNMENT;
    if (!g_smem_raised) {
        cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        g_smem_raised = true;
    }
    cudaError_t e;
    ChainArgs g;
    g.maps = (const CUtensorMap*)maps;
    g.ops = (const ChainOp*)ops;
    g.first = first; g.count = count; g.M = M;
    g.positions = (const int*)positions;
    g.cache_rows[0] = (const int*)rows0; g.cache_rows[1] = (const int*)rows1;
    g.cache_rows[2] = (const int*)rows2; g.cache_rows[3] = (const int*)rows3;
    g.sync = (unsigned*)sync;
    g.trace = (long long*)trace;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tc::device_sms());
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;              // the blocks wait on one another: all must be resident
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (g_coop_pdl && pdl_enabled()) {
        cfg.numAttrs = 2;
        e = cudaLaunchKernelEx(&cfg, decode_chain_kernel, g);
        if (e == cudaSuccess) return BROLM_OK;
        cudaGetLastError();
        g_coop_pdl = 0;                                       // not together on this driver: cooperative alone
    }
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, decode_chain_kernel, g);
}

BROLM_API int brolm_decode_chain_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_chain_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_chain_error, &zero, sizeof(int));
    }
    return v;
}
