// Soft-capped, windowed, causal grouped-query attention for bfloat16 on the
// tensor cores (mma.sync m16n8k16, float accumulation), sm_100a.
//
// Two kernels share the tile machinery:
//
// * attn_prefill_mma: prompts.  Keys and values are the packed projection
//   output of the step.  One block owns 64 rows of one (sequence, kv head); a
//   row is a (query token, query head of the group) pair, so the query heads
//   that share a kv head share every staged key/value tile.  Each of the four
//   warps owns 16 rows.
//
// * attn_decode_mma: one new token per sequence over the paged cache.  The
//   rows are the query heads of the group (padded to 16); the key range of a
//   sequence is cut into splits, one block per (split, kv head, sequence).
//   The four warps of a block share each staged page and own 16 of its 64
//   keys each; their partial results are merged in shared memory, and when
//   there is more than one split a second kernel merges the splits from
//   float scratch.
//
// Scores follow wlejon/brolm src/gemma2.cpp:360-367: s = (q.k) * scale, then
// cap * tanh(s / cap), then the mask, then softmax; scores, statistics and the
// output accumulator are float; probabilities are rounded to bfloat16 for the
// second product.  Key j is visible from position p iff 0 <= p - j < window.
// tanh is computed as 1 - 2 / (1 + 2^(2x log2 e)) with the hardware's
// approximate exp2 and reciprocal (absolute error about 1e-7), exp as exp2.
#pragma once

#include "common.cuh"

namespace {

constexpr int KT = 64;        // keys per tile = one cache page
constexpr int BM = 64;        // rows per block (prompt kernel)
constexpr int NTHREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tanh(x) = 1 - 2 / (1 + e^(2x))
__device__ __forceinline__ float fast_tanh(float x) {
    return 1.0f - 2.0f * fast_rcp(1.0f + fast_exp2(x * (2.0f * LOG2E)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of the 16-byte chunk c of row r in a tile whose rows hold hd
// bf16.  Rows of whole 128-byte lines are XOR-swizzled so that the eight rows
// an ldmatrix phase reads fall into eight different bank groups.
__device__ __forceinline__ uint32_t tile_off(int r, int c, int hd, bool swz) {
    const int cs = swz ? (c ^ (r & 7)) : c;
    return (uint32_t)(r * hd + cs * 8) * 2u;
}

struct MmaArgs {
    const bf16* q;          // rows of q_stride elements; head h at h*hd
    bf16* out;
    int q_stride, out_stride;
    const int32_t* cu_q;    // [B+1]
    const int32_t* kv_len;  // [B]
    const bf16* k;          // packed source
    const bf16* v;
    int kv_stride;
    const bf16* k_pages;    // paged source [page][n_kv][KT][hd]
    const bf16* v_pages;
    const int32_t* page_table;
    int pt_stride, ring;
    int n_kv, group, hd;
    float scale, cap;
    int window;
    int sms;                // SMs of the device (prompt kernel: pairing of heavy and light tiles)
    // split-KV scratch
    int n_splits;
    float* part_o;          // [B][n_q][n_splits][hd]
    float* part_ml;         // [B][n_q][n_splits][2]  (max in log2 units, sum)
    int merge_here;         // decoding: the last block of a (sequence, kv head) merges the splits itself
};

// Tickets of the split-KV decode kernel, one per (sequence, kv head); zero between launches.
constexpr int MAX_TICKETS = 1 << 16;
__device__ unsigned g_decode_tickets[MAX_TICKETS];
constexpr int MAX_MERGED_SPLITS = 64;

// s (raw dot product) -> score in log2 units, soft-capped
__device__ __forceinline__ float score_of(float s, float scale, float cap, float inv_cap) {
    s *= scale;
    if (cap > 0.0f) s = cap * fast_tanh(s * inv_cap);
    return s * LOG2E;
}

// ===========================================================================
// prompts
// ===========================================================================
// EXACT: head_dim == HD_MAX, known to the compiler (all index arithmetic folds).
template <int HD_MAX, bool EXACT>
__global__ void __launch_bounds__(NTHREADS) attn_prefill_mma_kernel(MmaArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hd = EXACT ? HD_MAX : a.hd, hd16 = hd >> 4, cpr = hd >> 3;
    const bool swz = (hd & 63) == 0;
    const uint32_t rowb = (uint32_t)hd * 2u;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + BM * hd;
    bf16* Vs = Ks + KT * hd;
    const uint32_t qs_base = smem_u32(Qs), ks_base = smem_u32(Ks), vs_base = smem_u32(Vs);

    // Which (row tile, kv head, sequence) this block takes.  A causal row tile
    // costs as many key tiles as its index, so blocks are handed out heaviest
    // first; and when all blocks fit on the device at once (at most two per
    // SM), the blocks after the first `sms` take the lightest tiles in rising
    // order, so that an SM that got the k-th heaviest tile gets the k-th
    // lightest next to it and all SMs finish together.
    const int per_x = gridDim.y * gridDim.z, total = gridDim.x * per_x;
    const int n = blockIdx.x * per_x + blockIdx.z * gridDim.y + blockIdx.y;      // launch order
    const int rank = (total <= 2 * a.sms && n >= a.sms) ? total - 1 - (n - a.sms) : n;
    const int xt = gridDim.x - 1 - rank / per_x;                                // row tile, heaviest first
    const int b = (rank % per_x) / gridDim.y, g = (rank % per_x) % gridDim.y;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int n_rows = q_len * a.group;
    const int row0 = xt * BM;
    if (row0 >= n_rows) return;
    const int rows_here = min(BM, n_rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int tok_lo = row0 / a.group, tok_hi = (row0 + rows_here - 1) / a.group;
    const int key_lo = max(0, tok_lo - window + 1), key_hi = tok_hi;
    const int t_first = key_lo / KT, t_last = key_hi / KT;

    // queries of this block; rows past the end read as zero
    for (int idx = threadIdx.x; idx < BM * cpr; idx += NTHREADS) {
        const int r = idx / cpr, c = idx - r * cpr;
        const int row = row0 + r;
        const bool ok = r < rows_here;
        const int tok = ok ? row / a.group : 0, head = g * a.group + (ok ? row % a.group : 0);
        cp_async16(qs_base + tile_off(r, c, hd, swz), a.q + (size_t)(q0 + tok) * a.q_stride + head * hd + c * 8,
                   ok ? 16 : 0);
    }
    auto load_kv = [&](const bf16* src, uint32_t base, int t) {
        for (int idx = threadIdx.x; idx < KT * cpr; idx += NTHREADS) {
            const int r = idx / cpr, c = idx - r * cpr;
            const int kp = t * KT + r;
            const bool ok = kp <= key_hi;        // key_hi < q_len
            cp_async16(base + tile_off(r, c, hd, swz), src + (size_t)(q0 + (ok ? kp : 0)) * a.kv_stride + g * hd + c * 8,
                       ok ? 16 : 0);
        }
    };
    load_kv(a.k, ks_base, t_first);
    cp_async_commit();

    float o[HD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < HD_MAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    // positions of this thread's two rows (r and r + 8 of the warp's 16)
    int rpos[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        rpos[i] = r < rows_here ? (row0 + r) / a.group : -1;
    }
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;

    // Per-thread ldmatrix addresses.  The chunk (2 ks + j) of a row r lives at
    // ((32 ks) ^ xhi) + lo with xhi = ((r & 7) & 6) << 4 and lo = (j ^ (r & 1)) << 4
    // when the tile is swizzled (xhi = 0, lo = j << 4 when it is not); r & 7 is
    // lane & 7 for every row a thread addresses.
    const uint32_t x = lane & 7;
    const uint32_t xhi = swz ? (x & 6u) << 4 : 0u;
    const uint32_t jq = lane >> 4, jk = (lane >> 3) & 1, jv = lane >> 4;
    const uint32_t q_addr = qs_base + (warp * 16 + (lane & 15)) * rowb + ((swz ? (jq ^ (x & 1u)) : jq) << 4);
    const uint32_t k_addr = ks_base + ((lane & 7) + ((lane >> 4) << 3)) * rowb + ((swz ? (jk ^ (x & 1u)) : jk) << 4);
    const uint32_t v_addr = vs_base + ((lane & 7) + (((lane >> 3) & 1) << 3)) * rowb + ((swz ? (jv ^ (x & 1u)) : jv) << 4);
    const uint32_t kt_stride = 16u * rowb;

    for (int t = t_first; t <= t_last; ++t) {
        load_kv(a.v, vs_base, t);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                       // queries and keys of this tile are in shared memory

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < HD_MAX / 16; ++ks) {
            if (ks < hd16) {
                uint32_t af[4];
                const uint32_t coff = ((uint32_t)ks << 5) ^ xhi;
                ldmatrix_x4(q_addr + coff, af[0], af[1], af[2], af[3]);
#pragma unroll
                for (int kt = 0; kt < 4; ++kt) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(k_addr + kt * kt_stride + coff, b0, b1, b2, b3);
                    mma_bf16(s[2 * kt], af, b0, b1);
                    mma_bf16(s[2 * kt + 1], af, b2, b3);
                }
            }
        }
        // scale, soft-cap, mask
        const int tile_lo = t * KT, tile_hi = tile_lo + KT - 1;
        const bool edge = tile_hi > tok_lo || tile_lo < tok_hi - window + 1;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = score_of(s[nt][e], a.scale, a.cap, inv_cap);
                if (edge) {
                    const int kp = tile_lo + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int p = rpos[e >> 1];
                    if (!(p >= 0 && kp <= p && p - kp < window)) v = -INFINITY;
                }
                s[nt][e] = v;
            }
        }
        // online softmax, two rows per thread
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * i], s[nt][2 * i + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[i], mx);
            const float base = m_new == -INFINITY ? 0.0f : m_new;     // a row that has seen nothing yet
            const float corr = fast_exp2(m[i] - base);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float p0 = fast_exp2(s[nt][2 * i] - base), p1 = fast_exp2(s[nt][2 * i + 1] - base);
                s[nt][2 * i] = p0;
                s[nt][2 * i + 1] = p1;
                sum += p0 + p1;
            }
            l[i] = l[i] * corr + sum;
            m[i] = m_new;
#pragma unroll
            for (int d = 0; d < HD_MAX / 8; ++d) {
                o[d][2 * i] *= corr;
                o[d][2 * i + 1] *= corr;
            }
        }
        uint32_t pf[4][4];
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
            pf[kt][0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            pf[kt][1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            pf[kt][2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            pf[kt][3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
        }
        cp_async_wait<0>();
        __syncthreads();                       // values are in; every warp is done with the keys
        if (t < t_last) load_kv(a.k, ks_base, t + 1);
        cp_async_commit();
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
#pragma unroll
            for (int dp = 0; dp < HD_MAX / 16; ++dp) {
                if (dp < hd16) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_addr + kt * kt_stride + (((uint32_t)dp << 5) ^ xhi), b0, b1, b2, b3);
                    mma_bf16(o[2 * dp], pf[kt], b0, b1);
                    mma_bf16(o[2 * dp + 1], pf[kt], b2, b3);
                }
            }
        }
        __syncthreads();                       // every warp is done with the values
    }
    cp_async_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float sum = l[i];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int r = warp * 16 + (lane >> 2) + 8 * i;
        if (r >= rows_here) continue;
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
        bf16* dst = a.out + (size_t)(q0 + tok) * a.out_stride + head * hd + (lane & 3) * 2;
#pragma unroll
        for (int d = 0; d < HD_MAX / 8; ++d) {
            if (d * 8 < hd)
                *reinterpret_cast<__nv_bfloat162*>(dst + d * 8) = __floats2bfloat162_rn(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
        }
    }
}

// ===========================================================================
// decoding over the paged cache
// ===========================================================================
constexpr int STAGES = 3;
constexpr int PT_ROW = 512;          // entries of a page-table row kept in shared memory (32768 keys)

template <int HD_MAX, bool EXACT>
__global__ void __launch_bounds__(NTHREADS) attn_decode_mma_kernel(MmaArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int hd = EXACT ? HD_MAX : a.hd, hd16 = hd >> 4, cpr = hd >> 3;
    const bool swz = (hd & 63) == 0;
    const uint32_t rowb = (uint32_t)hd * 2u;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);            // [16][hd]
    bf16* stage0 = Qs + 16 * hd;                             // STAGES x ([KT][hd] keys, [KT][hd] values)
    const uint32_t qs_base = smem_u32(Qs), st_base = smem_u32(stage0);
    const uint32_t stage_bytes = 2u * KT * hd * 2u;

    const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // The sequence's length and its row of the page table were written by the host before the step's
    // first kernel: they are fetched together, ahead of the wait, so that the first tile's address
    // does not take two more round trips to the L2 after it.
    __shared__ int pt_row[PT_ROW];
    for (int i = threadIdx.x; i < min(a.pt_stride, PT_ROW); i += NTHREADS) pt_row[i] = a.page_table[(size_t)b * a.pt_stride + i];
    const int kv_len = a.kv_len[b];
    const int q_row = a.cu_q[b];                              // (also the host's)
    __syncthreads();
    pdl_wait();               // q and the newest key and value come from the kernels before this one
    const int n_q = a.n_kv * a.group;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int pos = kv_len - 1;
    const int key_lo = max(0, pos - window + 1);
    int t_begin = 0, t_end = 0;                               // tiles [t_begin, t_end) of this split
    if (kv_len > 0) {
        const int t_lo = key_lo / KT, t_hi = pos / KT;
        const int per = (t_hi - t_lo + 1 + a.n_splits - 1) / a.n_splits;
        t_begin = t_lo + split * per;
        t_end = min(t_hi + 1, t_begin + per);
    }
    const int n_tiles = max(0, t_end - t_begin);

    // the query row of this sequence: heads of the group, rows >= group are zero
    for (int idx = threadIdx.x; idx < 16 * cpr; idx += NTHREADS) {
        const int r = idx / cpr, c = idx - r * cpr;
        const bool ok = r < a.group && kv_len > 0;
        cp_async16(qs_base + tile_off(r, c, hd, swz),
                   a.q + (size_t)q_row * a.q_stride + (g * a.group + (ok ? r : 0)) * hd + c * 8, ok ? 16 : 0);
    }
    auto page_of = [&](int i) -> int {                        // page that holds the i-th tile of the split
        const int ridx = (int)(((long long)(t_begin + i) * KT) % a.ring);
        const int entry = ridx / KT;
        return entry < PT_ROW ? pt_row[entry] : a.page_table[(size_t)b * a.pt_stride + entry];
    };
    auto load_tile = [&](int i, int page) {                   // i-th tile of the split into stage i % STAGES
        const int t = t_begin + i;
        const size_t src = ((size_t)page * a.n_kv + g) * KT * hd;
        const uint32_t kb = st_base + (i % STAGES) * stage_bytes, vb = kb + KT * hd * 2u;
        for (int idx = threadIdx.x; idx < KT * cpr; idx += NTHREADS) {
            const int r = idx / cpr, c = idx - r * cpr;
            const uint32_t off = tile_off(r, c, hd, swz);
            const int kp = t * KT + r;
            const int bytes = (kp >= key_lo && kp <= pos) ? 16 : 0;   // places never written read as zero
            cp_async16(kb + off, a.k_pages + src + r * hd + c * 8, bytes);
            cp_async16(vb + off, a.v_pages + src + r * hd + c * 8, bytes);
        }
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < n_tiles) load_tile(i, page_of(i));
        cp_async_commit();
    }
    // the page id of the tile that the next iteration will load is fetched one iteration early
    int page_next = (STAGES - 1 < n_tiles) ? page_of(STAGES - 1) : 0;

    const uint32_t x = lane & 7;
    const uint32_t xhi = swz ? (x & 6u) << 4 : 0u;
    const uint32_t jq = lane >> 4, jk = (lane >> 3) & 1, jv = lane >> 4;
    const uint32_t q_addr = qs_base + (lane & 15) * rowb + ((swz ? (jq ^ (x & 1u)) : jq) << 4);
    const uint32_t k_thr = (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * rowb + ((swz ? (jk ^ (x & 1u)) : jk) << 4);
    const uint32_t v_thr = KT * rowb + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * rowb +
                           ((swz ? (jv ^ (x & 1u)) : jv) << 4);

    float o[HD_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < HD_MAX / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const float inv_cap = a.cap > 0.0f ? 1.0f / a.cap : 0.0f;

    for (int i = 0; i < n_tiles; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                       // tile i has landed; everyone is done with tile i - 1
        if (i + STAGES - 1 < n_tiles) load_tile(i + STAGES - 1, page_next);
        cp_async_commit();
        if (i + STAGES < n_tiles) page_next = page_of(i + STAGES);
        const uint32_t sb = st_base + (i % STAGES) * stage_bytes;
        const int t = t_begin + i;

        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < HD_MAX / 16; ++ks) {
            if (ks < hd16) {
                uint32_t af[4], b0, b1, b2, b3;
                const uint32_t coff = ((uint32_t)ks << 5) ^ xhi;
                ldmatrix_x4(q_addr + coff, af[0], af[1], af[2], af[3]);
                ldmatrix_x4(sb + k_thr + coff, b0, b1, b2, b3);
                mma_bf16(s[0], af, b0, b1);
                mma_bf16(s[1], af, b2, b3);
            }
        }
        const int kbase = t * KT + warp * 16 + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kp = kbase + nt * 8 + (e & 1);
                const float v = score_of(s[nt][e], a.scale, a.cap, inv_cap);
                s[nt][e] = (kp >= key_lo && kp <= pos) ? v : -INFINITY;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[r], mx);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = fast_exp2(m[r] - base);
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float p0 = fast_exp2(s[nt][2 * r] - base), p1 = fast_exp2(s[nt][2 * r + 1] - base);
                s[nt][2 * r] = p0;
                s[nt][2 * r + 1] = p1;
                sum += p0 + p1;
            }
            l[r] = l[r] * corr + sum;
            m[r] = m_new;
#pragma unroll
            for (int d = 0; d < HD_MAX / 8; ++d) {
                o[d][2 * r] *= corr;
                o[d][2 * r + 1] *= corr;
            }
        }
        uint32_t pf[4];
        pf[0] = pack_bf16(s[0][0], s[0][1]);
        pf[1] = pack_bf16(s[0][2], s[0][3]);
        pf[2] = pack_bf16(s[1][0], s[1][1]);
        pf[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < HD_MAX / 16; ++dp) {
            if (dp < hd16) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(sb + v_thr + (((uint32_t)dp << 5) ^ xhi), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], pf, b0, b1);
                mma_bf16(o[2 * dp + 1], pf, b2, b3);
            }
        }
    }
    cp_async_wait<0>();
    pdl_trigger();                             // the keys are read: the next kernel may move in
    __syncthreads();                           // the stages are free: they now hold the warps' partial results

    // merge the four warps.  Layout in shared memory (float):
    //   wm[4][16], wl[4][16], wo[4][group][hd]
    float* wm = reinterpret_cast<float*>(stage0);
    float* wl = wm + 4 * 16;
    float* wo = wl + 4 * 16;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = l[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = (lane >> 2) + 8 * r;
        if ((lane & 3) == 0) {
            wm[warp * 16 + row] = m[r];
            wl[warp * 16 + row] = sum;
        }
        if (row < a.group) {
            float* dst = wo + ((size_t)warp * a.group + row) * hd + (lane & 3) * 2;
#pragma unroll
            for (int d = 0; d < HD_MAX / 8; ++d) {
                if (d * 8 < hd) {
                    dst[d * 8] = o[d][2 * r];
                    dst[d * 8 + 1] = o[d][2 * r + 1];
                }
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < a.group * hd; idx += NTHREADS) {
        const int row = idx / hd, d = idx - row * hd;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, wm[w * 16 + row]);
        float sum = 0.0f, acc = 0.0f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(wm[w * 16 + row] - mx);
                sum += wl[w * 16 + row] * f;
                acc += wo[((size_t)w * a.group + row) * hd + d] * f;
            }
        }
        const int head = g * a.group + row;
        if (a.n_splits == 1) {
            a.out[(size_t)q_row * a.out_stride + head * hd + d] = __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
        } else {
            const size_t slot = ((size_t)b * n_q + head) * a.n_splits + split;
            a.part_o[slot * hd + d] = acc;
            if (d == 0) {
                a.part_ml[slot * 2] = mx;
                a.part_ml[slot * 2 + 1] = sum;
            }
        }
    }
    if (a.n_splits == 1 || !a.merge_here) return;

    // The block that finishes last among the splits of this (sequence, kv head) merges them:
    //     out = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m).
    // Every block publishes its partial results (fence), then takes a ticket; the last ticket sees them all.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ticket = &g_decode_tickets[(size_t)b * a.n_kv + g];
        const unsigned prev = atomicAdd(ticket, 1u);
        is_last = prev == (unsigned)a.n_splits - 1u;
        if (is_last) *ticket = 0u;                       // all have arrived: ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (a.n_splits <= 4) {
        // up to four splits: a thread fetches the statistics of its row's splits and its four outputs of
        // every split at once and merges them by itself: one round trip to the L2, no exchange
        const int q4 = hd >> 2;
        for (int idx = threadIdx.x; idx < a.group * q4; idx += NTHREADS) {
            const int row = idx / q4, d = (idx - row * q4) * 4;
            const size_t slot0 = ((size_t)b * n_q + g * a.group + row) * a.n_splits;
            float4 v[4];
            float2 ml[4];
#pragma unroll
            for (int s = 0; s < 4; ++s)
                if (s < a.n_splits) {
                    ml[s] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot0 + s) * 2));
                    v[s] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (slot0 + s) * hd + d));
                }
            float mx = -INFINITY;
#pragma unroll
            for (int s = 0; s < 4; ++s)
                if (s < a.n_splits) mx = fmaxf(mx, ml[s].x);
            float sum = 0.0f;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < 4; ++s)
                if (s < a.n_splits) {
                    const float f = mx > -INFINITY ? fast_exp2(ml[s].x - mx) : 0.0f;
                    sum += ml[s].y * f;
                    acc.x += v[s].x * f; acc.y += v[s].y * f; acc.z += v[s].z * f; acc.w += v[s].w * f;
                }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            bf16* dst = a.out + (size_t)q_row * a.out_stride + (g * a.group + row) * hd + d;
            dst[0] = __float2bfloat16_rn(acc.x * inv);
            dst[1] = __float2bfloat16_rn(acc.y * inv);
            dst[2] = __float2bfloat16_rn(acc.z * inv);
            dst[3] = __float2bfloat16_rn(acc.w * inv);
        }
        return;
    }
    float* factor = reinterpret_cast<float*>(stage0);    // [group][n_splits], then the sums [group]
    float* total = factor + a.group * a.n_splits;
    for (int row = warp; row < a.group; row += NTHREADS / 32) {      // a warp per head
        const size_t slot0 = ((size_t)b * n_q + g * a.group + row) * a.n_splits;
        // (maximum, sum) of up to 64 splits live in the lanes' registers: one fetch for both passes
        float2 ml0 = make_float2(-INFINITY, 0.0f), ml1 = ml0;
        if (lane < a.n_splits) ml0 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot0 + lane) * 2));
        if (lane + 32 < a.n_splits) ml1 = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (slot0 + lane + 32) * 2));
        const float mx = warp_max(fmaxf(ml0.x, ml1.x));
        float sum = 0.0f;
        if (lane < a.n_splits) {
            const float f = mx > -INFINITY ? fast_exp2(ml0.x - mx) : 0.0f;
            factor[row * a.n_splits + lane] = f;
            sum += ml0.y * f;
        }
        if (lane + 32 < a.n_splits) {
            const float f = mx > -INFINITY ? fast_exp2(ml1.x - mx) : 0.0f;
            factor[row * a.n_splits + lane + 32] = f;
            sum += ml1.y * f;
        }
        sum = warp_sum(sum);
        if (lane == 0) total[row] = sum;
    }
    __syncthreads();
    // four outputs per thread and step, the splits' loads of a step issued together (a step is one
    // round trip to the L2; with 128 threads, a group of 2 and 256 wide heads there is one step)
    const int q4 = hd >> 2;
    for (int idx = threadIdx.x; idx < a.group * q4; idx += NTHREADS) {
        const int row = idx / q4, d = (idx - row * q4) * 4;
        const size_t slot0 = ((size_t)b * n_q + g * a.group + row) * a.n_splits;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s0 = 0; s0 < a.n_splits; s0 += 8) {
            float4 v[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s0 + s < a.n_splits) v[s] = __ldcg(reinterpret_cast<const float4*>(a.part_o + (slot0 + s0 + s) * hd + d));
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s0 + s < a.n_splits) {
                    const float f = factor[row * a.n_splits + s0 + s];
                    acc.x += v[s].x * f; acc.y += v[s].y * f; acc.z += v[s].z * f; acc.w += v[s].w * f;
                }
        }
        const float sum = total[row];
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        bf16* dst = a.out + (size_t)q_row * a.out_stride + (g * a.group + row) * hd + d;
        dst[0] = __float2bfloat16_rn(acc.x * inv);
        dst[1] = __float2bfloat16_rn(acc.y * inv);
        dst[2] = __float2bfloat16_rn(acc.z * inv);
        dst[3] = __float2bfloat16_rn(acc.w * inv);
    }
}

// Merge the splits of one (sequence, head): out = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m).
// The statistics of all splits are fetched at once (one per thread) and the
// factors go to shared memory, so the loop over the partial outputs has no
// dependent loads.
__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml, bf16* __restrict__ out,
                                                           const int32_t* __restrict__ cu_q, int out_stride, int n_q,
                                                           int n_splits, int hd) {
    extern __shared__ float factor[];                 // [n_splits], then scratch for the block reductions
    float* scratch = factor + n_splits;
    const int head = blockIdx.x, b = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    const size_t slot0 = ((size_t)b * n_q + head) * n_splits;
    float mx = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) mx = fmaxf(mx, part_ml[(slot0 + s) * 2]);
    mx = block_max(mx, scratch);
    float sum = 0.0f;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        const float f = mx > -INFINITY ? fast_exp2(part_ml[(slot0 + s) * 2] - mx) : 0.0f;
        factor[s] = f;
        sum += part_ml[(slot0 + s) * 2 + 1] * f;
    }
    sum = block_sum(sum, scratch);                    // also makes factor[] visible to every thread
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) acc += part_o[(slot0 + s) * hd + d] * factor[s];
        out[(size_t)cu_q[b] * out_stride + head * hd + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD_MAX, bool EXACT>
int launch_prefill(const MmaArgs& a, int batch, int max_q_len, cudaStream_t stream) {
    const size_t smem = (size_t)(BM + 2 * KT) * a.hd * sizeof(bf16);
    static size_t allowed = 0;               // raised once per size, not at every launch
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD_MAX, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid((max_q_len * a.group + BM - 1) / BM, a.n_kv, batch);
    attn_prefill_mma_kernel<HD_MAX, EXACT><<<grid, NTHREADS, smem, stream>>>(a);
    return launch_status();
}

template <int HD_MAX, bool EXACT>
int launch_decode(const MmaArgs& a, int batch, cudaStream_t stream) {
    size_t smem = (size_t)(16 + STAGES * 2 * KT) * a.hd * sizeof(bf16);
    const size_t merge = (size_t)(8 * 16 + 4 * a.group * a.hd) * sizeof(float) + 16 * a.hd * sizeof(bf16);
    if (merge > smem) smem = merge;
    static size_t allowed = 0;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD_MAX, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    dim3 grid(a.n_splits, a.n_kv, batch);
    MmaArgs b = a;
    b.merge_here = a.n_splits > 1 && a.n_splits <= MAX_MERGED_SPLITS && (long long)batch * a.n_kv <= MAX_TICKETS &&
                   (size_t)(a.group * a.n_splits + a.group) * sizeof(float) <= smem - 16 * a.hd * sizeof(bf16);
    int st = launch_pdl(attn_decode_mma_kernel<HD_MAX, EXACT>, grid, dim3(NTHREADS), smem, stream, b);
    if (st != 0 || a.n_splits == 1 || b.merge_here) return st;
    dim3 cgrid(a.n_kv * a.group, batch);
    return launch_pdl(attn_combine_kernel, cgrid, dim3(128), (a.n_splits + 33) * sizeof(float), stream,
                      (const float*)a.part_o, (const float*)a.part_ml, a.out, a.cu_q, a.out_stride,
                      a.n_kv * a.group, a.n_splits, a.hd);
}

int check_common(int hd, int group, int n_kv, int q_stride, int out_stride, int batch) {
    if (hd <= 0 || hd % 16 != 0 || group <= 0 || n_kv <= 0) return BROLM_ERR_BAD_SIZE;
    if (hd > 256) return BROLM_ERR_TOO_LARGE;
    if (q_stride % 8 != 0 || out_stride % 2 != 0) return BROLM_ERR_ALIGNMENT;
    if (batch > 65535 || n_kv > 65535) return BROLM_ERR_TOO_LARGE;
    return BROLM_OK;
}

}  // namespace
