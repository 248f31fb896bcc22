// Soft-capped, windowed, causal grouped-query attention of whole prompts on the
// 5th-generation tensor cores (tcgen05), bfloat16, sm_100a.
//
// One block owns 128 rows of one (sequence, kv head); a row is a (query token,
// query head of the group) pair, so the query heads that share a kv head share
// every key/value tile.  Keys and values come from the packed projection output
// of the step, 64 keys per tile:
//
//   warp 0    one thread issues the TMA loads: the query tile once, then a
//             two-stage ring of key tiles and of value tiles (128-byte swizzle);
//   warp 1    one thread issues tcgen05.mma: S = Q K^T (M 128, N 64) into one of
//             two score buffers in tensor memory, and O += P V (M 128, N head
//             size) into the output accumulator in tensor memory; the values
//             are used as they lie in memory (keys x head size, an MN-major
//             operand), so nothing is transposed;
//   warps 2-9 softmax: two threads own each row, 32 of the tile's 64 scores
//             each.  A thread reads its scores with tcgen05.ld, applies scale,
//             soft-cap and mask, agrees with its partner on the row's reference
//             maximum, writes the probabilities as bfloat16 into shared memory
//             (the A operand of the second product, two buffers), and at the
//             end scales its half of the accumulator by 1 / sum and stores it.
//
// The reference maximum of a row is only raised when the tile's maximum exceeds
// it by more than 8 (in log2 units): probabilities then stay below 2^8, and the
// accumulator in tensor memory has to be rescaled (read, multiply, write back)
// only on those rare tiles instead of on every tile.  Scores, statistics and
// the accumulator are float (wlejon/brolm src/gemma2.cpp:360-367 for the order:
// scale, cap * tanh(s / cap), mask, softmax).  Key j is visible from position p
// iff 0 <= p - j < window.
//
// Every mbarrier wait is bounded; a wait that runs out records a code that
// brolm_attn_tc_status() returns, lets outstanding loads land, frees the tensor
// memory and returns (the launch's results are then not valid).
#include "common.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128, BN = 64;
constexpr int THREADS = 320;      // loader warp, issuer warp, eight softmax warps
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_CYCLES = 2000000000ll;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_GAP = 8.0f;

__device__ int g_attn_tc_error;

struct TcArgs {
    bf16* out;
    int out_stride;
    const int32_t* cu_q;
    int n_kv, group, hd;
    float scale, cap;
    int window;
    uint32_t v_lbo, v_sbo;      // descriptor strides of the value operand, in 16-byte units
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try(bar, parity)) return true;
        if (*give_up) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *give_up = 1;
            atomicCAS(&g_attn_tc_error, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// K-major operand: rows of 128 bytes, 128-byte swizzle, eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (the values: 64 head-size elements contiguous, keys strided), 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo & 0x3fffu) << 16) | ((uint64_t)(sbo & 0x3fffu) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint32_t idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
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
// barrier slots
enum : int { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11, P_FULL = 13,
             PV_DONE = 15, N_BARS = 17 };

template <int HD>
__global__ void __launch_bounds__(THREADS, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                     const __grid_constant__ CUtensorMap map_k,
                                                                     const __grid_constant__ CUtensorMap map_v, TcArgs a) {
    constexpr int DB = HD / 64;                          // 64-wide blocks of the head size
    constexpr int Q_BYTES = BM * HD * 2, KV_BYTES = BN * HD * 2, P_BYTES = BM * BN * 2;      // P: two buffers
    constexpr uint32_t S_COL = 0, O_COL = 2 * BN;        // tensor-memory columns: two score buffers, then the output
    extern __shared__ __align__(1024) uint8_t smem_raw[];     // the swizzled tiles need 1024-byte alignment
    uint8_t* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {                      // never seen; refuse rather than compute wrongly
        if (threadIdx.x == 0) atomicCAS(&g_attn_tc_error, 0, 13);
        return;
    }
    const uint32_t q_s = smem_u32(base), k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES, p_s = v_s + 2 * KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + Q_BYTES + 4 * KV_BYTES + 2 * P_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars + N_BARS) + 16);   // [2][2][BM]: maxima by tile parity and half; the sums reuse it
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heaviest row blocks first
    const int per_x = gridDim.y * gridDim.z;
    const int n = blockIdx.x * per_x + blockIdx.z * gridDim.y + blockIdx.y;
    const int xt = gridDim.x - 1 - n / per_x;
    const int b = (n % per_x) / gridDim.y, g = (n % per_x) % gridDim.y;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int n_rows = q_len * a.group;
    const int row0 = xt * BM;
    const bool active = row0 < n_rows;                   // whole-block condition
    const int rows_here = active ? min(BM, n_rows - row0) : 0;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int tok0 = row0 / a.group;                     // BM is a multiple of the group
    const int tok_hi = active ? (row0 + rows_here - 1) / a.group : 0;
    const int t_first = active ? max(0, tok0 - window + 1) / BN : 0;
    const int n_tiles = active ? tok_hi / BN - t_first + 1 : 0;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(K_FULL + s), 1);
            mbar_init(bar(K_EMPTY + s), 1);
            mbar_init(bar(V_FULL + s), 1);
            mbar_init(bar(V_EMPTY + s), 1);
            mbar_init(bar(S_FULL + s), 1);
            mbar_init(bar(S_EMPTY + s), 8);
            mbar_init(bar(P_FULL + s), 8);
            mbar_init(bar(PV_DONE + s), 1);
        }
        give_up[0] = 0;
        give_up[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            mbar_expect_tx(bar(Q_FULL), Q_BYTES);
            for (int d = 0; d < DB; ++d)
                tma_load_3d(q_s + d * (BM * 128), &map_q, d * 64, g * a.group, q0 + tok0, bar(Q_FULL));
            int issued_k = 0, issued_v = 0;
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int key0 = q0 + (t_first + j) * BN;
                ok = mbar_wait(bar(K_EMPTY + s), ph ^ 1, give_up, 1);
                if (!ok) break;
                mbar_expect_tx(bar(K_FULL + s), KV_BYTES);
                for (int d = 0; d < DB; ++d)
                    tma_load_3d(k_s + s * KV_BYTES + d * (BN * 128), &map_k, d * 64, g, key0, bar(K_FULL + s));
                ++issued_k;
                ok = mbar_wait(bar(V_EMPTY + s), ph ^ 1, give_up, 2);
                if (!ok) break;
                mbar_expect_tx(bar(V_FULL + s), KV_BYTES);
                for (int d = 0; d < DB; ++d)
                    tma_load_3d(v_s + s * KV_BYTES + d * (BN * 128), &map_v, d * 64, g, key0, bar(V_FULL + s));
                ++issued_v;
            }
            if (*give_up) {        // let the loads in flight land before the block goes away
                mbar_wait(bar(Q_FULL), 0, give_up + 1, 9);
                for (int j = max(0, issued_k - 2); j < issued_k; ++j) mbar_wait(bar(K_FULL + (j & 1)), (j >> 1) & 1, give_up + 1, 9);
                for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_wait(bar(V_FULL + (j & 1)), (j >> 1) & 1, give_up + 1, 9);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_tiles > 0) {
            const uint32_t id_qk = idesc(BM, BN, 0), id_pv = idesc(BM, HD, 1);
            bool ok = mbar_wait(bar(Q_FULL), 0, give_up, 3);
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                if (!mbar_wait(bar(K_FULL + s), ph, give_up, 4)) return false;
                if (!mbar_wait(bar(S_EMPTY + s), ph ^ 1, give_up, 5)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int d = 0; d < DB; ++d) {
                    const uint64_t qa = desc_kmajor(q_s + d * (BM * 128)), kb = desc_kmajor(k_s + s * KV_BYTES + d * (BN * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma(tmem + S_COL + s * BN, qa + 2 * k, kb + 2 * k, id_qk, (d | k) != 0);
                }
                umma_commit(bar(S_FULL + s));
                umma_commit(bar(K_EMPTY + s));
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) { ok = issue_qk(j + 1); if (!ok) break; }
                const int s = j & 1;
                ok = mbar_wait(bar(P_FULL + s), (j >> 1) & 1, give_up, 6) && mbar_wait(bar(V_FULL + s), (j >> 1) & 1, give_up, 7);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t pa = desc_kmajor(p_s + s * P_BYTES);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    // sixteen keys further: 32 bytes along a row of P, sixteen 128-byte rows down in V
                    const uint64_t vb = desc_mnmajor(v_s + s * KV_BYTES + k * (16 * 128), a.v_lbo, a.v_sbo);
                    umma(tmem + O_COL, pa + 2 * k, vb, id_pv, (j | k) != 0);
                }
                umma_commit(bar(V_EMPTY + s));
                umma_commit(bar(PV_DONE + s));
            }
        }
    } else if (n_tiles > 0) {
        // Two warps share each quarter of the rows (a warp may only read the 32 lanes of tensor memory of its
        // quarter): warp w and warp w + 4 own the same 32 rows, the first takes score columns 0-31, the second
        // 32-63.  They agree on the row's reference maximum through shared memory and a 64-thread barrier.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;                  // this thread's row of the block
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const bool row_ok = r < rows_here;
        const int pos = tok0 + r / a.group;                 // position of the row's token (prompts start at 0)
        const float c0 = a.cap > 0.0f ? a.scale / a.cap * (2.0f * LOG2E) : a.scale * LOG2E;
        const float c1 = a.cap * LOG2E, c2 = 2.0f * a.cap * LOG2E;
        float m_ref = -INFINITY, l = 0.0f;                  // l: the sum over this thread's columns only
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            ok = mbar_wait(bar(S_FULL + s), (j >> 1) & 1, give_up, 8);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[32];
            tmem_ld32(tmem + lane_addr + S_COL + s * BN + half * 32, sv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(S_EMPTY + s));

            const int key_base = (t_first + j) * BN;
            const bool edge = key_base + BN - 1 > tok0 || key_base < tok_hi - window + 1;
            // score in log2 units: with the cap,  cap log2e tanh(x) = c1 - c2 / (1 + 2^(s c0));  without,  s c0
            float sc[32];
            float m_t = -INFINITY;
            if (a.cap > 0.0f) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const float t = fast_exp2(__uint_as_float(sv[c]) * c0);
                    sc[c] = fmaf(-c2, fast_rcp(1.0f + t), c1);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) sc[c] = __uint_as_float(sv[c]) * c0;
            }
            if (edge) {
                const int kp0 = key_base + half * 32;
                // visible: kp <= pos and pos - kp < window, i.e. lo <= c <= hi for column c of this thread
                const int hi = row_ok ? pos - kp0 : -1, lo = pos - window + 1 - kp0;
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (c > hi || c < lo) sc[c] = -INFINITY;
            }
#pragma unroll
            for (int c = 0; c < 32; ++c) m_t = fmaxf(m_t, sc[c]);
            float* slot = xch + (s * 2 + half) * BM + r;    // double-buffered by the tile's parity
            *slot = m_t;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            m_t = fmaxf(m_t, xch[(s * 2 + (half ^ 1)) * BM + r]);
            // raise the reference only when the tile goes well beyond it
            const bool raise = m_t > m_ref + RESCALE_GAP;       // also true for the first visible tile of a row
            const float m_new = raise ? m_t : m_ref;
            const float corr = (raise && m_ref > -INFINITY) ? fast_exp2(m_ref - m_new) : 1.0f;

            if (j >= 2) {
                // the product that read this buffer of P two tiles ago is done
                ok = mbar_wait(bar(PV_DONE + s), ((j - 2) >> 1) & 1, give_up, 10);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            }
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // rare: the accumulator has to be at rest (the product of the tile before is done), then every
                // row of the warp is rescaled (rows that keep their reference multiply by 1); each warp of the
                // pair takes half of the head size
                ok = mbar_wait(bar(PV_DONE + (s ^ 1)), ((j - 1) >> 1) & 1, give_up, 12);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem + lane_addr + O_COL + c, ov);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_st32(tmem + lane_addr + O_COL + c, ov);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            l *= corr;
            m_ref = m_new;
            // probabilities -> shared memory, bfloat16, row r of a K-major tile with 128-byte swizzle
            float sum = 0.0f;
            const float m_sub = m_ref > -INFINITY ? m_ref : 0.0f;     // a row that has seen nothing: 2^(-inf - 0) = 0
            const uint32_t prow = p_s + s * P_BYTES + r * 128;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p0 = fast_exp2(sc[ch * 8 + 2 * e] - m_sub), p1 = fast_exp2(sc[ch * 8 + 2 * e + 1] - m_sub);
                    sum += p0 + p1;
                    __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                    w[e] = *reinterpret_cast<uint32_t*>(&t);
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + (((half * 4 + ch) ^ (r & 7)) << 4)),
                             "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
            l += sum;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the tensor core reads P through the async proxy
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL + s));
        }
        if (ok) {
            ok = mbar_wait(bar(PV_DONE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, give_up, 11);
            ok = __all_sync(0xffffffffu, ok);
        }
        // the row's sum is the sum of the two halves (always added in the same order)
        const int fin = (n_tiles & 1) * 2;                  // the buffer the next tile would have used
        xch[(fin + half) * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float total = xch[fin * BM + r] + xch[(fin + 1) * BM + r];
            const float inv = total > 0.0f ? 1.0f / total : 0.0f;
            const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
            bf16* dst = a.out + (size_t)(q0 + tok) * a.out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem + lane_addr + O_COL + c, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pk;
                        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            p2[e] = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * e]) * inv, __uint_as_float(ov[i + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = pk;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}
// [tokens][heads][hd] bfloat16 with `stride` elements between tokens; box = 64 x box_heads x box_tokens.
int make_map(CUtensorMap* map, const void* ptr, long long tokens, int heads, int hd, long long stride, int box_heads,
             int box_tokens) {
    EncodeTiled enc = encoder();
    if (!enc) return BROLM_ERR_BAD_SIZE;
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BROLM_OK : BROLM_ERR_ALIGNMENT;
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcArgs& a, dim3 grid,
           cudaStream_t stream) {
    constexpr size_t smem = (size_t)BM * HD * 2 + 4 * (size_t)BN * HD * 2 + 2 * (size_t)BM * BN * 2 + N_BARS * 8 + 16 + 4 * BM * 4;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    attn_prefill_tc_kernel<HD><<<grid, THREADS, smem, stream>>>(mq, mk, mv, a);
    return launch_status();
}

}  // namespace

// Prompts that start at position 0, bfloat16, head_dim 64, 128 or 256, 128 % group == 0.  q, k and v are
// rows of q_stride / kv_stride elements (token major; head h at h * hd).  v_lbo and v_sbo are the two
// strides of the value operand's shared-memory descriptor in bytes (0: the defaults).
BROLM_API int brolm_attn_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                    const void* k, const void* v, int kv_stride, int total_tokens, int n_kv, int group,
                                    int hd, float scale, float cap, int window, int batch, int max_q_len, int v_lbo,
                                    int v_sbo, cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    if (hd != 64 && hd != 128 && hd != 256) return BROLM_ERR_BAD_SIZE;
    if (group <= 0 || BM % group != 0 || n_kv <= 0 || batch > 65535 || n_kv > 65535) return BROLM_ERR_BAD_SIZE;
    if (q_stride % 8 || kv_stride % 8 || out_stride % 8) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)out & 15)) return BROLM_ERR_ALIGNMENT;
    CUtensorMap mq, mk, mv;
    int st = make_map(&mq, q, total_tokens, n_kv * group, hd, q_stride, group, BM / group);
    if (st) return st;
    st = make_map(&mk, k, total_tokens, n_kv, hd, kv_stride, 1, BN);
    if (st) return st;
    st = make_map(&mv, v, total_tokens, n_kv, hd, kv_stride, 1, BN);
    if (st) return st;
    TcArgs a;
    a.out = (bf16*)out; a.out_stride = out_stride; a.cu_q = (const int32_t*)cu_q;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window;
    a.v_lbo = (uint32_t)((v_lbo > 0 ? v_lbo : BN * 128) >> 4);      // next 64 head-size elements: the next box
    a.v_sbo = (uint32_t)((v_sbo > 0 ? v_sbo : 1024) >> 4);          // next eight keys
    dim3 grid((max_q_len * group + BM - 1) / BM, n_kv, batch);
    if (hd == 64) return launch<64>(mq, mk, mv, a, grid, stream);
    if (hd == 128) return launch<128>(mq, mk, mv, a, grid, stream);
    return launch<256>(mq, mk, mv, a, grid, stream);
}

BROLM_API int brolm_attn_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    }
    return v;
}
