// Soft-capped, windowed, causal grouped-query attention of whole prompts on the
// 5th-generation tensor cores (tcgen05), bfloat16, sm_100a.
//
// One block owns 128 rows of one (sequence, kv head); a row is a (query token,
// query head of the group) pair, so the query heads that share a kv head share
// every key/value tile.  Keys and values come from the packed projection output
// of the step, 128 keys per tile (a tcgen05.mma of 128 rows costs the same 64
// or so cycles for 64 as for 128 columns, so narrower score tiles waste half
// of the first product's time):
//
//   warp 0    one thread issues the TMA loads: the query tile once, then key
//             and value units into one ring of shared-memory slots in the
//             order in which the products use them (a key tile comes as two
//             halves of the head size, a value tile as two halves of its keys,
//             so a slot is free again as soon as its half is multiplied);
//   warp 1    one thread issues tcgen05.mma: S = Q K^T (M 128, N 128) into one of
//             two score buffers in tensor memory, and O += P V (M 128, N head
//             size, P read from tensor memory) into the output accumulator in
//             tensor memory; the values are used as they lie in memory (keys x
//             head size, an MN-major operand): nothing is transposed;
//   warps 2-9 softmax: two threads own each row, 64 of the tile's 128 scores
//             each.  A thread reads its scores with tcgen05.ld, applies scale,
//             soft-cap and mask, agrees with its partner on the row's reference
//             maximum, writes the probabilities as bfloat16 pairs over the
//             first half of the score buffer (tcgen05.st), and at the end
//             scales its half of the accumulator by 1 / sum and stores it.
//
// The tensor core runs the products in the order of issue, which is what keeps
// the score buffers safe: S(j+2) is issued after P(j) V(j), which read the same
// columns.
//
// The reference maximum of a row is only raised when the tile's maximum exceeds
// it by more than 8 (in log2 units): probabilities then stay below 2^8, and the
// accumulator in tensor memory has to be rescaled (read, multiply, write back)
// only on those rare tiles instead of on every tile.  Scores, statistics and
// the accumulator are float (wlejon/brolm src/gemma2.cpp:360-367 for the order:
// scale, cap * tanh(s / cap), mask, softmax).  Key j is visible from position p
// iff 0 <= p - j < window.
//
// A prompt of a model with few kv heads gives few blocks, and causal blocks of very different lengths
// (1 to 16 key tiles at 2,048 tokens).  The launcher then cuts the row blocks with the most key tiles
// in two along the keys (brolm_attn_prefill_tc_plan decides how many, by laying the blocks out over
// the SMs in the order in which they start): both halves write their unnormalised accumulator and
// their (reference maximum, sum) as float partial results, take a ticket, and the half that comes
// second merges the other's partial result into its own and writes the rows.  No block waits for
// another.
//
// Every mbarrier wait is bounded; a wait that runs out records a code that
// brolm_attn_tc_status() returns, lets outstanding loads land, frees the tensor
// memory and returns (the launch's results are then not valid).
#include "tcgen05.cuh"

#include <algorithm>
#include <functional>
#include <vector>

namespace {

constexpr int BM = 128, BN = 128;
constexpr int MAX_SLOTS = 8;
constexpr int THREADS = 320;      // loader warp, issuer warp, eight softmax warps
constexpr int TMEM_COLS = 512;
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
    int n_split;                // the heaviest n_split row blocks of every (sequence, kv head) run as two halves of their keys
    float* part_o;              // [pair][2][hd / 4][BM][4] unnormalised accumulators of the halves
    float* part_ml;             // [pair][2][BM][2] reference maximum (log2 units) and sum
};

// One ticket per pair of halves; the half that comes second sets it back to zero.
constexpr int MAX_PAIRS = 1024;
__device__ int g_pair_tickets[MAX_PAIRS];

using namespace tc;

__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_attn_tc_error, code);
}
// after the block gave up: loads in flight are waited for under the second flag
__device__ __forceinline__ bool drain_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_attn_tc_error, code, true);
}
__device__ __forceinline__ uint32_t idesc(int m, int n, int b_mn_major) { return idesc_bf16(m, n, b_mn_major); }

// The shapes that depend on the head size.  A key tile is KU units (parts of the head size, all 128 keys), a
// value tile two units (64 keys each, the whole head size); a ring slot holds either.
template <int HD>
struct Shape {
    static constexpr int DB = HD / 64;                           // 64-wide blocks of the head size
    static constexpr int KU = HD >= 128 ? 2 : 1;
    static constexpr int K_BOXES = DB / KU;                      // blocks of the head size in a key unit
    static constexpr int K_UNIT = BN * (HD / KU) * 2, V_UNIT = 64 * HD * 2;
    static constexpr int SLOT = K_UNIT > V_UNIT ? K_UNIT : V_UNIT;
    static constexpr int SLOTS = HD == 256 ? 5 : MAX_SLOTS;
    static constexpr int Q_BYTES = BM * HD * 2;
};

// barrier slots
enum : int { Q_FULL = 0, S_FULL = 1, P_FULL = 3, PV_DONE = 5, U_FULL = 7, U_EMPTY = U_FULL + MAX_SLOTS,
             N_BARS = U_EMPTY + MAX_SLOTS };

template <int HD>
__global__ void __launch_bounds__(THREADS, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                     const __grid_constant__ CUtensorMap map_k,
                                                                     const __grid_constant__ CUtensorMap map_v, TcArgs a) {
    using SH = Shape<HD>;
    constexpr int DB = SH::DB, KU = SH::KU, SLOTS = SH::SLOTS;
    constexpr uint32_t S_COL = 0, O_COL = 2 * BN;        // tensor-memory columns: two score buffers, then the output
    static_assert(O_COL + HD <= TMEM_COLS, "tensor memory");
    extern __shared__ __align__(1024) uint8_t smem_raw[];     // the swizzled tiles need 1024-byte alignment
    uint8_t* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {                      // never seen; refuse rather than compute wrongly
        if (threadIdx.x == 0) atomicCAS(&g_attn_tc_error, 0, 13);
        return;
    }
    const uint32_t q_s = smem_u32(base), ring = q_s + SH::Q_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SH::Q_BYTES + SLOTS * SH::SLOT);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* ticket_s = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars + N_BARS) + 16);
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars + N_BARS) + 32);   // [2][2][BM]: maxima by tile parity and half; the sums reuse it
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks start in the order of their linear index (x fastest); the blocks with the most key tiles come
    // first, over all sequences and kv heads: rank 0 is the last row block.  The first 2 * n_split ranks are
    // the halves of the n_split heaviest row blocks.
    const int per_x = gridDim.y * gridDim.z;
    const int d = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int rank = d / per_x, which = d % per_x;
    const int b = which / gridDim.y, g = which % gridDim.y;
    const int row_tiles = gridDim.x - a.n_split;
    int part = rank < 2 * a.n_split ? (rank & 1) : -1;   // 0, 1: a half; -1: the whole row block
    const int xt = part >= 0 ? row_tiles - 1 - (rank >> 1) : row_tiles - 1 - (rank - a.n_split);
    const int pair = (rank >> 1) * per_x + which;
    const int q0 = a.cu_q[b], q_len = a.cu_q[b + 1] - q0;
    const int n_rows = q_len * a.group;
    const int row0 = xt * BM;
    const bool active = row0 < n_rows;                   // whole-block condition
    const int rows_here = active ? min(BM, n_rows - row0) : 0;
    const int window = a.window > 0 ? a.window : 0x3fffffff;
    const int tok0 = row0 / a.group;                     // BM is a multiple of the group
    const int tok_hi = active ? (row0 + rows_here - 1) / a.group : 0;
    int t_first = active ? max(0, tok0 - window + 1) / BN : 0;
    int n_tiles = active ? tok_hi / BN - t_first + 1 : 0;
    if (part >= 0) {
        if (n_tiles < 2) {                  // nothing to cut: the first half does the row block alone
            if (part == 1) n_tiles = 0;
            part = -1;
        } else {                            // the second half gets the tile on the diagonal and the odd one
            const int first_half = n_tiles / 2;
            if (part == 1) t_first += first_half;
            n_tiles = part == 1 ? n_tiles - first_half : first_half;
        }
    }

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(S_FULL + s), 1);
            mbar_init(bar(P_FULL + s), 8);
            mbar_init(bar(PV_DONE + s), 1);
        }
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(bar(U_FULL + s), 1);
            mbar_init(bar(U_EMPTY + s), 1);
        }
        give_up[0] = 0;
        give_up[1] = 0;
        give_up[2] = tc::g_stall_code;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // Units go through the ring in the order of their use: K(0); then K(j+1), V(j) for every tile j.
    if (warp == 0) {
        if (lane == 0 && n_tiles > 0) {
            // Launched with programmatic stream serialization: the block may be here while the kernel before it
            // (the rotation that writes q and k) still runs.  Nothing of this kernel touches memory before its
            // first tiles have arrived, so the loader's wait is the kernel's.
            pdl_wait();
            mbar_expect_tx(bar(Q_FULL), SH::Q_BYTES);
            for (int d = 0; d < DB; ++d)
                tma_load_3d(q_s + d * (BM * 128), &map_q, d * 64, g * a.group, q0 + tok0, bar(Q_FULL));
            int u = 0;
            bool ok = true;
            auto slot_free = [&]() -> bool {
                ok = wait_on(bar(U_EMPTY + u % SLOTS), ((u / SLOTS) & 1) ^ 1, give_up, 1);
                return ok;
            };
            auto load_k = [&](int j) {
                const int key0 = q0 + (t_first + j) * BN;
                for (int ku = 0; ku < KU && ok; ++ku) {
                    if (!slot_free()) return;
                    const int sl = u % SLOTS;
                    mbar_expect_tx(bar(U_FULL + sl), SH::K_UNIT);
                    for (int d = 0; d < SH::K_BOXES; ++d)
                        tma_load_3d(ring + sl * SH::SLOT + d * (BN * 128), &map_k, (ku * SH::K_BOXES + d) * 64, g, key0,
                                    bar(U_FULL + sl));
                    ++u;
                }
            };
            auto load_v = [&](int j) {
                const int key0 = q0 + (t_first + j) * BN;
                for (int vu = 0; vu < 2 && ok; ++vu) {
                    if (!slot_free()) return;
                    const int sl = u % SLOTS;
                    mbar_expect_tx(bar(U_FULL + sl), SH::V_UNIT);
                    for (int d = 0; d < DB; ++d)
                        tma_load_3d(ring + sl * SH::SLOT + d * (64 * 128), &map_v, d * 64, g, key0 + vu * 64, bar(U_FULL + sl));
                    ++u;
                }
            };
            load_k(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) load_k(j + 1);
                if (ok) load_v(j);
            }
            pdl_trigger();         // every tile is asked for: the next kernel may move in
            if (*give_up) {        // let the loads in flight land before the block goes away
                drain_on(bar(Q_FULL), 0, give_up, 9);
                for (int i = max(0, u - SLOTS); i < u; ++i) drain_on(bar(U_FULL + i % SLOTS), (i / SLOTS) & 1, give_up, 9);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_tiles > 0) {
            const uint32_t id_qk = idesc(BM, BN, 0), id_pv = idesc(BM, HD, 1);
            bool ok = wait_on(bar(Q_FULL), 0, give_up, 3);
            int u = 0;
            // S(j) goes over the buffer that P(j-2) was read from: the product that read it was issued before
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
#pragma unroll
                for (int ku = 0; ku < KU; ++ku) {
                    const int sl = u % SLOTS;
                    if (!wait_on(bar(U_FULL + sl), (u / SLOTS) & 1, give_up, 4)) return false;
                    fence_after_sync();
#pragma unroll
                    for (int d = 0; d < SH::K_BOXES; ++d) {
                        const uint64_t qa = desc_kmajor(q_s + (ku * SH::K_BOXES + d) * (BM * 128));
                        const uint64_t kb = desc_kmajor(ring + sl * SH::SLOT + d * (BN * 128));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma(tmem + S_COL + s * BN, qa + 2 * k, kb + 2 * k, id_qk, (ku | d | k) != 0);
                    }
                    umma_commit(bar(U_EMPTY + sl));
                    ++u;
                }
                umma_commit(bar(S_FULL + s));
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) { ok = issue_qk(j + 1); if (!ok) break; }
                const int s = j & 1;
                ok = wait_on(bar(P_FULL + s), (j >> 1) & 1, give_up, 6);
                if (!ok) break;
#pragma unroll
                for (int vu = 0; vu < 2; ++vu) {
                    const int sl = u % SLOTS;
                    ok = wait_on(bar(U_FULL + sl), (u / SLOTS) & 1, give_up, 7);
                    if (!ok) break;
                    fence_after_sync();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        // sixteen keys further: eight columns of P, sixteen 128-byte rows down in V
                        const uint64_t vb = desc_mnmajor(ring + sl * SH::SLOT + k * (16 * 128), a.v_lbo, a.v_sbo);
                        umma_ts(tmem + O_COL, tmem + S_COL + s * BN + (vu * 4 + k) * 8, vb, id_pv, (j | vu | k) != 0);
                    }
                    umma_commit(bar(U_EMPTY + sl));
                    ++u;
                }
                if (!ok) break;
                umma_commit(bar(PV_DONE + s));
            }
        }
    } else if (n_tiles > 0) {
        // Two warps share each quarter of the rows (a warp may only touch the 32 lanes of tensor memory of its
        // quarter): warp w and warp w + 4 own the same 32 rows, the first takes score columns 0-63, the second
        // 64-127.  They agree on the row's reference maximum through shared memory and a 64-thread barrier.
        constexpr int W = BN / 2;                           // scores of a thread per tile
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
            ok = wait_on(bar(S_FULL + s), (j >> 1) & 1, give_up, 8);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            fence_after_sync();
            uint32_t sv[W];
            {
                uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[0]);
                uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sv[32]);
                tmem_ld32(tmem + lane_addr + S_COL + s * BN + half * W, lo);
                tmem_ld32(tmem + lane_addr + S_COL + s * BN + half * W + 32, hi);
            }
            tmem_wait_ld();

            const int key_base = (t_first + j) * BN;
            const bool edge = key_base + BN - 1 > tok0 || key_base < tok_hi - window + 1;
            // score in log2 units: with the cap,  cap log2e tanh(x) = c1 - c2 / (1 + 2^(s c0));  without,  s c0
            float sc[W];
            float m_t = -INFINITY;
            if (a.cap > 0.0f) {
#pragma unroll
                for (int c = 0; c < W; ++c) {
                    const float t = fast_exp2(__uint_as_float(sv[c]) * c0);
                    sc[c] = fmaf(-c2, fast_rcp(1.0f + t), c1);
                }
            } else {
#pragma unroll
                for (int c = 0; c < W; ++c) sc[c] = __uint_as_float(sv[c]) * c0;
            }
            if (edge) {
                const int kp0 = key_base + half * W;
                // visible: kp <= pos and pos - kp < window, i.e. lo <= c <= hi for column c of this thread
                const int hi = row_ok ? pos - kp0 : -1, lo = pos - window + 1 - kp0;
#pragma unroll
                for (int c = 0; c < W; ++c)
                    if (c > hi || c < lo) sc[c] = -INFINITY;
            }
#pragma unroll
            for (int c = 0; c < W; ++c) m_t = fmaxf(m_t, sc[c]);
            float* slot = xch + (s * 2 + half) * BM + r;    // double-buffered by the tile's parity
            *slot = m_t;
            // after this barrier both threads of the row hold their scores in registers, so the probabilities
            // may go over the partner's score columns
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            m_t = fmaxf(m_t, xch[(s * 2 + (half ^ 1)) * BM + r]);
            // raise the reference only when the tile goes well beyond it
            const bool raise = m_t > m_ref + RESCALE_GAP;       // also true for the first visible tile of a row
            const float m_new = raise ? m_t : m_ref;
            const float corr = (raise && m_ref > -INFINITY) ? fast_exp2(m_ref - m_new) : 1.0f;

            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // rare: the accumulator has to be at rest (the product of the tile before is done), then every
                // row of the warp is rescaled (rows that keep their reference multiply by 1); each warp of the
                // pair takes half of the head size
                ok = wait_on(bar(PV_DONE + (s ^ 1)), ((j - 1) >> 1) & 1, give_up, 12);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                fence_after_sync();
#pragma unroll 1
                for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem + lane_addr + O_COL + c, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_st32(tmem + lane_addr + O_COL + c, ov);
                }
            }
            l *= corr;
            m_ref = m_new;
            // probabilities -> tensor memory, bfloat16 pairs: keys 2c, 2c+1 of this thread in column c of its 32
            float sum = 0.0f;
            const float m_sub = m_ref > -INFINITY ? m_ref : 0.0f;     // a row that has seen nothing: 2^(-inf - 0) = 0
            uint32_t pw[W / 2];
#pragma unroll
            for (int c = 0; c < W / 2; ++c) {
                const float p0 = fast_exp2(sc[2 * c] - m_sub), p1 = fast_exp2(sc[2 * c + 1] - m_sub);
                sum += p0 + p1;
                __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                pw[c] = *reinterpret_cast<uint32_t*>(&t);
            }
            l += sum;
            tmem_st32(tmem + lane_addr + S_COL + s * BN + half * (W / 2), pw);
            tmem_wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL + s));
        }
        if (ok) {
            ok = wait_on(bar(PV_DONE + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, give_up, 11);
            ok = __all_sync(0xffffffffu, ok);
        }
        // the row's sum is the sum of the two halves (always added in the same order)
        const int fin = (n_tiles & 1) * 2;                  // the buffer the next tile would have used
        xch[(fin + half) * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
        if (ok) fence_after_sync();
        const float total = xch[fin * BM + r] + xch[(fin + 1) * BM + r];
        // A half: the partial result goes to memory, then the ticket says whether the other half is done.
        // (Every softmax warp takes part in the two barriers, whatever its waits did: a block that gave up
        // has already made the launch invalid.)
        float own = 1.0f, theirs = 0.0f, sum_all = total;
        const float4* their_o = nullptr;
        bool writes = true;
        if (part >= 0) {
            // A half's accumulator lies in memory as [head size / 4][row][4 floats]: the 32 rows of a warp write
            // 512 consecutive bytes per instruction, and the thread of the other half that owns the same row
            // and columns reads them back in the same way.
            float4* my_o = reinterpret_cast<float4*>(a.part_o) + (size_t)(pair * 2 + part) * (HD / 4) * BM + r;
            if (ok) {
#pragma unroll 1
                for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem + lane_addr + O_COL + c, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        my_o[(size_t)((c + i) / 4) * BM] = make_float4(__uint_as_float(ov[i]), __uint_as_float(ov[i + 1]),
                                                                         __uint_as_float(ov[i + 2]), __uint_as_float(ov[i + 3]));
                }
                if (half == 0) {
                    float* ml = a.part_ml + ((size_t)(pair * 2 + part) * BM + r) * 2;
                    ml[0] = m_ref;
                    ml[1] = total;
                }
            }
            __threadfence();
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (threadIdx.x == 64) *ticket_s = atomicAdd(&g_pair_tickets[pair], 1);
            asm volatile("bar.sync 5, 256;" ::: "memory");
            if (*ticket_s == 0) {
                writes = false;                             // the other half will find this one's result
            } else {
                if (threadIdx.x == 64) g_pair_tickets[pair] = 0;
                const float2 other = __ldcg(reinterpret_cast<const float2*>(a.part_ml) + (size_t)(pair * 2 + (part ^ 1)) * BM + r);
                const float m_o = other.x, l_o = other.y;
                const float m_all = fmaxf(m_ref, m_o);
                if (m_all > -INFINITY) {                    // (a half that saw nothing of a row: 2^(-inf) = 0)
                    own = fast_exp2(m_ref - m_all);
                    theirs = fast_exp2(m_o - m_all);
                } else {
                    own = theirs = 0.0f;
                }
                sum_all = total * own + l_o * theirs;
                their_o = reinterpret_cast<const float4*>(a.part_o) + (size_t)(pair * 2 + (part ^ 1)) * (HD / 4) * BM + r;
            }
        }
        if (ok && writes) {
            const float inv = sum_all > 0.0f ? 1.0f / sum_all : 0.0f;
            const float k_own = own * inv, k_theirs = theirs * inv;
            const int row = row0 + r, tok = row / a.group, head = g * a.group + row % a.group;
            bf16* dst = a.out + (size_t)(q0 + tok) * a.out_stride + (size_t)head * HD;
            // the other half's values: a piece of 32 is asked for while the piece before it is merged and stored
            const bool merge = their_o != nullptr && row_ok;
            float4 th[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                th[i] = merge ? __ldcg(their_o + (size_t)(half * (HD / 8) + i) * BM) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 1
            for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                float4 tn[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    tn[i] = (merge && c + 32 < (half + 1) * (HD / 2)) ? __ldcg(their_o + (size_t)((c + 32) / 4 + i) * BM)
                                                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                uint32_t ov[32];
                tmem_ld32(tmem + lane_addr + O_COL + c, ov);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        const float4 t0 = th[i / 4], t1 = th[i / 4 + 1];
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(ov[i + e]) * k_own;
                        f[0] = fmaf(t0.x, k_theirs, f[0]); f[1] = fmaf(t0.y, k_theirs, f[1]);
                        f[2] = fmaf(t0.z, k_theirs, f[2]); f[3] = fmaf(t0.w, k_theirs, f[3]);
                        f[4] = fmaf(t1.x, k_theirs, f[4]); f[5] = fmaf(t1.y, k_theirs, f[5]);
                        f[6] = fmaf(t1.z, k_theirs, f[6]); f[7] = fmaf(t1.w, k_theirs, f[7]);
                        uint4 pk;
                        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                        *reinterpret_cast<uint4*>(dst + c + i) = pk;
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) th[i] = tn[i];
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// [tokens][heads][hd] bfloat16 with `stride` elements between tokens; box = 64 x box_heads x box_tokens.
int make_map(CUtensorMap* map, const void* ptr, long long tokens, int heads, int hd, long long stride, int box_heads,
             int box_tokens) {
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_tokens};
    return make_map_bf16(map, ptr, 3, dims, strides, box);
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcArgs& a, dim3 grid,
           cudaStream_t stream) {
    using SH = Shape<HD>;
    constexpr size_t smem = (size_t)SH::Q_BYTES + (size_t)SH::SLOTS * SH::SLOT + N_BARS * 8 + 32 + 4 * BM * 4;
    static_assert(smem <= 232448, "shared memory of a block");
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    return launch_pdl(attn_prefill_tc_kernel<HD>, grid, dim3(THREADS), smem, stream, mq, mk, mv, a);
}

}  // namespace

// How many of the heaviest row blocks of every (sequence, kv head) to cut in two along the keys, for
// prompts of max_q_len tokens (all taken to be that long).  Blocks are laid out over the SMs in the order
// in which they start (each to the SM that is free first), a block costing its key tiles plus a fixed
// start, a half also the merge; the candidate with the shortest schedule wins, none when the blocks
// already outnumber the SMs twice over.  Returns 0 .. row blocks; pairs = result * n_kv * batch.
BROLM_API int brolm_attn_prefill_tc_plan(int max_q_len, int n_kv, int group, int window, int batch) {
    if (max_q_len <= 0 || n_kv <= 0 || group <= 0 || batch <= 0 || BM % group != 0) return 0;
    const int sms = device_sm_count();
    const long long per_x = (long long)n_kv * batch;
    const int rows = max_q_len * group, row_tiles = (rows + BM - 1) / BM;
    if (row_tiles * per_x >= 2LL * sms || row_tiles < 2) return 0;
    struct Key { int q, kv, group, window, batch, sms, result; };
    static Key memo[8];
    static int memo_next = 0;
    for (const Key& k : memo)
        if (k.q == max_q_len && k.kv == n_kv && k.group == group && k.window == window && k.batch == batch && k.sms == sms)
            return k.result;
    const int w = window > 0 ? window : 0x3fffffff;
    std::vector<int> tiles(row_tiles);                              // by rank: the last row block first
    for (int rank = 0; rank < row_tiles; ++rank) {
        const int xt = row_tiles - 1 - rank;
        const int tok0 = xt * BM / group, tok_hi = (std::min(rows, (xt + 1) * BM) - 1) / group;
        tiles[rank] = tok_hi / BN - std::max(0, tok0 - w + 1) / BN + 1;
    }
    // in key tiles (2.5 us each at head size 256).  Measured: 2.4 for a block's start, 2.5 for a half's merge; the
    // merge counts a little less here because only the half that finishes second pays all of it
    const float START = 2.4f, MERGE = 2.0f;
    std::vector<float> free_at(sms);
    auto schedule = [&](int n_split) {
        std::fill(free_at.begin(), free_at.end(), 0.0f);
        std::make_heap(free_at.begin(), free_at.end(), std::greater<float>());
        float end = 0.0f;
        auto run = [&](float cost) {
            std::pop_heap(free_at.begin(), free_at.end(), std::greater<float>());
            const float t = free_at.back() + cost;
            free_at.back() = t;
            std::push_heap(free_at.begin(), free_at.end(), std::greater<float>());
            end = std::max(end, t);
        };
        for (int rank = 0; rank < row_tiles; ++rank) {
            const int t = tiles[rank];
            if (rank < n_split && t >= 2) {
                for (int h = 0; h < 2; ++h)
                    for (long long i = 0; i < per_x; ++i) run(START + MERGE + (h ? t - t / 2 : t / 2));
            } else {
                for (long long i = 0; i < per_x; ++i) run(START + t);
            }
        }
        return end;
    };
    int best = 0;
    float best_end = schedule(0);
    const int most = (int)std::min<long long>(row_tiles, std::min<long long>((2LL * sms - row_tiles * per_x) / per_x, MAX_PAIRS / per_x));
    for (int c = 1; c <= 16; ++c) {                                 // sixteen candidates up to `most`
        const int n_split = (int)((long long)most * c / 16);
        if (n_split <= 0 || (c > 1 && n_split == (int)((long long)most * (c - 1) / 16))) continue;
        const float end = schedule(n_split);
        if (end < best_end * 0.97f) { best_end = end; best = n_split; }
    }
    memo[memo_next] = Key{max_q_len, n_kv, group, window, batch, sms, best};
    memo_next = (memo_next + 1) % 8;
    return best;
}

// Prompts that start at position 0, bfloat16, head_dim 64, 128 or 256, 128 % group == 0.  q, k and v are
// rows of q_stride / kv_stride elements (token major; head h at h * hd).  v_lbo and v_sbo are the two
// strides of the value operand's shared-memory descriptor in bytes (0: the defaults).  n_split > 0: the
// heaviest n_split row blocks run as two halves of their keys; part_o holds n_split * n_kv * batch * 2 *
// 128 * hd floats, part_ml n_split * n_kv * batch * 2 * 128 * 2 (n_split * n_kv * batch <= 1024).
BROLM_API int brolm_attn_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                    const void* k, const void* v, int kv_stride, int total_tokens, int n_kv, int group,
                                    int hd, float scale, float cap, int window, int batch, int max_q_len, int v_lbo,
                                    int v_sbo, int n_split, void* part_o, void* part_ml, cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    if (hd != 64 && hd != 128 && hd != 256) return BROLM_ERR_BAD_SIZE;
    if (group <= 0 || BM % group != 0 || n_kv <= 0 || batch > 65535 || n_kv > 65535) return BROLM_ERR_BAD_SIZE;
    if (q_stride % 8 || kv_stride % 8 || out_stride % 8) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)out & 15)) return BROLM_ERR_ALIGNMENT;
    const int row_tiles = (max_q_len * group + BM - 1) / BM;
    if (n_split < 0 || n_split > row_tiles || (long long)n_split * n_kv * batch > MAX_PAIRS) return BROLM_ERR_BAD_SIZE;
    if (n_split > 0 && (!part_o || !part_ml || ((uintptr_t)part_o & 15) || ((uintptr_t)part_ml & 7))) return BROLM_ERR_ALIGNMENT;
    CUtensorMap mq, mk, mv;
    int st = make_map(&mq, q, total_tokens, n_kv * group, hd, q_stride, group, BM / group);
    if (st) return st;
    st = make_map(&mk, k, total_tokens, n_kv, hd, kv_stride, 1, BN);      // a key unit: all keys of the tile
    if (st) return st;
    st = make_map(&mv, v, total_tokens, n_kv, hd, kv_stride, 1, 64);      // a value unit: 64 keys
    if (st) return st;
    TcArgs a;
    a.out = (bf16*)out; a.out_stride = out_stride; a.cu_q = (const int32_t*)cu_q;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window;
    a.v_lbo = (uint32_t)((v_lbo > 0 ? v_lbo : 64 * 128) >> 4);      // next 64 head-size elements: the next box
    a.v_sbo = (uint32_t)((v_sbo > 0 ? v_sbo : 1024) >> 4);          // next eight keys
    a.n_split = n_split; a.part_o = (float*)part_o; a.part_ml = (float*)part_ml;
    dim3 grid(row_tiles + n_split, n_kv, batch);
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

BROLM_WAIT_CONTROL(attn_tc)
