// Matrix product for few tokens (decode steps, up to 128 rows of X) on tcgen05:
//     Y[M,N] = X[M,K] * W[N,K]^T,  bfloat16 operands, float accumulation in tensor memory.
//
// With few tokens the product is a stream of W from memory, and the kernel is
// built as one: the roles of the operands are swapped (128 rows of W fill the M
// side of tcgen05.mma, the tokens the N side), and a persistent block per SM
// pulls its share of W through a deep ring of TMA stages (up to ten 16 KB
// tiles in flight per SM), so the stream never drains between the block's work
// items.  A work item is a (128-row tile of W, slice of K) pair; for the
// 2304-wide outputs of the model K is cut into slices so that every SM has an
// item, and the float partial sums of the slices are added, in order, by the
// kernel that reads them (the residual kernel).
//
//   warp 0    one thread issues the TMA loads of a stage: a 128 x 64 tile of W and
//             the matching tokens x 64 tile of X (rows past M read as zero);
//   warp 1    one thread issues tcgen05.mma (M 128, N tokens padded to 16/32/64/128)
//             into one of two accumulators, and hands stages and accumulators on
//             with tcgen05.commit;
//   warps 2-5 read an accumulator (lane = row of W = output column), apply the
//             epilogue and store Y[token][column] (a warp writes 32 consecutive
//             columns of a token).
// Epilogues: store (bfloat16, float, or float partial sums of a K slice); the
// gated activation act(X Wg^T) * (X Wu^T) for W = [Wg; Wu] (a tile holds 64 gate
// rows and the 64 up rows of the same outputs; wlejon/brolm src/gemma2.cpp:378-381);
// cap * tanh(y / cap) into float logits (src/gemma2.cpp:406-412).
//
// The weights depend on no earlier kernel, so the loader fills the ring with W
// before it waits for the kernel before it (programmatic dependent launch) and
// adds the X tiles afterwards.  Every mbarrier wait is bounded (tcgen05.cuh).
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BR = 128, BK = 64;
constexpr int THREADS = 192;
constexpr int W_BYTES = BR * BK * 2;
constexpr int RING_BYTES = 200 * 1024;

enum : int { EPI_STORE = 0, EPI_GATED = 1, EPI_SOFTCAP = 2 };

__device__ int g_gemm_stream_error;

struct StreamArgs {
    void* y;
    int ldy;
    int M, N, K;             // N: output columns (EPI_GATED: W has 2N rows, gate then up)
    int out_f32;
    int act;
    float cap;
    int ksplit;
    long long part_stride;   // elements between the float partial sums of two K slices
    int row_tiles, items;
};

__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_stream_error, code);
}
// after the block gave up: loads in flight are waited for under the second flag
__device__ __forceinline__ bool drain_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_stream_error, code, true);
}

template <int BT, int EPI>
struct Shape {
    static constexpr int OUT_ROWS = EPI == EPI_GATED ? BR / 2 : BR;        // output columns of a tile
    static constexpr int X_BYTES = BT * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES > 10 ? 10 : RING_BYTES / STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BT < 32 ? 32 : 2 * BT;            // two accumulators; a power of two
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16 +
                                   (EPI == EPI_GATED ? (size_t)64 * BT * 4 : 0);
};

template <int BT, int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x,
                                                                 StreamArgs g) {
    using S = Shape<BT, EPI>;
    constexpr int STAGES = S::STAGES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = smem_raw;
    if ((smem_u32(base) & 1023u) != 0) {                      // never seen; refuse rather than compute wrongly
        if (threadIdx.x == 0) atomicCAS(&g_gemm_stream_error, 0, 13);
        return;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * S::STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* upx = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars + 2 * STAGES + 4) + 16);   // gated: up values
    const uint32_t stage0 = smem_u32(base);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                   acc_empty0 = acc_full0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (g.K + BK - 1) / BK;
    const int per = (nkb + g.ksplit - 1) / g.ksplit;          // K blocks per slice
    auto kb_lo = [&](int item) { return (item / g.row_tiles) * per; };
    auto kb_hi = [&](int item) { return min(nkb, (item / g.row_tiles) * per + per); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8 * s, 1);
            mbar_init(acc_empty0 + 8 * s, 4);
        }
        give_up[0] = 0;
        give_up[1] = 0;
        give_up[2] = tc::g_stall_code;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), S::TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // the walk over (item, K block) of this block
            int item = blockIdx.x, kb = item < g.items ? kb_lo(item) : 0;
            auto valid = [&]() { return item < g.items; };
            auto advance = [&]() {
                if (++kb >= kb_hi(item)) {
                    item += gridDim.x;
                    if (item < g.items) kb = kb_lo(item);
                }
            };
            auto load_w = [&](int s, int it_item, int it_kb) {
                const int rt = it_item % g.row_tiles;
                const uint32_t full = full0 + 8 * s, dst = stage0 + s * S::STAGE_BYTES;
                mbar_expect_tx(full, S::STAGE_BYTES);
                if (EPI == EPI_GATED) {
                    tma_load_2d(dst, &map_w, it_kb * BK, rt * 64, full);                       // 64 gate rows
                    tma_load_2d(dst + W_BYTES / 2, &map_w, it_kb * BK, g.N + rt * 64, full);   // their 64 up rows
                } else {
                    tma_load_2d(dst, &map_w, it_kb * BK, rt * BR, full);
                }
            };
            auto load_x = [&](int s, int it_kb) {
                tma_load_2d(stage0 + s * S::STAGE_BYTES + W_BYTES, &map_x, it_kb * BK, 0, full0 + 8 * s);
            };
            // fill the ring with weights before the kernel before this one has finished
            int early_kb[STAGES];
            int n_early = 0;
            while (n_early < STAGES && valid()) {
                load_w(n_early, item, kb);                  // the stages are empty: nothing to wait for
                early_kb[n_early++] = kb;
                advance();
            }
            pdl_wait();
            for (int i = 0; i < n_early; ++i) load_x(i, early_kb[i]);
            int it = n_early;
            bool ok = true;
            while (valid()) {
                const int s = it % STAGES;
                ok = wait_on(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 1);
                if (!ok) break;
                load_w(s, item, kb);
                load_x(s, kb);
                advance();
                ++it;
            }
            pdl_trigger();                                   // the stream is issued: the next kernel may move in
            if (*give_up) {
                for (int j = max(0, it - STAGES); j < it; ++j)
                    drain_on(full0 + 8 * (j % STAGES), (j / STAGES) & 1, give_up, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id = idesc_bf16(BR, BT);
            int it = 0, local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < g.items && ok; item += gridDim.x, ++local) {
                const int as = local & 1;
                ok = wait_on(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, give_up, 5);
                if (!ok) break;
                fence_after_sync();
                const uint32_t acc = tmem + as * BT;
                const int lo = kb_lo(item), hi = kb_hi(item);
                for (int kb = lo; kb < hi; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = wait_on(full0 + 8 * s, (it / STAGES) & 1, give_up, 2);
                    if (!ok) break;
                    fence_after_sync();
                    const uint64_t a = desc_kmajor(stage0 + s * S::STAGE_BYTES), b = desc_kmajor(stage0 + s * S::STAGE_BYTES + W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) umma(acc, a + 2 * k, b + 2 * k, id, (kb > lo) | (k > 0));
                    umma_commit(empty0 + 8 * s);
                }
                if (ok) umma_commit(acc_full0 + 8 * as);
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        for (int item = blockIdx.x; item < g.items; item += gridDim.x, ++local) {
            const int rt = item % g.row_tiles, ks = item / g.row_tiles;
            const int as = local & 1;
            const bool ready = wait_on(acc_full0 + 8 * as, (local >> 1) & 1, give_up, 3);
            if (!__all_sync(0xffffffffu, ready)) break;
            fence_after_sync();
            const uint32_t acc = tmem + as * BT + ((uint32_t)(quarter * 32) << 16);
            const int lrow = quarter * 32 + lane;               // row of the tile = lane of tensor memory
            for (int c = 0; c < BT; c += 16) {
                uint32_t v[16];
                tmem_ld16(acc + c, v);
                tmem_wait_ld();
                if (c + 16 >= BT) {                             // all of this accumulator is in registers
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * as);
                }
                float o[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = __uint_as_float(v[i]);
                int col;
                bool writer = true;
                if (EPI == EPI_GATED) {
                    // lanes 0-63 hold the gate values of 64 outputs, lanes 64-127 their up values
                    col = rt * 64 + (lrow & 63);
                    if (quarter >= 2) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) upx[(lrow - 64) * BT + c + i] = o[i];
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (quarter < 2) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = fast_gate_act(o[i], g.act) * upx[lrow * BT + c + i];
                    }
                    writer = quarter < 2;
                    asm volatile("bar.sync 1, 128;" ::: "memory");          // upx may be written again
                } else {
                    col = rt * BR + lrow;
                    if (EPI == EPI_SOFTCAP) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = soft_cap(o[i], g.cap);
                    }
                }
                if (writer && col < g.N) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int tok = c + i;
                        if (tok < g.M) {
                            if (g.ksplit > 1) reinterpret_cast<float*>(g.y)[ks * g.part_stride + (size_t)tok * g.ldy + col] = o[i];
                            else if (g.out_f32) reinterpret_cast<float*>(g.y)[(size_t)tok * g.ldy + col] = o[i];
                            else reinterpret_cast<bf16*>(g.y)[(size_t)tok * g.ldy + col] = __float2bfloat16_rn(o[i]);
                        }
                    }
                }
            }
        }
    }
    pdl_trigger();
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, S::TMEM_COLS);
}

template <int BT, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const StreamArgs& g, cudaStream_t stream) {
    using S = Shape<BT, EPI>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<BT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const int sms = device_sms();
    return launch_pdl(gemm_stream_kernel<BT, EPI>, dim3(g.items < sms ? g.items : sms), dim3(THREADS), S::SMEM, stream, mw, mx, g);
}

template <int EPI>
int dispatch(const CUtensorMap& mw, const CUtensorMap& mx, const StreamArgs& g, int bt, cudaStream_t stream) {
    if (bt == 16) return launch<16, EPI>(mw, mx, g, stream);
    if (bt == 32) return launch<32, EPI>(mw, mx, g, stream);
    if (bt == 64) return launch<64, EPI>(mw, mx, g, stream);
    return launch<128, EPI>(mw, mx, g, stream);
}

}  // namespace

// epilogue 0: Y = X W^T (bfloat16 or float; with ksplit > 1 float partial sums, slice s at y + s * part_stride);
// 1: Y = act(X Wg^T) * (X Wu^T), W = [Wg; Wu] of 2N rows, N a multiple of 64; 2: Y = cap * tanh(X W^T / cap), float.
// M <= 128; K, ldx and ldw multiples of 8 elements; base addresses 16-byte aligned.
BROLM_API int brolm_gemm_stream(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
                                int epilogue, int out_f32, int act, float cap, int ksplit, long long part_stride,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BROLM_OK;
    if (M > 128) return BROLM_ERR_TOO_LARGE;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return BROLM_ERR_ALIGNMENT;
    if (epilogue < 0 || epilogue > 2) return BROLM_ERR_BAD_SIZE;
    if (epilogue == EPI_GATED && (N % 64 != 0 || act < 0 || act > 1)) return BROLM_ERR_BAD_SIZE;
    const int nkb = (K + BK - 1) / BK;
    if (ksplit < 1 || ksplit > nkb || (ksplit > 1 && epilogue != EPI_STORE)) return BROLM_ERR_BAD_SIZE;
    const int bt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    CUtensorMap mw, mx;
    int st = make_map_2d(&mw, w, epilogue == EPI_GATED ? 2LL * N : N, K, ldw, epilogue == EPI_GATED ? 64 : BR);
    if (st) return st;
    st = make_map_2d(&mx, x, M, K, ldx, bt);
    if (st) return st;
    StreamArgs g;
    g.y = y; g.ldy = ldy; g.M = M; g.N = N; g.K = K; g.out_f32 = epilogue == EPI_SOFTCAP ? 1 : out_f32; g.act = act;
    g.cap = cap; g.ksplit = ksplit; g.part_stride = part_stride;
    const int out_rows = epilogue == EPI_GATED ? 64 : BR;
    g.row_tiles = (N + out_rows - 1) / out_rows;
    // slices that would be empty (K blocks do not divide evenly) are left out
    const int per = (nkb + ksplit - 1) / ksplit;
    if ((ksplit - 1) * per >= nkb) return BROLM_ERR_BAD_SIZE;
    g.items = g.row_tiles * ksplit;
    if (epilogue == EPI_STORE) return dispatch<EPI_STORE>(mw, mx, g, bt, stream);
    if (epilogue == EPI_GATED) return dispatch<EPI_GATED>(mw, mx, g, bt, stream);
    return dispatch<EPI_SOFTCAP>(mw, mx, g, bt, stream);
}

BROLM_API int brolm_gemm_stream_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_stream_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_stream_error, &zero, sizeof(int));
    }
    return v;
}

BROLM_WAIT_CONTROL(gemm_stream)
