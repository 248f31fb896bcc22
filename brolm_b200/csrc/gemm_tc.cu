// bfloat16 matrix product for many tokens on the 5th-generation tensor cores:
//     Y[M,N] = X[M,K] * W[N,K]^T        (float accumulation)
// with the epilogues the decoder needs: store (bfloat16 or float), or the gated
// activation act(X Wg^T) * (X Wu^T) for W = [Wg; Wu] (wlejon/brolm
// src/gemma2.cpp:378-381), so that the 2F-wide intermediate never goes to
// memory.  sm_100a only.
//
// Structure (persistent: one block of 192 threads per SM walks over the 128 x 256 tiles of Y, rows
// of tiles first so that blocks running together share the same rows of W in L2):
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte
//            swizzle) of a 128 x 64 tile of X and a 256 x 64 tile of W per
//            stage into a ring of 4 stages, each announced on an mbarrier;
//   warp 1   allocates all 512 columns of tensor memory (two accumulators);
//            one thread issues tcgen05.mma (M 128, N 256, K 16, four per
//            stage) straight from shared memory into one accumulator, and
//            tcgen05.commit hands each stage back to the loader and each
//            finished accumulator to the epilogue;
//   warps 2-5  read an accumulator with tcgen05.ld (32 lanes x 32 columns per
//            warp and step), apply the epilogue and store, while the next
//            tile is already being multiplied into the other accumulator.
// For the gated epilogue the W tile of a stage is two 128-row loads (gate rows
// n.. and up rows F+n..), so accumulator columns 0-127 are the gate and 128-255
// the up values of the same 128 outputs.
//
// Every wait on an mbarrier is bounded (about a second of clock cycles).  A
// wait that runs out raises a flag that the other roles poll, records an
// error code that brolm_gemm_tc_status() returns, lets the loads in flight
// land, frees the tensor memory and returns; results of that launch are then
// not valid, the device stays usable.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;      // two accumulators of 256 columns

enum : int { EPI_STORE = 0, EPI_GATED = 1 };

__device__ int g_gemm_tc_error;      // 0, or the code of the first wait that ran out

struct GemmArgs {
    void* y;
    int ldy;
    int M, N, K;          // N: output columns (EPI_GATED: W has 2N rows)
    int out_f32;
    int act;
    int m_tiles, n_tiles;
};

using namespace tc;

// Operand and instruction descriptors of this kernel's tile shapes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) { return desc_kmajor(smem_addr); }
__device__ __forceinline__ uint32_t umma_idesc() { return idesc_bf16(BM, BN); }
__device__ __forceinline__ float act_apply(float z, int act) { return fast_gate_act(z, act); }
__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_tc_error, code);
}
// after the block gave up: loads in flight are waited for under the second flag
__device__ __forceinline__ bool drain_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_tc_error, code, true);
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                             const __grid_constant__ CUtensorMap map_w, GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE_BYTES);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(base);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                   acc_empty0 = acc_full0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;
    const int total_tiles = g.m_tiles * g.n_tiles;
    constexpr int OUT_COLS = EPI == EPI_GATED ? BN / 2 : BN;      // output columns of a tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8 * s, 1);
            mbar_init(acc_empty0 + 8 * s, 4);     // one arrival per epilogue warp
        }
        give_up[0] = 0;
        give_up[1] = 0;      // the flag of the drain waits below
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

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                   // stages filled so far, over all tiles
            bool ok = true;
            pdl_wait();                                   // (nothing of this kernel touches memory before its first operands)
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m_tile = tile % g.m_tiles, n_tile = tile / g.m_tiles;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    if (!wait_on(empty0 + 8 * s, phase ^ 1, give_up, 1)) { ok = false; break; }
                    const uint32_t full = full0 + 8 * s, a_dst = stage0 + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_x, kb * BK, m_tile * BM, full);
                    if (EPI == EPI_GATED) {
                        tma_load_2d(b_dst, &map_w, kb * BK, n_tile * OUT_COLS, full);
                        tma_load_2d(b_dst + B_BYTES / 2, &map_w, kb * BK, g.N + n_tile * OUT_COLS, full);
                    } else {
                        tma_load_2d(b_dst, &map_w, kb * BK, n_tile * BN, full);
                    }
                }
            }
            pdl_trigger();
            if (*give_up) {
                // let the loads that are still in flight land before the block goes away
                for (int j = max(0, it - STAGES); j < it; ++j)
                    drain_on(full0 + 8 * (j % STAGES), (j / STAGES) & 1, give_up, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc();
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
                const int as = local & 1;                 // accumulator of this tile
                ok = wait_on(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, give_up, 5);
                if (!ok) break;
                fence_after_sync();
                const uint32_t acc = tmem + as * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = wait_on(full0 + 8 * s, (it / STAGES) & 1, give_up, 2);
                    if (!ok) break;
                    fence_after_sync();
                    const uint64_t a = umma_desc(stage0 + s * STAGE_BYTES), b = umma_desc(stage0 + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma(acc, a + 2 * k, b + 2 * k, idesc, (kb | k) != 0);     // 32 bytes along K per step
                    umma_commit(empty0 + 8 * s);
                }
                if (ok) umma_commit(acc_full0 + 8 * as);
            }
        }
    } else {
        const int quarter = warp & 3;                        // the 32 lanes of tensor memory this warp may read
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const int m_tile = tile % g.m_tiles, n_tile = tile / g.m_tiles;
            const int as = local & 1;
            const bool ready = wait_on(acc_full0 + 8 * as, (local >> 1) & 1, give_up, 3);
            if (!__all_sync(0xffffffffu, ready)) break;       // the warp leaves together
            fence_after_sync();
            const uint32_t acc = tmem + as * BN + ((uint32_t)(quarter * 32) << 16);
            const int row = m_tile * BM + quarter * 32 + lane;
            const int col0 = n_tile * OUT_COLS;
            for (int c = 0; c < OUT_COLS; c += 32) {
                uint32_t v[32], u[32];
                tmem_ld32(acc + c, v);
                if (EPI == EPI_GATED) tmem_ld32(acc + OUT_COLS + c, u);
                tmem_wait_ld();
                if (c + 32 >= OUT_COLS) {
                    // everything of this accumulator is in registers: hand it back before the stores
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * as);
                }
                float o[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    o[i] = __uint_as_float(v[i]);
                    if (EPI == EPI_GATED) o[i] = act_apply(o[i], g.act) * __uint_as_float(u[i]);
                }
                if (row < g.M) {
                    const int col = col0 + c;
                    const bool whole = col + 32 <= g.N;
                    if (g.out_f32) {
                        float* dst = reinterpret_cast<float*>(g.y) + (size_t)row * g.ldy + col;
                        if (whole && (g.ldy & 3) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4)
                                *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                        } else {
                            for (int i = 0; i < 32; ++i) if (col + i < g.N) dst[i] = o[i];
                        }
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(g.y) + (size_t)row * g.ldy + col;
                        if (whole && (g.ldy & 7) == 0) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 p;
                                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&p);
#pragma unroll
                                for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(o[i + 2 * e], o[i + 2 * e + 1]);
                                *reinterpret_cast<uint4*>(dst + i) = p;
                            }
                        } else {
                            for (int i = 0; i < 32; ++i) if (col + i < g.N) dst[i] = __float2bfloat16_rn(o[i]);
                        }
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    return make_map_2d(map, ptr, rows, cols, ld, box_rows);
}

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;

template <int EPI>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& g, cudaStream_t stream) {
    static bool raised = false;
    const int sms = device_sms();
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const int tiles = g.m_tiles * g.n_tiles;
    return launch_pdl(gemm_tc_kernel<EPI>, dim3(tiles < sms ? tiles : sms), dim3(THREADS), SMEM_BYTES, stream, mx, mw, g);
}

}  // namespace

// epilogue 0: Y = X W^T (W has N rows); 1: Y = act(X Wg^T) * (X Wu^T), W = [Wg; Wu] has 2N rows and N is a
// multiple of 128.  X: M x K with ldx between rows; W: rows x K with ldw; Y: M x N with ldy, bfloat16 or
// float (out_f32).  K, ldx and ldw multiples of 8 elements, base addresses 16-byte aligned.
BROLM_API int brolm_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
                            int epilogue, int out_f32, int act, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BROLM_OK;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15)) return BROLM_ERR_ALIGNMENT;
    if (epilogue == EPI_GATED && (N % 128 != 0 || act < 0 || act > 1)) return BROLM_ERR_BAD_SIZE;
    if (epilogue != EPI_STORE && epilogue != EPI_GATED) return BROLM_ERR_BAD_SIZE;
    CUtensorMap mx, mw;
    int st = make_map(&mx, x, M, K, ldx, BM);
    if (st) return st;
    st = make_map(&mw, w, epilogue == EPI_GATED ? 2LL * N : N, K, ldw, epilogue == EPI_GATED ? BN / 2 : BN);
    if (st) return st;
    GemmArgs g;
    g.y = y; g.ldy = ldy; g.M = M; g.N = N; g.K = K; g.out_f32 = out_f32; g.act = act;
    g.m_tiles = (M + BM - 1) / BM;
    const int out_cols = epilogue == EPI_GATED ? BN / 2 : BN;
    g.n_tiles = (N + out_cols - 1) / out_cols;
    if (epilogue == EPI_GATED) return launch<EPI_GATED>(mx, mw, g, stream);
    return launch<EPI_STORE>(mx, mw, g, stream);
}

// 0 when no bounded wait of any launch so far ran out; else the code of the first one (1 loader,
// 2 and 5 issuer, 3 epilogue, 4 drain).  Synchronises the device.  `reset` clears it.
BROLM_API int brolm_gemm_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_tc_error, &zero, sizeof(int));
    }
    return v;
}

BROLM_WAIT_CONTROL(gemm_tc)
