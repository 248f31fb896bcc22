// bfloat16 matrix product for many tokens on pairs of SMs (tcgen05 cta_group::2):
//     Y[M,N] = X[M,K] * W[N,K]^T        (float accumulation)
// The same product and epilogues as gemm_tc.cu, with two blocks of a cluster working on one 256 x 256
// tile of Y.  Each block loads its own 128 rows of X and only its own half (128 rows) of the W tile;
// one thread of the first block issues tcgen05.mma.cta_group::2 (M 256, N 256), which reads A and the
// halves of B from both blocks' shared memory and leaves rows 0-127 of the tile in the first block's
// tensor memory and rows 128-255 in the second's.  A stage is 32 KB per block instead of 48 KB (six
// stages instead of four), and every byte of W is read from shared memory by one multiplication for
// 256 rows of X instead of 128.
//
//   warp 0 (both blocks)   one thread: TMA loads of this block's tiles; their bytes are counted on the
//                          first block's barrier (the cta_group::2 form of the load)
//   warp 1 (first block)   one thread: the multiplications; tcgen05.commit with a multicast hands a stage
//                          back to both loaders and a finished accumulator to both epilogues
//   warps 2-5 (both)       epilogue of this block's 128 rows; the accumulator is handed back on the first
//                          block's barrier (the second block arrives there through the cluster)
//
// Every mbarrier wait is bounded as in gemm_tc.cu; the two blocks meet at a cluster barrier after set-up
// and before they free their tensor memory.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, PM = 256, BN = 256, HN = 128, BK = 64, STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = HN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;      // two accumulators of 256 columns

enum : int { EPI_STORE = 0, EPI_GATED = 1 };

__device__ int g_gemm_tc2_error;

struct GemmArgs {
    void* y;
    int ldy;
    int M, N, K;          // N: output columns (EPI_GATED: W has 2N rows)
    int out_f32;
    int act;
    int m_tiles, n_tiles;
};

using namespace tc;

__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_tc2_error, code);
}
// after the block gave up: loads in flight are waited for under the second flag
__device__ __forceinline__ bool drain_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_gemm_tc2_error, code, true);
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
// The cta_group::2 forms.  A shared-memory address with bit 24 cleared names the same place in the first
// block of the pair.
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar & PEER_MASK) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {      // arrives on the barrier in both blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {     // whole warp, in both blocks
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mbar_arrive_first_block(uint32_t bar) {                  // from either block
    asm volatile("{\n.reg .b32 remote;\nmapa.shared::cluster.u32 remote, %0, 0;\nmbarrier.arrive.shared::cluster.b64 _, [remote];\n}"
                 ::"r"(bar) : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, GemmArgs g) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = smem_raw;
    const uint32_t rank = cluster_rank();
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(base);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                   acc_empty0 = acc_full0 + 16;
    const bool aligned = (stage0 & 1023u) == 0;               // both blocks have the same layout

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;
    const int total_tiles = g.m_tiles * g.n_tiles;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    constexpr int OUT_COLS = EPI == EPI_GATED ? BN / 2 : BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8 * s, 1);
            mbar_init(acc_empty0 + 8 * s, 8);     // four epilogue warps of each block
        }
        give_up[0] = aligned ? 0 : 1;
        give_up[1] = 0;
        give_up[2] = tc::g_stall_code;
        if (!aligned) atomicCAS(&g_gemm_tc2_error, 0, 13);
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    fence_before_sync();
    cluster_sync_all();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = !*give_up;
            // Launched with programmatic stream serialization: the block may be here while the kernel before
            // it still runs.  Nothing of this kernel touches memory before its first operands have arrived,
            // so the loader's wait is the kernel's.
            pdl_wait();
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
                const int m_tile = tile % g.m_tiles, n_tile = tile / g.m_tiles;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_on(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 1)) { ok = false; break; }
                    const uint32_t full = full0 + 8 * s, a_dst = stage0 + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    if (rank == 0) mbar_expect_tx(full, 2 * STAGE_BYTES);          // both blocks' bytes land on this barrier
                    tma_load_2d_pair(a_dst, &map_x, kb * BK, m_tile * PM + (int)rank * BM, full);
                    if (EPI == EPI_GATED)
                        tma_load_2d_pair(b_dst, &map_w, kb * BK, (rank == 0 ? 0 : g.N) + n_tile * OUT_COLS, full);
                    else
                        tma_load_2d_pair(b_dst, &map_w, kb * BK, n_tile * BN + (int)rank * HN, full);
                }
            }
            pdl_trigger();                                  // the operands are asked for: the next kernel may move in
            if (*give_up && rank == 0) {
                for (int j = max(0, it - STAGES); j < it; ++j)
                    drain_on(full0 + 8 * (j % STAGES), (j / STAGES) & 1, give_up, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = idesc_bf16(PM, BN);
            int it = 0, local = 0;
            bool ok = !*give_up;
            for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local) {
                const int as = local & 1;
                ok = wait_on(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, give_up, 5);
                if (!ok) break;
                fence_after_sync();
                const uint32_t acc = tmem + as * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = wait_on(full0 + 8 * s, (it / STAGES) & 1, give_up, 2);
                    if (!ok) break;
                    fence_after_sync();
                    const uint64_t a = desc_kmajor(stage0 + s * STAGE_BYTES), b = desc_kmajor(stage0 + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) umma_pair(acc, a + 2 * k, b + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(empty0 + 8 * s);
                }
                if (ok) umma_commit_pair(acc_full0 + 8 * as);
            }
        }
    } else {
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = pair; tile < total_tiles; tile += n_pairs, ++local) {
            const int m_tile = tile % g.m_tiles, n_tile = tile / g.m_tiles;
            const int as = local & 1;
            const bool ready = wait_on(acc_full0 + 8 * as, (local >> 1) & 1, give_up, 3);
            if (!__all_sync(0xffffffffu, ready)) break;
            fence_after_sync();
            const uint32_t acc = tmem + as * BN + ((uint32_t)(quarter * 32) << 16);
            const int row = m_tile * PM + (int)rank * BM + quarter * 32 + lane;
            const int col0 = n_tile * OUT_COLS;
            for (int c = 0; c < OUT_COLS; c += 32) {
                uint32_t v[32], u[32];
                tmem_ld32(acc + c, v);
                if (EPI == EPI_GATED) tmem_ld32(acc + OUT_COLS + c, u);
                tmem_wait_ld();
                if (c + 32 >= OUT_COLS) {
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_first_block(acc_empty0 + 8 * as);
                }
                float o[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    o[i] = __uint_as_float(v[i]);
                    if (EPI == EPI_GATED) o[i] = fast_gate_act(o[i], g.act) * __uint_as_float(u[i]);
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
    cluster_sync_all();                 // neither block frees memory the other may still signal
    if (warp == 1) tmem_dealloc_pair(tmem, TMEM_COLS);
}

constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;

template <int EPI>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& g, cudaStream_t stream) {
    static bool raised = false;
    const int sms = device_sms();
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const int tiles = g.m_tiles * g.n_tiles;
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    return launch_pdl(gemm_tc2_kernel<EPI>, dim3(2 * pairs), dim3(THREADS), SMEM_BYTES, stream, mx, mw, g);
}

}  // namespace

// The arguments of brolm_gemm_tc.
BROLM_API int brolm_gemm_tc2(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
                             int epilogue, int out_f32, int act, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BROLM_OK;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15)) return BROLM_ERR_ALIGNMENT;
    if (epilogue == EPI_GATED && (N % 128 != 0 || act < 0 || act > 1)) return BROLM_ERR_BAD_SIZE;
    if (epilogue != EPI_STORE && epilogue != EPI_GATED) return BROLM_ERR_BAD_SIZE;
    CUtensorMap mx, mw;
    int st = make_map_2d(&mx, x, M, K, ldx, BM);
    if (st) return st;
    st = make_map_2d(&mw, w, epilogue == EPI_GATED ? 2LL * N : N, K, ldw, HN);
    if (st) return st;
    GemmArgs g;
    g.y = y; g.ldy = ldy; g.M = M; g.N = N; g.K = K; g.out_f32 = out_f32; g.act = act;
    g.m_tiles = (M + PM - 1) / PM;
    const int out_cols = epilogue == EPI_GATED ? BN / 2 : BN;
    g.n_tiles = (N + out_cols - 1) / out_cols;
    if (epilogue == EPI_GATED) return launch<EPI_GATED>(mx, mw, g, stream);
    return launch<EPI_STORE>(mx, mw, g, stream);
}

BROLM_API int brolm_gemm_tc2_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_tc2_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_tc2_error, &zero, sizeof(int));
    }
    return v;
}

BROLM_WAIT_CONTROL(gemm_tc2)
