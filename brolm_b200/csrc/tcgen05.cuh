// Building blocks shared by the tcgen05 kernels (sm_100a): mbarriers with bounded
// waits, TMA tile loads, shared-memory and instruction descriptors for
// tcgen05.mma, tensor-memory loads and stores, and the host-side tensor-map encoder.
//
// Bounded waits.  No wait in these kernels can spin for ever: mbar_wait gives up
// after g_wait_cycles clock cycles (about a second unless the host sets another
// limit), raises the block's give-up flag that every other waiting role polls,
// and records a code in the kernel file's error word.  The kernel then lets its
// outstanding loads land, frees its tensor memory and returns; the launch's
// results are not valid and the host learns of it through the file's status
// function.
//
// That path can be exercised without a fault: every library built from this
// header exports brolm_<library>_wait_control(cycles, stall_code).  `cycles`
// sets the limit (<= 0: the default); a non-zero `stall_code` makes the waits
// that carry this code behave as if their barrier never completed, so they run
// into the limit and the kernel gives up as it would for a load that never
// arrived.  Nothing hangs and nothing traps; the context stays usable.
#pragma once

#include "common.cuh"

#include <cuda.h>

namespace tc {

constexpr long long WAIT_CYCLES = 2000000000ll;
__device__ long long g_wait_cycles = WAIT_CYCLES;     // one copy per library: this header is its only definition
__device__ int g_stall_code = 0;                      // tests only: waits with this code never see their barrier
                                                      // (a kernel copies it to give_up[2] when it starts)

static inline int set_wait_control(long long cycles, int stall_code) {
    const long long c = cycles > 0 ? cycles : WAIT_CYCLES;
    cudaError_t e = cudaMemcpyToSymbol(g_wait_cycles, &c, sizeof(c));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_stall_code, &stall_code, sizeof(stall_code));
    return (int)e;
}
#define BROLM_WAIT_CONTROL(library)                                                        \
    BROLM_API int brolm_##library##_wait_control(long long cycles, int stall_code) {       \
        return tc::set_wait_control(cycles, stall_code);                                   \
    }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
// Returns false when it gave up: its own limit ran out (then *error gets `code`, if it was 0) or
// another role of the block had already given up.  give_up: three ints in shared memory that the
// kernel sets when it starts: [0] the block's give-up flag, [1] that of the drain waits, [2] g_stall_code.
// `flags`: the three ints; `drain`: one of the waits that let loads in flight land after the block gave up
// (they watch flags[1] and are never stalled).
__device__ inline bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* flags, int* error, int code,
                                 bool drain = false) {
    volatile int* give_up = flags + (drain ? 1 : 0);
    const bool stalled = !drain && flags[2] == code;          // (0 in every ordinary launch)
    if (!stalled && mbar_try(bar, parity)) return true;       // (try_wait itself may hold the thread for a while)
    const long long t0 = clock64(), limit = g_wait_cycles;
    while (true) {
        if (!stalled && mbar_try(bar, parity)) return true;
        if (*give_up) return false;
        if (clock64() - t0 > limit) {
            *give_up = 1;
            atomicCAS(error, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}

// Shared-memory operand descriptors (128-byte swizzle, descriptor version of sm_100).
// K-major: rows of 128 bytes (64 bf16 along K), eight-row groups 1024 bytes apart; 16 further
// along K is +32 bytes on the start address, i.e. +2 on the descriptor.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major: 64 elements of the M or N side contiguous (128 bytes), rows are steps along K.  lbo: bytes
// / 16 to the next 64 elements of the M/N side; sbo: bytes / 16 to the next eight K rows.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo & 0x3fffu) << 16) | ((uint64_t)(sbo & 0x3fffu) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor of kind::f16: bf16 x bf16 -> f32, A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n, int b_mn_major = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
// The A operand from tensor memory: row i of A in lane i, two consecutive bfloat16 along K in each
// 32-bit column (K 16 = eight columns); A is K-major by construction.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {     // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {       // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns: thread t of the warp gets lane (quarter * 32 + t), columns c .. c + 31.
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
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
// act(z) = z * sigmoid(k):  k = z for silu (act 1);  k = 2 sqrt(2/pi) (z + 0.044715 z^3) for the tanh form of
// gelu (act 0), since 0.5 (1 + tanh(u)) = sigmoid(2u).  The approximations' relative error is about 1e-6.
__device__ __forceinline__ float fast_gate_act(float z, int act) {
    const float k = act == 0 ? 1.5957691216057308f * (z + 0.044715f * z * z * z) : z;
    return z * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * k));
}

// ---- host: tensor maps (the driver's encoder is fetched through the runtime, nothing links to libcuda)
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static inline EncodeTiled encoder() {
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
// bfloat16 tensor of `rank` dims (innermost first), 128-byte swizzle, out-of-range reads as zero.
// strides_bytes has rank - 1 entries (dims 1 .. rank-1); box[0] * 2 must be 128.
static inline int make_map_bf16(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims,
                                const cuuint64_t* strides_bytes, const cuuint32_t* box) {
    EncodeTiled enc = encoder();
    if (!enc) return BROLM_ERR_BAD_SIZE;
    const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims,
                           strides_bytes, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BROLM_OK : BROLM_ERR_ALIGNMENT;
}
// rows x cols matrix, row-major with `ld` elements between rows; box = box_rows x 64 columns.
static inline int make_map_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld,
                              int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    return make_map_bf16(map, ptr, 2, dims, strides, box);
}

static inline int device_sms() { return device_sm_count(); }

}  // namespace tc
