// Shared device helpers of the brolm_b200 kernels (sm_100a).
//
// Element types: activations and weights are float or __nv_bfloat16; every
// reduction, norm statistic, rotation, softmax and residual sum is float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define BROLM_API extern "C" __attribute__((visibility("default")))

// Element type codes used across the C interface.
enum : int { BROLM_F32 = 0, BROLM_BF16 = 1 };

// Error codes returned by the launchers (cudaError_t values are passed
// through as they are; these sit above that range).
enum : int {
    BROLM_OK = 0,
    BROLM_ERR_BAD_DTYPE = 10001,
    BROLM_ERR_BAD_SIZE = 10002,
    BROLM_ERR_TOO_LARGE = 10003,
    BROLM_ERR_ALIGNMENT = 10004,
};

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads, in a fixed order (the result does
// not depend on scheduling).  `scratch` holds at least 33 floats.  Every
// thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();               // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// The same sum with one barrier: every thread adds the warps' sums itself, in warp order.  `scratch`
// holds 2 x 32 floats and `turn` alternates (0, 1, 0, ...) between consecutive calls of a kernel, so a
// call never writes what a slower thread may still be reading from the call before.
__device__ __forceinline__ float block_sum_once(float v, float* scratch, int turn) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    float* mine = scratch + 32 * (turn & 1);
    if (lane == 0) mine[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nwarps; ++w) t += mine[w];
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// cap * tanh(x / cap); cap <= 0 leaves x as it is.
__device__ __forceinline__ float soft_cap(float x, float cap) {
    return cap > 0.0f ? cap * tanhf(x / cap) : x;
}

// Loads 8 consecutive elements (16-byte aligned for bf16, 32-byte span for
// float) into floats.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

static inline int launch_status() {
    return (int)cudaGetLastError();
}

// How many SMs the current device has (asked once per process; a host that cannot say gets the B200's 148).
static inline int device_sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl may begin
// while the kernel before it in the stream is still running; it must call
// pdl_wait() before it touches anything that kernel (or any earlier one) wrote,
// and may do work that depends on nothing before it (index arithmetic, fetching
// weights).  pdl_trigger() lets the kernel after this one start launching.
// The environment variable BROLM_NO_PDL=1 falls back to plain stream order.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// The 128-byte line at p on its way into the L1, holding no register.
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

static inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("BROLM_NO_PDL");
        on = (e && e[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
