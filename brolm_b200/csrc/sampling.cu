// Token sampling on the device, one block per row of float logits.
//
// Greedy: the first maximum wins (wlejon/brolm src/detail/generate.cpp:38-48).
// Temperature sampling follows src/detail/generate.cpp:68-142: logits / T,
// softmax, top-k, then top-p over what top-k kept, then one draw from the
// renormalised rest.  Two things differ from the reference by design and are
// restated in the test oracle: the kept set is found by a threshold on the
// probability instead of a sort, so tokens that tie with the last kept one are
// all kept; and the draw walks the kept tokens in token-id order with a
// counter-based uniform number instead of std::mt19937_64.
#include "common.cuh"

#include <algorithm>

#include <float.h>

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform number in [0, 1) with 24 bits, a pure function of (seed, stream, counter).
__device__ __forceinline__ float uniform24(uint64_t seed, uint64_t stream, uint64_t counter) {
    const uint64_t x = splitmix64(splitmix64(splitmix64(seed) ^ stream) ^ counter);
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int vocab,
                                                         int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // four values a load, four loads in flight: the row is read in a few trips to memory
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = vocab >> 2;
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = row4[i];
            const float vs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (vs[e] > best) { best = vs[e]; idx = 4 * i + e; }     // ids rise within a thread: the first maximum stays
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (v > best) { best = v; idx = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
        idx = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

struct CountMass { float count, mass; };

// Number and mass of the entries with e >= the float whose bits are thr.
__device__ CountMass count_mass(const float* row, int vocab, float inv_t, float zmax, uint32_t thr, float* scratch) {
    float c = 0.0f, s = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float e = expf(row[i] * inv_t - zmax);
        if (__float_as_uint(e) >= thr) { c += 1.0f; s += e; }
    }
    CountMass r;
    r.count = block_sum(c, scratch);
    r.mass = block_sum(s, scratch);
    return r;
}

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int vocab,
                                                         float temperature, int top_k, float top_p, uint64_t seed,
                                                         const int32_t* __restrict__ streams, uint64_t counter,
                                                         int32_t* __restrict__ out) {
    __shared__ float scratch[33];
    __shared__ float warp_tot[32];
    __shared__ int chosen, last_kept;
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const float inv_t = 1.0f / temperature;

    float zmax = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) zmax = fmaxf(zmax, row[i] * inv_t);
    zmax = block_max(zmax, scratch);
    float total = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) total += expf(row[i] * inv_t - zmax);
    total = block_sum(total, scratch);

    // the kept set is {e >= float(thr)}
    uint32_t thr = 0;
    const uint32_t top = 0x3f800001u;   // just above 1.0f, the largest e
    if (top_k > 0 && top_k < vocab) {
        uint32_t lo = 0, hi = top;      // count(lo) >= k, count(hi) = 0
        while (hi - lo > 1) {
            const uint32_t mid = lo + ((hi - lo) >> 1);
            if (count_mass(row, vocab, inv_t, zmax, mid, scratch).count >= (float)top_k) lo = mid; else hi = mid;
        }
        thr = lo;
    }
    if (top_p < 1.0f) {
        const float target = fmaxf(top_p * total, FLT_MIN);
        if (count_mass(row, vocab, inv_t, zmax, thr, scratch).mass >= target) {
            uint32_t lo = thr, hi = top;   // mass(lo) >= target, mass(hi) = 0
            while (hi - lo > 1) {
                const uint32_t mid = lo + ((hi - lo) >> 1);
                if (count_mass(row, vocab, inv_t, zmax, mid, scratch).mass >= target) lo = mid; else hi = mid;
            }
            thr = lo;
        }
    }

    // draw in token-id order: thread t owns ids [t*chunk, (t+1)*chunk)
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
    float mine = 0.0f;
    int my_last = -1;
    for (int i = begin; i < end; ++i) {
        const float e = expf(row[i] * inv_t - zmax);
        if (__float_as_uint(e) >= thr) { mine += e; my_last = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (threadIdx.x == 0) { chosen = 0x7fffffff; last_kept = -1; }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    float before = 0.0f, kept_total = 0.0f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) {
        if (w < warp) before += warp_tot[w];
        kept_total += warp_tot[w];
    }
    const float excl = before + (incl - mine);
    const float u = uniform24(seed, (uint64_t)(uint32_t)streams[blockIdx.x], counter);
    const float r = u * kept_total;
    if (my_last >= 0) atomicMax(&last_kept, my_last);
    if (mine > 0.0f && r >= excl && r < excl + mine) {
        float acc = excl;
        for (int i = begin; i < end; ++i) {
            const float e = expf(row[i] * inv_t - zmax);
            if (__float_as_uint(e) >= thr) {
                acc += e;
                if (r < acc) { atomicMin(&chosen, i); break; }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = chosen != 0x7fffffff ? chosen : max(last_kept, 0);
}

// The same result with several blocks per row, for a few rows of a large vocabulary (one block would
// read a megabyte alone).  A block folds its part of the row, then offers (value, index) as one 64-bit key
// whose order is: greater value first, then smaller index; the row's key is an atomic maximum, and the block
// that arrives last writes the index and puts the row's key and counter back to zero, so that the launch
// needs no memset before it (it can be captured in a graph).  The keys and counters are static: launches
// that use them at the same time on different streams would disturb each other.
constexpr int ARGMAX_MAX_ROWS = 1024;
__device__ unsigned long long g_argmax_key[ARGMAX_MAX_ROWS];
__device__ unsigned int g_argmax_count[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(THREADS) argmax_parts_kernel(const float* __restrict__ logits, int vocab,
                                                               int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const int r = blockIdx.x, parts = gridDim.y;
    const float4* row4 = reinterpret_cast<const float4*>(logits + (size_t)r * vocab);     // vocab % 4 == 0, aligned
    const int n4 = vocab >> 2, per = (n4 + parts - 1) / parts;
    const int lo = blockIdx.y * per, hi = min(n4, lo + per);
    float best = -INFINITY;
    int idx = 0x7fffffff;
#pragma unroll 4
    for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) {
        const float4 v = row4[i];
        const float vs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (vs[e] > best) { best = vs[e]; idx = 4 * i + e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = idx; }
    __syncthreads();
    if (warp != 0) return;
    best = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
    idx = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (lane != 0) return;
    const unsigned int bits = __float_as_uint(best);
    const unsigned int ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);     // rises with the value
    atomicMax(&g_argmax_key[r], ((unsigned long long)ordered << 32) | (0xffffffffu - (unsigned int)idx));
    __threadfence();
    if (atomicAdd(&g_argmax_count[r], 1u) == (unsigned int)parts - 1) {
        __threadfence();
        const unsigned long long key = atomicExch(&g_argmax_key[r], 0ull);
        g_argmax_count[r] = 0;
        const unsigned int found = 0xffffffffu - (unsigned int)(key & 0xffffffffu);
        out[r] = found == 0x7fffffffu ? 0 : (int32_t)found;
    }
}

}  // namespace

BROLM_API int brolm_argmax(const void* logits, int rows, int vocab, void* out, cudaStream_t stream) {
    if (rows <= 0) return BROLM_OK;
    if (vocab <= 0) return BROLM_ERR_BAD_SIZE;
    // about two blocks per SM in all, each with at least 8192 values
    const int parts = std::min(std::min(64, 2 * device_sm_count() / rows), vocab / 8192);
    if (parts >= 2 && rows <= ARGMAX_MAX_ROWS && (vocab & 3) == 0 && ((uintptr_t)logits & 15) == 0) {
        argmax_parts_kernel<<<dim3(rows, parts), THREADS, 0, stream>>>((const float*)logits, vocab, (int32_t*)out);
        return launch_status();
    }
    argmax_kernel<<<rows, THREADS, 0, stream>>>((const float*)logits, vocab, (int32_t*)out);
    return launch_status();
}

// temperature > 0.  top_k <= 0 and top_p >= 1 switch the filters off.
BROLM_API int brolm_sample(const void* logits, int rows, int vocab, float temperature, int top_k, float top_p,
                           unsigned long long seed, const void* streams, unsigned long long counter, void* out,
                           cudaStream_t stream) {
    if (rows <= 0) return BROLM_OK;
    if (vocab <= 0 || !(temperature > 0.0f)) return BROLM_ERR_BAD_SIZE;
    sample_kernel<<<rows, THREADS, 0, stream>>>((const float*)logits, vocab, temperature, top_k, top_p,
                                                (uint64_t)seed, (const int32_t*)streams, (uint64_t)counter,
                                                (int32_t*)out);
    return launch_status();
}
