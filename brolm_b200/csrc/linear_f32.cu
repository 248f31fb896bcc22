// True 32-bit matrix product  Y[M,N] = X[M,K] * W[N,K]^T  on CUDA cores
// (wlejon/brolm include/brolm/detail/compute.h:49-86, the float branch).
//
// No tensor cores and no reduced-precision mode: every product and sum is an
// IEEE float fma.  Each output element is the sum over k in ascending order,
// whatever M is and wherever the row stands in the batch, so a row gives the
// same bits alone, in a prompt or in a batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ X, int ldx,
                                                         const float* __restrict__ W, int ldw,
                                                         float* __restrict__ Y, int ldy, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;            // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;        // loader: row lr, k offset lk..lk+3
    const bool vec = (K % 4 == 0) && (ldx % 4 == 0) && (ldw % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
        const int k = k0 + lk;
        if (m0 + lr < M) {
            const float* p = X + (size_t)(m0 + lr) * ldx + k;
            if (vec && k + 3 < K) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                a[0] = t.x; a[1] = t.y; a[2] = t.z; a[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) a[i] = p[i];
            }
        }
        if (n0 + lr < N) {
            const float* p = W + (size_t)(n0 + lr) * ldw + k;
            if (vec && k + 3 < K) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                b[0] = t.x; b[1] = t.y; b[2] = t.z; b[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) b[i] = p[i];
            }
        }
        __syncthreads();   // the tile before this one is consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = a[i];
            Bs[lk + i][lr] = b[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Y[(size_t)m * ldy + n] = acc[i][j];
        }
    }
}

}  // namespace

BROLM_API int brolm_linear_f32(const void* x, int ldx, const void* w, int ldw, void* y, int ldy, int M, int N, int K,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return BROLM_OK;
    if (K <= 0) return BROLM_ERR_BAD_SIZE;
    const long long gy = (M + BM - 1) / BM;
    if (gy > 65535) return BROLM_ERR_TOO_LARGE;
    dim3 grid((N + BN - 1) / BN, (unsigned)gy);
    linear_f32_kernel<<<grid, 256, 0, stream>>>((const float*)x, ldx, (const float*)w, ldw, (float*)y, ldy, M, N, K);
    return launch_status();
}
