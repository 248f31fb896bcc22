// The allocation-free variant of the split-KV decode attention; see
// attn_decode_noalloc.h for who needs it and what its limits are.  The
// kernels are the ones of attn_mma.cuh, unchanged; only the scratch differs.
#include "attn_decode_noalloc.h"

#include "attn_mma.cuh"

namespace {

// Partial outputs first, then the (max, sum) pairs of the splits.
static __device__ __align__(256) float g_noalloc_scratch[BROLM_ATTN_NOALLOC_MAX_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES];     // device address of the array, per device, looked up once

// In host code the array's name stands for a host-side shadow, not for device
// memory; the address a kernel can use comes from cudaGetSymbolAddress.
int scratch_address(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return BROLM_ERR_TOO_LARGE;
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_addr[dev];
    return BROLM_OK;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int brolm_attn_decode_mma_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                  const void* kv_len, const void* k_pages, const void* v_pages,
                                  const void* page_table, int pt_stride, int ring, int page_size, int n_kv,
                                  int group, int hd, float scale, float cap, int window, int batch, int n_splits,
                                  cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    int st = check_common(hd, group, n_kv, q_stride, out_stride, batch);
    if (st) return st;
    if (group > 16) return BROLM_ERR_TOO_LARGE;
    if (page_size != KT || ring <= 0 || ring % KT != 0 || n_splits < 1 || n_splits > 4096) return BROLM_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return BROLM_ERR_ALIGNMENT;
    const long long slots = (long long)batch * n_kv * group * n_splits;
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (n_splits > 1) {
        if (slots * (hd + 2) > (long long)BROLM_ATTN_NOALLOC_MAX_FLOATS) return BROLM_ERR_TOO_LARGE;
        float* base = nullptr;
        st = scratch_address(&base);
        if (st) return st;
        part_o = base;
        part_ml = base + slots * hd;
    }
    MmaArgs a = {};
    a.q = (const bf16*)q; a.out = (bf16*)out; a.q_stride = q_stride; a.out_stride = out_stride;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len;
    a.k_pages = (const bf16*)k_pages; a.v_pages = (const bf16*)v_pages; a.page_table = (const int32_t*)page_table;
    a.pt_stride = pt_stride; a.ring = ring;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window;
    a.n_splits = n_splits; a.part_o = part_o; a.part_ml = part_ml;
    if (hd == 64) return launch_decode<64, true>(a, batch, stream);
    if (hd == 128) return launch_decode<128, true>(a, batch, stream);
    if (hd == 256) return launch_decode<256, true>(a, batch, stream);
    if (hd < 64) return launch_decode<64, false>(a, batch, stream);
    if (hd < 128) return launch_decode<128, false>(a, batch, stream);
    return launch_decode<256, false>(a, batch, stream);
}
