// Entry points of the bfloat16 tensor-core attention; the kernels are in attn_mma.cuh.
#include "attn_mma.cuh"

// Prompts that start at position 0: kv_len[b] == cu_q[b+1] - cu_q[b].  bfloat16 only,
// head_dim a multiple of 16 up to 256.
BROLM_API int brolm_attn_prefill_mma(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                     const void* k, const void* v, int kv_stride, int n_kv, int group, int hd,
                                     float scale, float cap, int window, int batch, int max_q_len,
                                     cudaStream_t stream) {
    if (batch <= 0 || max_q_len <= 0) return BROLM_OK;
    int st = check_common(hd, group, n_kv, q_stride, out_stride, batch);
    if (st) return st;
    if (kv_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return BROLM_ERR_ALIGNMENT;
    MmaArgs a = {};
    a.q = (const bf16*)q; a.out = (bf16*)out; a.q_stride = q_stride; a.out_stride = out_stride;
    a.cu_q = (const int32_t*)cu_q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.kv_stride = kv_stride;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window; a.n_splits = 1;
    a.sms = device_sm_count();
    if (hd == 64) return launch_prefill<64, true>(a, batch, max_q_len, stream);
    if (hd == 128) return launch_prefill<128, true>(a, batch, max_q_len, stream);
    if (hd == 256) return launch_prefill<256, true>(a, batch, max_q_len, stream);
    if (hd < 64) return launch_prefill<64, false>(a, batch, max_q_len, stream);
    if (hd < 128) return launch_prefill<128, false>(a, batch, max_q_len, stream);
    return launch_prefill<256, false>(a, batch, max_q_len, stream);
}

// One query token per sequence (row cu_q[b] of q) over the paged cache.  The page size is
// 64 keys.  group <= 16.  With n_splits > 1, part_o holds batch * n_q * n_splits * hd floats
// and part_ml batch * n_q * n_splits * 2 floats of scratch.
BROLM_API int brolm_attn_decode_mma(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                    const void* kv_len, const void* k_pages, const void* v_pages,
                                    const void* page_table, int pt_stride, int ring, int page_size, int n_kv,
                                    int group, int hd, float scale, float cap, int window, int batch, int n_splits,
                                    void* part_o, void* part_ml, cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    int st = check_common(hd, group, n_kv, q_stride, out_stride, batch);
    if (st) return st;
    if (group > 16) return BROLM_ERR_TOO_LARGE;
    if (page_size != KT || ring <= 0 || ring % KT != 0 || n_splits < 1 || n_splits > 4096) return BROLM_ERR_BAD_SIZE;
    if (n_splits > 1 && (!part_o || !part_ml)) return BROLM_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return BROLM_ERR_ALIGNMENT;
    MmaArgs a = {};
    a.q = (const bf16*)q; a.out = (bf16*)out; a.q_stride = q_stride; a.out_stride = out_stride;
    a.cu_q = (const int32_t*)cu_q; a.kv_len = (const int32_t*)kv_len;
    a.k_pages = (const bf16*)k_pages; a.v_pages = (const bf16*)v_pages; a.page_table = (const int32_t*)page_table;
    a.pt_stride = pt_stride; a.ring = ring;
    a.n_kv = n_kv; a.group = group; a.hd = hd; a.scale = scale; a.cap = cap; a.window = window;
    a.n_splits = n_splits; a.part_o = (float*)part_o; a.part_ml = (float*)part_ml;
    if (hd == 64) return launch_decode<64, true>(a, batch, stream);
    if (hd == 128) return launch_decode<128, true>(a, batch, stream);
    if (hd == 256) return launch_decode<256, true>(a, batch, stream);
    if (hd < 64) return launch_decode<64, false>(a, batch, stream);
    if (hd < 128) return launch_decode<128, false>(a, batch, stream);
    return launch_decode<256, false>(a, batch, stream);
}
