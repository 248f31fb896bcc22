// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in wlejon/brolm; it exists for hosts of
// this library that must not call cudaMalloc: code that runs inside someone
// else's memory plan (an embedding runtime with a fixed arena, a real-time
// loop that forbids allocator calls after start-up, a process whose device
// memory is handed out by another component).  The split-KV decode attention
// normally wants float scratch for the partial results of its splits, which
// the Python layer takes from the torch allocator.  Here that scratch is a
// fixed array inside the library instead.
//
// What to know before calling it:
//
// * The scratch is one file-scope __device__ array of
//   BROLM_ATTN_NOALLOC_MAX_FLOATS floats (4 MiB).  Every GPU on which this
//   library is loaded holds it until the process exits.
// * A call needs  batch * n_kv * group * n_splits * (head_dim + 2)  floats.
//   A call that needs more is refused with BROLM_ERR_TOO_LARGE (10003) and
//   launches nothing.  n_splits == 1 needs none.
// * The first call on a device looks up the array's device address
//   (cudaGetSymbolAddress, with that device current) and keeps it.  Make that
//   first call before any stream capture begins on that device.
// * All calls share the array and it keeps what the last call left.  Nothing
//   in it has to start at zero: every split of every (sequence, head) of a
//   call writes its place before the merge reads it.  Two calls that overlap
//   on the GPU (different streams, or a second call issued before the first
//   has finished on another stream) race on the array; keep calls on one
//   stream or order them yourself.
// * The splits of a (sequence, kv head) are merged by whichever of their
//   blocks finishes last; the blocks count themselves on a second file-scope
//   __device__ array of ticket words (g_decode_tickets in attn_mma.cuh, one
//   copy per loaded library).  Those words are shared between calls in the
//   same way as the scratch, and by the ordinary entry point
//   brolm_attn_decode_mma as well: two launches of either kind that overlap
//   on the GPU would count on the same words.  The same rule covers both:
//   one stream, or your own ordering.
// * The function calls no cudaMalloc, cudaFree or any allocating routine.
//
// Arguments and result are those of brolm_attn_decode_mma (attn_mma.cu)
// without the two scratch pointers.
#pragma once

#include <cuda_runtime.h>

#define BROLM_ATTN_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C"
#endif
int brolm_attn_decode_mma_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* cu_q,
                                  const void* kv_len, const void* k_pages, const void* v_pages,
                                  const void* page_table, int pt_stride, int ring, int page_size, int n_kv,
                                  int group, int hd, float scale, float cap, int window, int batch, int n_splits,
                                  cudaStream_t stream);
