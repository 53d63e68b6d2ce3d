// rb_attn_decode_static: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference (wenhaoli-xmu/ReTurn allocates the
// partial-result buffers of its split decode kernel with torch on every call,
// rollout/attention.py:566-569).  It exists for callers of this library that cannot allocate
// device memory at the moment of the call:
//   * a host program that handed all free device memory to the KV pool at start-up and keeps no
//     allocator around that could serve a later request;
//   * a latency-critical decode loop, where cudaMalloc / cudaFree may stall the whole device and a
//     caching allocator may fall back to them at any call;
//   * code that links this library without PyTorch and so has no tensor allocator at all.
// The partial results of the splits (what rb_attn_decode takes as `scratch`) live in a
// file-scope device array inside the library instead: RB_ATTN_STATIC_SCRATCH_FLOATS floats
// (4 MiB), which every GPU that loads the library holds until the process exits.
//
// Arguments are those of rb_attn_decode without `scratch`.  Returns 0, a cudaError_t of the
// launch, or RB_ERR_SCRATCH_TOO_LARGE when n_dec * Hq * num_splits * (HEAD_DIM + 2) exceeds the
// array (use fewer splits or fewer tokens per call).  It calls no cudaMalloc, cudaFree or any
// allocating library routine.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
// that device current) and sets the kernels' shared-memory limit on that device; both are kept
// per device and guarded by a lock, so any device and any host thread may make the first call.
// Make that first call before any stream capture begins.
//
// All calls share the one array, which keeps the last call's contents.  Nothing in it has to
// start at zero: every slot that the merge step reads was written earlier in the same call.
// Two calls that overlap on the GPU (different streams, or the same stream from two threads
// without ordering) race on the array: keep calls of this entry point ordered on one stream.
#pragma once

#include <cuda_runtime.h>

#define RB_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)
#define RB_ERR_SCRATCH_TOO_LARGE (-2)
#define RB_ERR_SCRATCH_LOOKUP (-3)

extern "C" {
// Floats of the built-in scratch array (RB_ATTN_STATIC_SCRATCH_FLOATS).
long long rb_attn_decode_static_capacity();

int rb_attn_decode_static(const void* q, int ld, const void* kpool, const void* vpool, const int* dec_segs,
                          int n_dec, const int* cu_q, const int* seg_kv_len, const int* block_table,
                          int bt_stride, int page_size, void* out, int Hq, int Hkv, float scale, int window,
                          int num_splits, cudaStream_t st);
}
