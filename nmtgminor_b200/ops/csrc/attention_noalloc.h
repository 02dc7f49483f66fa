// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference toolkit.  It exists for hosts that embed the kernels
// without a device allocator of their own to lend: a serving process whose memory manager reserved the whole
// GPU up front, a plug-in running inside another runtime's memory pool, code that sits between the begin and
// the end of a stream capture (where cudaMalloc is not permitted), or a real-time loop that may not take the
// allocator's lock.  The regular entry point (nmtg_attn_bwd in ops_api.h) needs, for sequences longer than
// one 128-key tile, an fp32 accumulation buffer [total_q, heads * 64] that the caller allocates; here that
// buffer is a fixed array compiled into the library.
//
// Limits and rules
//   * The built-in buffer holds NMTG_ATTN_NOALLOC_MAX_FLOATS floats (16 MiB).  Every GPU that loads the
//     library carries this array from load to process exit, used or not.  A problem with
//     total_q * heads * 64 above the limit (and max_k > 128, i.e. one that needs the buffer at all) is
//     rejected with return code 2 and a message in `err`; nothing is launched.
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress), raises the
//     backward kernel's shared-memory limit, and keeps both; make that first call outside any stream capture.
//     Later calls, from any host thread, only bind the device's context to the thread (cudaSetDevice), build
//     their descriptors and enqueue work.
//   * All calls share the one array and it keeps whatever the previous call left in it.  Each call clears the
//     part it is about to use (an asynchronous memset on `stream`) before its kernels run.  Two calls whose
//     work can overlap on the GPU (different streams, no dependency between them) would accumulate into the
//     same memory and corrupt each other: serialise them.
//   * No cudaMalloc, cudaFree, or other allocating routine is called.  All five tensor-map descriptors (q, k, v,
//     dO and the fp32 view of the built-in array) are encoded into variables on the caller's stack on every
//     call; the descriptor cache and its lock, which the regular entry point uses, are not touched.  Inputs
//     and outputs are the caller's.
//   * Dropout is supported with the same (seed, stream id) convention as the regular entry point.
//
// Returns 0 on success; 1 = bad argument, 2 = problem larger than the built-in buffer, 3 = CUDA error
// (message copied into `err`, which may be null).
#pragma once
#include <cuda_runtime.h>

#define NMTG_ATTN_NOALLOC_MAX_FLOATS (4L << 20)

#ifdef __cplusplus
extern "C" {
#endif

int nmtg_attn_bwd_noalloc(const void* q, int ld_q, const void* k, int ld_k, const void* v, int ld_v,   // bf16 [tokens, heads*64]
                          const void* out, int ld_out, const float* lse, long lse_stride,              // forward results
                          const void* d_out, int ld_dout,                                              // incoming gradient
                          void* dq, int ld_dq, void* dk, int ld_dk, void* dv, int ld_dv,               // outputs (bf16)
                          const int* cu_q, const int* cu_k, int batch, int num_heads, int max_q, int max_k, int total_q,
                          int total_k, int causal, float scale, float dropout_p, unsigned long long seed,
                          unsigned long long stream_id, int* status, cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
