// Allocation-free entry point of libapb200.so.
//
// This function has no counterpart in the reference platform: it exists for callers of this
// library that are not allowed to allocate device memory at the moment they need a result.
// Typical cases are code running inside a region where cudaMalloc/cudaFree are forbidden or
// would serialise the device (for instance between other libraries' stream-ordered phases),
// hosts that have handed every byte of GPU memory to a fixed arena at start-up and own no
// allocator, and latency-critical serving loops where an allocation stall is not acceptable.
//
// apb_lmhead_logprob_fwd_noalloc computes, for every row of `hidden`, the log-probability of
// `labels[row]` under softmax(hidden @ weight^T * scale), the entropy of that distribution and
// its log-sum-exp -- the same results as apb_lmhead_logprob_fwd -- but takes the per-tile
// reduction scratch from a fixed array that lives inside the library instead of from the caller.
//
// Limits and rules
//   * rows * ceil(vocab / 128) must not exceed APB_NOALLOC_MAX_TILE_RECORDS (1,310,720 records of
//     16 bytes = 20 MiB; e.g. 1024 rows at a 163,840-token vocabulary).  Larger problems are rejected
//     with APB_NOALLOC_TOO_LARGE and nothing is launched.  Every GPU that loads the library holds
//     these 20 MiB until the process exits.
//   * The function itself calls no cudaMalloc, cudaFree or any other allocating routine; inputs and
//     outputs are still supplied by the caller.
//   * The first call on a device looks up the device address of the scratch array (and configures
//     the kernel's shared-memory limit).  Make that first call outside any stream capture.  The
//     looked-up address is cached per device without a lock; host threads that race on the first
//     call each store the same address, so no serialisation is needed for that.
//   * All calls share the one scratch array, which keeps the contents of the previous call.  The
//     kernel overwrites every record it later reads, so nothing has to be cleared, but two calls
//     that overlap on the GPU (different streams, or concurrent host threads) race on the scratch:
//     serialise them.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define APB_NOALLOC_MAX_TILE_RECORDS 1310720
#define APB_NOALLOC_TOO_LARGE 301
#define APB_NOALLOC_SETUP_FAILED 302

// hidden [M,H] bf16 (row stride ldh), weight [V,H] bf16 (row stride ldw), labels [M] int32,
// row_scale [M] fp32 or NULL (then `scale` multiplies the logits).  Outputs lp / ent / lse: fp32 [M].
// Returns 0 on success, APB_NOALLOC_TOO_LARGE, APB_NOALLOC_SETUP_FAILED, or a CUDA / argument error code.
int apb_lmhead_logprob_fwd_noalloc(const void* hidden, const void* weight, const int* labels,
                                   const float* row_scale, float* lp, float* ent, float* lse, int M, int V, int H,
                                   long long ldh, long long ldw, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
