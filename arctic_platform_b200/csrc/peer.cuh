// Peer-memory primitives shared by the kernels that talk to other GPUs over NVLink: the per-rank pointer
// table, the epoch barrier on flags in symmetric memory (bounded waits) and the multimem helpers.
#pragma once
#include "common.cuh"

namespace apb {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  void* p[kMaxRanks];
};

// Announce `epoch` in slot `rank` of every peer's flag array, then wait until every
// slot of the local flag array has reached `epoch`.  Every block waits by itself so
// no grid-wide barrier is needed; only block 0 announces.
__device__ __forceinline__ bool epoch_barrier(const PeerPtrs& flags, int rank, int world, int epoch, int* status) {
  if (world <= 1) return true;
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    flag_store_release(static_cast<int*>(flags.p[threadIdx.x]) + rank, epoch);
  }
  if (threadIdx.x < world) {
    const int* slot = static_cast<const int*>(flags.p[rank]) + threadIdx.x;
    if (!flag_wait_ge(slot, epoch, status, kTimeoutFlag)) {
      ok_s = 0;
      // first reporter fills the record behind the code: expected epoch, the peer that never announced it, and
      // the epoch that peer's slot holds now (a stale epoch shows a peer that is a step behind, 0 one that never
      // started)
      if (status && atomicCAS(status + 1, 0, epoch) == 0) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
        status[2] = threadIdx.x;
        status[3] = seen;
      }
    }
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}


}  // namespace apb
