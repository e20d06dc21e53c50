// Tensor-parallel decode: the epilogue of a row-parallel projection fused with the residual add, the RMSNorm that
// follows it and the all-gather of the normalised rows.
//
// In a tensor-parallel replica of T ranks the output projection and the down projection are split along their
// input dimension, so every rank holds a partial [B, H] result, which its GEMM leaves in a LOCAL fp32 buffer in
// symmetric memory (split-K partials meet there through local red.add).  Rows are dealt out to the ranks in T
// contiguous blocks.  This kernel then runs on every rank, one CTA per owned row:
//   0. the partial buffer of the PREVIOUS call (all of its readers passed that call's barrier B) is cleared for its
//      next use while the ranks gather at barrier A;
//   1. epoch barrier A -- every rank has launched this kernel, i.e. every rank's partial is complete;
//   2. row = sum over ranks of their partial row, pulled with plain 16-byte peer loads (a reduce-scatter by
//      reading: 1/T of every peer's buffer crosses NVLink once, as full-width loads instead of fp32 atomics, which
//      measured ~25 us slower per projection at T = 8), plus the residual stream of the row;
//   3. the new residual row stays local (bf16); RMSNorm(row) * w is stored as bf16 into the activation buffer of
//      EVERY rank at the row's global position (plain peer stores over NVLink): the all-gather;
//   4. the last CTA to finish announces epoch B to all ranks, and every CTA waits until all ranks have announced
//      it, so when the kernel ends the local activation buffer holds all B rows and the next (column-parallel) GEMM
//      reads local memory only.
// Epoch numbers come from a device counter so that a captured CUDA graph can be replayed: the kernel uses
// *epoch_base + epoch_off and + 1; apb_tp_epoch_advance moves the counter on at the end of a decode step.  Every
// wait is bounded.  The reference obtains tensor-parallel decoding from vLLM's NCCL all-reduce
// (tensor_parallel_size, arctic_platform/common/ray_server.py:375-404).
#include "common.cuh"
#include "host_utils.cuh"
#include "peer.cuh"

namespace apb {

constexpr int kTpNormThreads = 256;

__global__ void __launch_bounds__(kTpNormThreads)
tp_norm_allgather_kernel(PeerPtrs flags, int rank, int world, const int* __restrict__ epoch_base, int epoch_off,
                         PeerPtrs part_ptrs, float4* __restrict__ clear_buf, long long clear_vec4,
                         __nv_bfloat16* __restrict__ resid, int has_resid,
                         const __nv_bfloat16* __restrict__ w, float eps, PeerPtrs out_ptrs, int rows_local, int H,
                         int* __restrict__ done_counter, int* status) {
  pdl_entry();
  if (clear_buf) {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i = static_cast<long long>(blockIdx.x) * kTpNormThreads + threadIdx.x; i < clear_vec4;
         i += static_cast<long long>(gridDim.x) * kTpNormThreads)
      clear_buf[i] = z;
  }
  const int epoch_a = *epoch_base + epoch_off;
  if (!epoch_barrier(flags, rank, world, epoch_a, status)) return;
  __shared__ float red[kTpNormThreads / 32];
  __shared__ int last_s;
  const int row = blockIdx.x;  // gridDim.x == rows_local
  const long long grow = static_cast<long long>(rank) * rows_local + row;
  __nv_bfloat16* rs = resid + static_cast<long long>(row) * H;
  // pass 1: x = acc (+ residual); keep x in registers (H <= 256 * 8 * 4)
  float x[4][8];
  float ss = 0.f;
  const int nv = H / 8;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int v = threadIdx.x + k * kTpNormThreads;
    if (v < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[k][j] = 0.f;
      // own partial first, then the peers in ring order so that the ranks do not all read the same peer at once
      for (int i = 0; i < world; ++i) {
        const int r = (rank + i) % world;
        const float* a = static_cast<const float*>(part_ptrs.p[r]) + grow * H + v * 8;
        const float4 p0 = *reinterpret_cast<const float4*>(a);
        const float4 p1 = *reinterpret_cast<const float4*>(a + 4);
        x[k][0] += p0.x; x[k][1] += p0.y; x[k][2] += p0.z; x[k][3] += p0.w;
        x[k][4] += p1.x; x[k][5] += p1.y; x[k][6] += p1.z; x[k][7] += p1.w;
      }
      if (has_resid) {
        const uint4 raw = *reinterpret_cast<const uint4*>(rs + v * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          x[k][2 * j] += f.x;
          x[k][2 * j + 1] += f.y;
        }
      }
      // the residual stream is carried in bf16: round first, normalise what was stored
      uint4 o;
      o.x = pack_bf16x2(x[k][0], x[k][1]);
      o.y = pack_bf16x2(x[k][2], x[k][3]);
      o.z = pack_bf16x2(x[k][4], x[k][5]);
      o.w = pack_bf16x2(x[k][6], x[k][7]);
      *reinterpret_cast<uint4*>(rs + v * 8) = o;
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(r2[j]);
        x[k][2 * j] = f.x;
        x[k][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kTpNormThreads / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
  // pass 2: normalised row to every rank's activation buffer
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int v = threadIdx.x + k * kTpNormThreads;
    if (v < nv) {
      const uint4 wraw = *reinterpret_cast<const uint4*>(w + v * 8);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
      float y[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 wf = __bfloat1622float2(w2[j]);
        y[2 * j] = x[k][2 * j] * rstd * wf.x;
        y[2 * j + 1] = x[k][2 * j + 1] * rstd * wf.y;
      }
      uint4 o;
      o.x = pack_bf16x2(y[0], y[1]);
      o.y = pack_bf16x2(y[2], y[3]);
      o.z = pack_bf16x2(y[4], y[5]);
      o.w = pack_bf16x2(y[6], y[7]);
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out_ptrs.p[r]) + grow * H + v * 8) = o;
    }
  }
  // barrier B: my rows have left; wait until everybody's rows have arrived here
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(done_counter, 1);
    last_s = (old == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
  }
  __syncthreads();
  if (last_s) {
    if (threadIdx.x == 0) *done_counter = 0;
    if (threadIdx.x < world) {
      __threadfence_system();
      flag_store_release(static_cast<int*>(flags.p[threadIdx.x]) + rank, epoch_a + 1);
    }
  }
  if (threadIdx.x < world) {
    const int* slot = static_cast<const int*>(flags.p[rank]) + threadIdx.x;
    if (!flag_wait_ge(slot, epoch_a + 1, status, kTimeoutFlag)) {
      if (status && atomicCAS(status + 1, 0, epoch_a + 1) == 0) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
        status[2] = threadIdx.x;
        status[3] = seen;
      }
    }
  }
}

__global__ void tp_epoch_advance_kernel(int* epoch_base, int by) {
  pdl_entry();
  if (threadIdx.x == 0 && blockIdx.x == 0) *epoch_base += by;
}

}  // namespace apb

extern "C" {

// part_ptrs[world]: every rank's [world * rows_local, H] fp32 partial of THIS call (read, never written here);
// clear_buf / clear_elems: this rank's partial buffer of the previous call, zeroed here for its next use (null / 0:
// nothing to clear; clear_elems % 4 == 0).  resid [rows_local, H] bf16 in/out (has_resid = 0: the sum alone is the new
// residual), w [H] bf16, out_ptrs[world]: every rank's [world * rows_local, H] bf16 activation buffer.  epoch_base:
// device int; the kernel consumes epochs *epoch_base + epoch_off and + 1.  done_counter: device int, zero between
// launches.  H % 8 == 0, H <= 8192.
int apb_tp_norm_allgather(void* const* flag_ptrs, int rank, int world, const int* epoch_base, int epoch_off,
                          void* const* part_ptrs, float* clear_buf, long long clear_elems, void* resid, int has_resid,
                          const void* w, float eps, void* const* out_ptrs, int rows_local, int H, int* done_counter,
                          cudaStream_t s) {
  using namespace apb;
  if (rows_local <= 0) return 0;
  if (world < 1 || world > kMaxRanks || (H % 8) || H > kTpNormThreads * 8 * 4 || !flag_ptrs || !epoch_base ||
      !part_ptrs || !resid || !w || !out_ptrs || !done_counter || (clear_elems % 4) || clear_elems < 0 ||
      (clear_buf && (reinterpret_cast<uintptr_t>(clear_buf) & 15)))
    return kBadArgument;
  PeerPtrs f, o, pp;
  for (int i = 0; i < kMaxRanks; ++i) {
    f.p[i] = i < world ? flag_ptrs[i] : nullptr;
    o.p[i] = i < world ? out_ptrs[i] : nullptr;
    pp.p[i] = i < world ? part_ptrs[i] : nullptr;
    if (i < world && (!f.p[i] || !o.p[i] || !pp.p[i])) return kBadArgument;
  }
  return static_cast<int>(launch_kernel(tp_norm_allgather_kernel, dim3(rows_local), dim3(kTpNormThreads), 0, s, f, rank,
                                        world, epoch_base, epoch_off, pp, reinterpret_cast<float4*>(clear_buf),
                                        clear_buf ? clear_elems / 4 : 0, static_cast<__nv_bfloat16*>(resid), has_resid,
                                        static_cast<const __nv_bfloat16*>(w), eps, o, rows_local, H, done_counter,
                                        status_device_ptr()));
}

int apb_tp_epoch_advance(int* epoch_base, int by, cudaStream_t s) {
  using namespace apb;
  if (!epoch_base) return kBadArgument;
  return static_cast<int>(launch_kernel(tp_epoch_advance_kernel, dim3(1), dim3(32), 0, s, epoch_base, by));
}
}
