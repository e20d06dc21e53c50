// Gradient reduce-scatter + clip + partitioned AdamW + parameter all-gather, as
// two kernels that talk to the other GPUs through peer-mapped (symmetric) buffers
// over NVLink instead of calling a collective library:
//
//   phase A  zero_reduce_kernel : this rank's shard of the fp32 gradient bucket is
//            summed over every rank's bucket with P2P loads (or one
//            multimem.ld_reduce through the switch when a multicast mapping is
//            given), scaled, written to the local reduced shard, and its sum of
//            squares is accumulated for the global gradient norm.
//   phase B  zero_adamw_kernel  : AdamW on the fp32 master shard with the clip
//            coefficient derived on the device from the global sum of squares,
//            then the updated bf16 values are stored into EVERY rank's parameter
//            buffer (P2P stores or multimem.st), which is the all-gather.
//
// With one rank both kernels degenerate to a fused local cast/clip/AdamW.  The
// reference leaves these steps to DeepSpeed's ZeRO reduce-scatter, its
// multi-tensor FusedAdam and a parameter all-gather
// (arctic_platform/common/deepspeed_worker.py:208-300).
//
// Cross-rank ordering uses epoch flags in symmetric memory: a kernel first
// announces its epoch to every peer and waits (bounded) until all peers have
// announced theirs, i.e. their earlier work on the stream -- the writes this kernel
// is about to read -- has completed.
#include "common.cuh"
#include "host_utils.cuh"
#include "peer.cuh"
#include <string.h>

namespace apb {

// grads: per-rank base pointers of the fp32 bucket (symmetric layout); this rank owns
// elements [shard_off, shard_off + n).  n % 4 == 0.
__global__ void __launch_bounds__(256)
zero_reduce_kernel(PeerPtrs grads, const float* mc_grads, PeerPtrs flags, int rank, int world, int epoch,
                   long long shard_off, long long n, float scale, float* __restrict__ reduced,
                   double* __restrict__ sumsq, int* status) {
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  double acc = 0.0;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 s;
    if (mc_grads) {
      s = multimem_ld_reduce_f32x4(mc_grads + shard_off + i * 4);
    } else {
      s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const int src = (rank + r) % world;  // start at the local copy, spread peers over links
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[src]) + shard_off + i * 4);
        s.x += v.x;
        s.y += v.y;
        s.z += v.z;
        s.w += v.w;
      }
    }
    s.x *= scale;
    s.y *= scale;
    s.z *= scale;
    s.w *= scale;
    *reinterpret_cast<float4*>(reduced + i * 4) = s;
    acc += static_cast<double>(s.x) * s.x + static_cast<double>(s.y) * s.y + static_cast<double>(s.z) * s.z +
           static_cast<double>(s.w) * s.w;
  }
  // block reduction of the sum of squares
  __shared__ double red[8];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < blockDim.x / 32; ++w) t += red[w];
    atomicAdd(sumsq, t);
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias1, bias2;       // 1 - beta^t
  float max_grad_norm;      // <= 0 : no clipping
};

// params: per-rank base pointers of the bf16 parameter bucket; every rank receives the
// updated values of this rank's shard [shard_off, shard_off + n).  n % 8 == 0.
__global__ void __launch_bounds__(256)
zero_adamw_kernel(PeerPtrs params, void* mc_params, PeerPtrs flags, int rank, int world, int epoch,
                  long long shard_off, long long n, const float* __restrict__ grad, float* __restrict__ master,
                  float* __restrict__ m, float* __restrict__ v, const double* __restrict__ total_sumsq,
                  AdamArgs a, int* status) {
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  float clip = 1.f;
  if (a.max_grad_norm > 0.f && total_sumsq) {
    const float nrm = static_cast<float>(sqrt(*total_sumsq));
    clip = fminf(1.f, a.max_grad_norm / (nrm + 1e-6f));
  }
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float out[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long e = i * 8 + h * 4;
      float4 g = *reinterpret_cast<const float4*>(grad + e);
      float4 w = *reinterpret_cast<const float4*>(master + e);
      float4 mm = *reinterpret_cast<const float4*>(m + e);
      float4 vv = *reinterpret_cast<const float4*>(v + e);
      float* gp = &g.x;
      float* wp = &w.x;
      float* mp = &mm.x;
      float* vp = &vv.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gp[j] * clip;
        mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
        vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
        const float mh = mp[j] / a.bias1;
        const float vh = vp[j] / a.bias2;
        wp[j] = wp[j] * (1.f - a.lr * a.weight_decay) - a.lr * mh / (sqrtf(vh) + a.eps);
        out[h * 4 + j] = wp[j];
      }
      *reinterpret_cast<float4*>(master + e) = w;
      *reinterpret_cast<float4*>(m + e) = mm;
      *reinterpret_cast<float4*>(v + e) = vv;
    }
    uint4 o;
    o.x = pack_bf16x2(out[0], out[1]);
    o.y = pack_bf16x2(out[2], out[3]);
    o.z = pack_bf16x2(out[4], out[5]);
    o.w = pack_bf16x2(out[6], out[7]);
    const long long e = shard_off + i * 8;
    if (mc_params) {
      multimem_st_b128(static_cast<__nv_bfloat16*>(mc_params) + e, o);
    } else {
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[dst]) + e) = o;
      }
    }
  }
}

// Waits until every peer has announced `epoch` (completion of the peers' stores into
// this rank's buffers before dependent work starts).
__global__ void epoch_wait_kernel(PeerPtrs flags, int rank, int world, int epoch, int* status) {
  epoch_barrier(flags, rank, world, epoch, status);
}

// All-gather of bf16 shards by pulling: dst[r*n .. ] = peer r's shard (n elements, n % 8 == 0).
__global__ void __launch_bounds__(256)
gather_shards_kernel(PeerPtrs shards, PeerPtrs flags, int rank, int world, int epoch, long long n,
                     __nv_bfloat16* __restrict__ dst, int* status) {
  // epoch <= 0: the caller guarantees the shards are final (they only change at optimizer steps)
  if (epoch > 0 && !epoch_barrier(flags, rank, world, epoch, status)) return;
  const long long n8 = n >> 3;
  const long long total = n8 * world;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int rr = static_cast<int>(i / n8);
    const int src = (rank + rr) % world;
    const long long off = (i - static_cast<long long>(rr) * n8) * 8;
    const uint4 val = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(shards.p[src]) + off);
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(src) * n + off) = val;
  }
}

// ZeRO-3 unit gather: every parameter of a unit is stored as `world` equal pieces, piece r in rank r's shard buffer.
// One launch rebuilds the whole unit in parameter-major layout by pulling the pieces from their owners (plain peer
// loads).  The grid is capped so the copy shares the GPU with the GEMMs of the unit that is computing meanwhile.
constexpr int kMaxGatherPieces = 24;
struct GatherTable {
  long long full_off[kMaxGatherPieces];   // element offset of the parameter inside the unit (destination)
  long long piece_len[kMaxGatherPieces];  // elements per rank, multiple of 8
  long long shard_off[kMaxGatherPieces];  // element offset of the piece inside the unit's part of a shard buffer
  long long vec_start[kMaxGatherPieces + 1];  // running count of 16-byte vectors (all ranks) before each parameter
  int n;
};

__global__ void __launch_bounds__(256)
gather_unit_kernel(PeerPtrs shards, GatherTable t, int rank, int world, __nv_bfloat16* __restrict__ dst) {
  const long long total = t.vec_start[t.n];
  // A peer load over NVLink takes microseconds: every thread keeps kUnroll 16-byte loads in flight so that the
  // capped grid still covers the bandwidth-delay product of the link.
  constexpr int kUnroll = 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * kUnroll) {
    uint4 val[kUnroll];
    __nv_bfloat16* out[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = i0 + u * stride;
      out[u] = nullptr;
      if (i < total) {
        int pc = 0;
        while (pc + 1 < t.n && i >= t.vec_start[pc + 1]) ++pc;
        const long long j = i - t.vec_start[pc];
        const long long n8 = t.piece_len[pc] >> 3;
        const int rr = static_cast<int>(j / n8);
        const int src = (rank + rr) % world;  // start with the local piece, then walk the peers
        const long long off = (j - static_cast<long long>(rr) * n8) * 8;
        val[u] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(shards.p[src]) + t.shard_off[pc] + off);
        out[u] = dst + t.full_off[pc] + static_cast<long long>(src) * t.piece_len[pc] + off;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (out[u]) *reinterpret_cast<uint4*>(out[u]) = val[u];
  }
}

// ZeRO-3 reduce-scatter of one unit: for every parameter, this rank's piece of the fp32 gradient is summed over all
// ranks' gradient buffers (P2P loads), scaled and written to the shard-layout buffer; the sum of squares feeds the
// global gradient norm.  Table fields: full_off = element offset of THIS rank's piece inside the unit's gradients,
// shard_off = destination offset, vec_start counts float4 groups.  One flag barrier per launch.
__global__ void __launch_bounds__(256)
zero3_reduce_unit_kernel(PeerPtrs grads, GatherTable t, PeerPtrs flags, int rank, int world, int epoch, float scale,
                         float* __restrict__ reduced, double* __restrict__ sumsq, int accumulate, int* status) {
  // accumulate = 1 (gradients reduced unit by unit DURING the backward pass): the sums are ADDED to this rank's
  // shard accumulator and every source range is cleared after it has been read (each element is read by exactly one
  // rank, its owner), so the staging slot is zero on all ranks when the kernel has ended everywhere; the squares
  // for the gradient norm are then taken from the accumulator at the optimizer step.
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  const long long total = t.vec_start[t.n];
  double acc = 0.0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    int pc = 0;
    while (pc + 1 < t.n && i >= t.vec_start[pc + 1]) ++pc;
    const long long off = (i - t.vec_start[pc]) * 4;
    float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const int src = (rank + r) % world;
      float4* sp = reinterpret_cast<float4*>(static_cast<float*>(grads.p[src]) + t.full_off[pc] + off);
      const float4 v = *sp;
      if (accumulate) *sp = make_float4(0.f, 0.f, 0.f, 0.f);
      s4.x += v.x;
      s4.y += v.y;
      s4.z += v.z;
      s4.w += v.w;
    }
    s4.x *= scale;
    s4.y *= scale;
    s4.z *= scale;
    s4.w *= scale;
    float4* dst = reinterpret_cast<float4*>(reduced + t.shard_off[pc] + off);
    if (accumulate) {
      const float4 old = *dst;
      s4.x += old.x;
      s4.y += old.y;
      s4.z += old.z;
      s4.w += old.w;
    }
    *dst = s4;
    acc += static_cast<double>(s4.x) * s4.x + static_cast<double>(s4.y) * s4.y + static_cast<double>(s4.z) * s4.z +
           static_cast<double>(s4.w) * s4.w;
  }
  __shared__ double red[8];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && !accumulate && sumsq) {
    double tt = 0.0;
    for (int w = 0; w < blockDim.x / 32; ++w) tt += red[w];
    atomicAdd(sumsq, tt);
  }
}

__global__ void sumsq_f32_kernel(const float* __restrict__ x, long long n, double* __restrict__ out) {
  double acc = 0.0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    acc += static_cast<double>(x[i]) * x[i];
  __shared__ double red[8];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < blockDim.x / 32; ++w) t += red[w];
    atomicAdd(out, t);
  }
}

}  // namespace apb

extern "C" {
using namespace apb;

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < kMaxRanks; ++i) p.p[i] = i < world ? ptrs[i] : nullptr;
  return p;
}
static int grid_for(long long work_items) {
  long long g = (work_items + 255) / 256;
  if (g < 1) g = 1;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(g < cap ? g : cap);
}

// Phase A.  grad_ptrs[world]: every rank's fp32 bucket base (peer-mapped); flag_ptrs[world]: every rank's
// int flag array (>= world ints).  mc_grads: multicast address of the bucket or null.
int apb_zero_reduce(void* const* grad_ptrs, const float* mc_grads, void* const* flag_ptrs, int rank, int world,
                    int epoch, long long shard_off, long long n, float scale, float* reduced, double* sumsq,
                    cudaStream_t s) {
  if (world < 1 || world > kMaxRanks || (n % 4) || (shard_off % 4)) return kBadArgument;
  if (n == 0 && world <= 1) return 0;
  // an engine whose state was moved to the host hands out null (empty-tensor) addresses: refuse them here
  if (!grad_ptrs || !reduced || !sumsq || (world > 1 && !flag_ptrs)) return kBadArgument;
  for (int i = 0; i < world; ++i)
    if (!grad_ptrs[i] || (world > 1 && !flag_ptrs[i])) return kBadArgument;
  zero_reduce_kernel<<<grid_for(n / 4), 256, 0, s>>>(to_peers(grad_ptrs, world), mc_grads, to_peers(flag_ptrs, world),
                                                     rank, world, epoch, shard_off, n, scale, reduced, sumsq,
                                                     status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

// Phase B.  param_ptrs[world]: every rank's bf16 parameter bucket base; mc_params: multicast address or null.
int apb_zero_adamw(void* const* param_ptrs, void* mc_params, void* const* flag_ptrs, int rank, int world, int epoch,
                   long long shard_off, long long n, const float* grad, float* master, float* m, float* v,
                   const double* total_sumsq, float lr, float beta1, float beta2, float eps, float weight_decay,
                   float bias1, float bias2, float max_grad_norm, cudaStream_t s) {
  if (world < 1 || world > kMaxRanks || (n % 8) || (shard_off % 8)) return kBadArgument;
  if (n == 0 && world <= 1) return 0;
  if (!param_ptrs || !grad || !master || !m || !v || !total_sumsq || (world > 1 && !flag_ptrs)) return kBadArgument;
  for (int i = 0; i < world; ++i)
    if (!param_ptrs[i] || (world > 1 && !flag_ptrs[i])) return kBadArgument;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias1, bias2, max_grad_norm};
  zero_adamw_kernel<<<grid_for(n / 8), 256, 0, s>>>(to_peers(param_ptrs, world), mc_params,
                                                    to_peers(flag_ptrs, world), rank, world, epoch, shard_off, n, grad,
                                                    master, m, v, total_sumsq, a, status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

int apb_epoch_wait(void* const* flag_ptrs, int rank, int world, int epoch, cudaStream_t s) {
  if (world > kMaxRanks) return kBadArgument;
  if (world <= 1) return 0;
  epoch_wait_kernel<<<1, 32, 0, s>>>(to_peers(flag_ptrs, world), rank, world, epoch, status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

int apb_gather_shards(void* const* shard_ptrs, void* const* flag_ptrs, int rank, int world, int epoch, long long n,
                      void* dst, cudaStream_t s) {
  if (world > kMaxRanks || (n % 8)) return kBadArgument;
  gather_shards_kernel<<<grid_for(n / 8 * world), 256, 0, s>>>(to_peers(shard_ptrs, world), to_peers(flag_ptrs, world),
                                                               rank, world, epoch, n,
                                                               static_cast<__nv_bfloat16*>(dst), status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

// shard_ptrs: per-rank pointers to the unit's part of the shard buffers.  full_off / piece_len / shard_off: host
// arrays of n_pieces entries (elements).  max_ctas caps the grid (0 = 64).
int apb_gather_unit(void* const* shard_ptrs, int rank, int world, const long long* full_off, const long long* piece_len,
                    const long long* shard_off, int n_pieces, void* dst, int max_ctas, cudaStream_t s) {
  if (world > kMaxRanks || n_pieces < 1 || n_pieces > kMaxGatherPieces) return kBadArgument;
  GatherTable t;
  t.n = n_pieces;
  long long acc = 0;
  for (int i = 0; i < n_pieces; ++i) {
    if (piece_len[i] % 8 || full_off[i] % 8 || shard_off[i] % 8) return kBadArgument;
    t.full_off[i] = full_off[i];
    t.piece_len[i] = piece_len[i];
    t.shard_off[i] = shard_off[i];
    t.vec_start[i] = acc;
    acc += piece_len[i] / 8 * world;
  }
  t.vec_start[n_pieces] = acc;
  if (acc == 0) return 0;
  const int cap = max_ctas > 0 ? max_ctas : 64;
  const long long need = (acc + 255) / 256;
  gather_unit_kernel<<<static_cast<int>(need < cap ? need : cap), 256, 0, s>>>(to_peers(shard_ptrs, world), t, rank, world,
                                                                              static_cast<__nv_bfloat16*>(dst));
  return static_cast<int>(cudaGetLastError());
}

// grad_ptrs: per-rank pointers to the unit's part of the fp32 gradient buffers.  src_off[i]: element offset of this
// rank's piece of parameter i inside the unit; piece_len[i] (multiple of 4); dst_off[i]: offset inside `reduced`.
int apb_zero3_reduce_unit(void* const* grad_ptrs, void* const* flag_ptrs, int rank, int world, int epoch,
                          const long long* src_off, const long long* piece_len, const long long* dst_off, int n_pieces,
                          float scale, float* reduced, double* sumsq, int accumulate, cudaStream_t s) {
  if (world > kMaxRanks || n_pieces < 1 || n_pieces > kMaxGatherPieces) return kBadArgument;
  GatherTable t;
  t.n = n_pieces;
  long long acc = 0;
  for (int i = 0; i < n_pieces; ++i) {
    if (piece_len[i] % 4 || src_off[i] % 4 || dst_off[i] % 4) return kBadArgument;
    t.full_off[i] = src_off[i];
    t.piece_len[i] = piece_len[i];
    t.shard_off[i] = dst_off[i];
    t.vec_start[i] = acc;
    acc += piece_len[i] / 4;
  }
  t.vec_start[n_pieces] = acc;
  zero3_reduce_unit_kernel<<<grid_for(acc > 0 ? acc : 1), 256, 0, s>>>(to_peers(grad_ptrs, world), t,
                                                                       to_peers(flag_ptrs, world), rank, world, epoch,
                                                                       scale, reduced, sumsq, accumulate,
                                                                       status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

int apb_sumsq_f32(const float* x, long long n, double* out, cudaStream_t s) {
  if (n <= 0) return 0;
  sumsq_f32_kernel<<<grid_for(n), 256, 0, s>>>(x, n, out);
  return static_cast<int>(cudaGetLastError());
}
}

// ---------------------------------------------------------------------------
// Trainer -> sampler weight synchronisation
// ---------------------------------------------------------------------------
namespace apb {

struct SyncUnits {
  // up to 160 units (embedding, one per block, final norm); offsets/lengths in elements
  long long offset[160];
  long long length[160];
  int n;
};

// dst[e] = source element e of the flat parameter space, read from the rank that owns it.
//   sharded = 0: every rank holds the whole flat buffer (src.p[rank] is read);
//   sharded = 1: rank r holds, for every unit u, elements [r*len_u/W, (r+1)*len_u/W) packed back to back
//                (the ZeRO shard layout); the owner is computed per element and read through its peer mapping.
// One pass, 16 bytes per thread per iteration; this is the whole "gather ZeRO shards + reshard to the
// sampler layout" step when both sides use the same fused layout.
__global__ void __launch_bounds__(256)
sync_weights_flat_kernel(PeerPtrs src, PeerPtrs flags, int rank, int world, int epoch, int sharded, SyncUnits units,
                         __nv_bfloat16* __restrict__ dst, long long total, int* status) {
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  const long long n8 = total >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i * 8;
    const __nv_bfloat16* sp;
    if (!sharded) {
      sp = static_cast<const __nv_bfloat16*>(src.p[rank]) + e;
    } else {
      int u = 0;
      long long shard_base = 0;  // start of unit u inside a rank's packed shard buffer
      while (u + 1 < units.n && e >= units.offset[u + 1]) {
        shard_base += units.length[u] / world;
        ++u;
      }
      const long long per = units.length[u] / world;
      const long long in_unit = e - units.offset[u];
      const int owner = static_cast<int>(in_unit / per);
      sp = static_cast<const __nv_bfloat16*>(src.p[owner]) + shard_base + (in_unit - owner * per);
    }
    *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(sp);
  }
}

// Block-scaled fp8 (e4m3) requantisation of a [rows, cols] bf16 weight with one fp32 scale per
// 128 x 128 block: scale = amax / 448, q = w / scale.  One CTA per block.
__global__ void __launch_bounds__(256)
quant_fp8_block128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw, int rows, int cols,
                          uint8_t* __restrict__ q, long long ldq, float* __restrict__ scales, int scale_ld) {
  const int bx = blockIdx.x, by = blockIdx.y;
  const int r0 = by * 128, c0 = bx * 128;
  __shared__ float red[8];
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 16; i += 256) {
    const int r = r0 + i / 16, c = c0 + (i % 16) * 8;
    if (r < rows && c < cols) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + r * ldw + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h2[k]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) amax = fmaxf(amax, red[k]);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  if (threadIdx.x == 0) scales[by * scale_ld + bx] = scale;
  for (int i = threadIdx.x; i < 128 * 16; i += 256) {
    const int r = r0 + i / 16, c = c0 + (i % 16) * 8;
    if (r < rows && c < cols) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + r * ldw + c);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      uint32_t out[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float2 a = __bfloat1622float2(h2[2 * k]);
        const float2 b = __bfloat1622float2(h2[2 * k + 1]);
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(a.y * inv), "f"(a.x * inv));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(b.y * inv), "f"(b.x * inv));
        out[k] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      *reinterpret_cast<uint2*>(q + r * ldq + c) = make_uint2(out[0], out[1]);
    }
  }
}

}  // namespace apb

extern "C" {

// src_ptrs[world]: per-rank source base pointers (full flat buffer if sharded == 0, packed ZeRO shards if 1).
// unit_offset / unit_length: n_units entries describing the flat parameter space (elements).
int apb_sync_weights_flat(void* const* src_ptrs, void* const* flag_ptrs, int rank, int world, int epoch, int sharded,
                          const long long* unit_offset, const long long* unit_length, int n_units, void* dst,
                          long long total, cudaStream_t s) {
  using namespace apb;
  if (world > kMaxRanks || n_units > 160 || (total % 8)) return kBadArgument;
  SyncUnits u;
  u.n = n_units;
  for (int i = 0; i < n_units; ++i) {
    u.offset[i] = unit_offset[i];
    u.length[i] = unit_length[i];
    if (sharded && (unit_length[i] % (8LL * world))) return kBadArgument;
  }
  sync_weights_flat_kernel<<<grid_for(total / 8), 256, 0, s>>>(to_peers(src_ptrs, world), to_peers(flag_ptrs, world),
                                                              rank, world, epoch, sharded, u,
                                                              static_cast<__nv_bfloat16*>(dst), total,
                                                              status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

// w [rows, cols] bf16 -> q [rows, cols] e4m3 + scales [ceil(rows/128), ceil(cols/128)] fp32.  cols % 8 == 0.
int apb_quant_fp8_block128(const void* w, long long ldw, int rows, int cols, void* q, long long ldq, float* scales,
                           cudaStream_t s) {
  using namespace apb;
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols % 8) || (ldw % 8) || (ldq % 8)) return kBadArgument;
  const dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  quant_fp8_block128_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(w), ldw, rows, cols,
                                                 static_cast<uint8_t*>(q), ldq, scales, (cols + 127) / 128);
  return static_cast<int>(cudaGetLastError());
}
}

// ---------------------------------------------------------------------------
// Table-driven weight synchronisation: gather + tensor-parallel reshard + cast / fp8 requantisation in one pass
// ---------------------------------------------------------------------------
namespace apb {

// One rectangular slice of one trainer parameter and where it goes in the sampler.  The source parameter is a
// row-major matrix (src_ld elements per row; a vector is one row) that lives at element `src_elem` of the full
// parameter-major flat space; when `piece_len` > 0 the trainer keeps it ZeRO-3 sharded -- cut into equal flat
// pieces, piece r on rank r at `shard_off` of that rank's shard buffer -- and every 16-byte vector is read from
// the rank that owns it.  The slice [row0, row0 + rows) x [col0, col0 + cols) is written to the destination as a
// dense [rows, dst_ld] matrix: bf16 at `dst_elem` of the bf16 buffer (dst_elem >= 0) and / or e4m3 at `q_off` of
// the fp8 buffer with one fp32 scale per 128 x 128 block of THE SLICE at `scale_off` (fp8 != 0).
struct SyncSeg {
  long long src_elem;
  long long piece_len;
  long long shard_off;
  long long dst_elem;    // < 0: no bf16 copy
  long long q_off;       // fp8 bytes
  long long scale_off;   // floats
  long long tile_start;  // 128 x 128 tiles of all earlier segments
  int src_ld, row0, col0, rows, cols, dst_ld, q_ld, scale_ld;
  int fp8;
  int tiles_c;           // ceil(cols / 128)
};

__device__ __forceinline__ const __nv_bfloat16* sync_src_ptr(const SyncSeg& sg, const PeerPtrs& src, int src_rank,
                                                             long long e_in_param) {
  if (sg.piece_len > 0) {
    const int owner = static_cast<int>(e_in_param / sg.piece_len);
    return static_cast<const __nv_bfloat16*>(src.p[owner]) + sg.shard_off + (e_in_param - owner * sg.piece_len);
  }
  return static_cast<const __nv_bfloat16*>(src.p[src_rank]) + sg.src_elem + e_in_param;
}

// One CTA per 128 x 128 tile of a segment (grid-stride over all tiles of the table).  A tile is read ONCE from the
// source (local memory, or a peer's over NVLink) into registers: 256 threads x 8 vectors of 8 bf16.
__global__ void __launch_bounds__(256)
sync_weights_table_kernel(const SyncSeg* __restrict__ segs, int n_seg, long long total_tiles, long long tile_rot,
                          PeerPtrs src, int src_rank, PeerPtrs flags, int rank, int world, int epoch,
                          __nv_bfloat16* __restrict__ dst_bf16, uint8_t* __restrict__ dst_q,
                          float* __restrict__ dst_scale, int* status) {
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  __shared__ float red[8];
  for (long long t0 = blockIdx.x; t0 < total_tiles; t0 += gridDim.x) {
    // every rank starts its walk at a different tile: the ranks would otherwise all pull the same stretch of a
    // tensor -- one owner's NVLink port -- at the same moment
    long long t = t0 + tile_rot;
    if (t >= total_tiles) t -= total_tiles;
    int lo = 0, hi = n_seg - 1;             // last segment whose tile_start <= t
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (segs[mid].tile_start <= t) lo = mid; else hi = mid - 1;
    }
    const SyncSeg sg = segs[lo];
    const long long lt = t - sg.tile_start;
    const int rb = static_cast<int>(lt / sg.tiles_c), cb = static_cast<int>(lt % sg.tiles_c);
    uint4 v[8];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = threadIdx.x + k * 256;          // vector index inside the tile: 128 rows x 16 vectors
      const int r = rb * 128 + (i >> 4), c = cb * 128 + (i & 15) * 8;
      v[k] = make_uint4(0u, 0u, 0u, 0u);
      if (r < sg.rows && c < sg.cols) {
        const long long e = static_cast<long long>(sg.row0 + r) * sg.src_ld + sg.col0 + c;
        v[k] = *reinterpret_cast<const uint4*>(sync_src_ptr(sg, src, src_rank, e));
        if (sg.dst_elem >= 0)
          *reinterpret_cast<uint4*>(dst_bf16 + sg.dst_elem + static_cast<long long>(r) * sg.dst_ld + c) = v[k];
        if (sg.fp8) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
        }
      }
    }
    if (sg.fp8) {                                   // uniform across the CTA
      amax = warp_max(amax);
      __syncthreads();                              // `red` of the previous tile has been read by everybody
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = red[0];
#pragma unroll
      for (int k = 1; k < 8; ++k) amax = fmaxf(amax, red[k]);
      const float scale = amax > 0.f ? amax / 448.f : 1.f;
      const float inv = 1.f / scale;
      if (threadIdx.x == 0) dst_scale[sg.scale_off + static_cast<long long>(rb) * sg.scale_ld + cb] = scale;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int i = threadIdx.x + k * 256;
        const int r = rb * 128 + (i >> 4), c = cb * 128 + (i & 15) * 8;
        if (r < sg.rows && c < sg.cols) {
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[k]);
          uint32_t out[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float2 a = __bfloat1622float2(h2[2 * j]);
            const float2 b = __bfloat1622float2(h2[2 * j + 1]);
            uint16_t lo16, hi16;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo16) : "f"(a.y * inv), "f"(a.x * inv));
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi16) : "f"(b.y * inv), "f"(b.x * inv));
            out[j] = static_cast<uint32_t>(lo16) | (static_cast<uint32_t>(hi16) << 16);
          }
          *reinterpret_cast<uint2*>(dst_q + sg.q_off + static_cast<long long>(r) * sg.q_ld + c) =
              make_uint2(out[0], out[1]);
        }
      }
    }
  }
}

}  // namespace apb

extern "C" {

// segs: DEVICE array of n_seg apb::SyncSeg records (tile_start filled, ascending); total_tiles = tiles of all
// segments.  src_ptrs[n_src]: the trainer ranks' parameter buffers (full flat buffers, of which src_rank's is read,
// or ZeRO-3 shard buffers, read by ownership) -- peer mappings of this process (symmetric memory or opened IPC
// handles).  flag_ptrs / rank / world / epoch: optional epoch barrier among the ranks that launch this kernel
// together (world <= 1: none).  dst_bf16 / dst_q / dst_scale: this sampler rank's buffers.
int apb_sync_weights_table(const void* segs, int n_seg, long long total_tiles, void* const* src_ptrs, int n_src,
                           int src_rank, void* const* flag_ptrs, int rank, int world, int epoch, void* dst_bf16,
                           void* dst_q, float* dst_scale, int max_ctas, cudaStream_t s) {
  using namespace apb;
  if (n_seg <= 0 || total_tiles <= 0) return 0;
  if (!segs || !src_ptrs || n_src < 1 || n_src > kMaxRanks || src_rank < 0 || src_rank >= n_src ||
      world > kMaxRanks || (world > 1 && !flag_ptrs))
    return kBadArgument;
  for (int i = 0; i < n_src; ++i)
    if (!src_ptrs[i]) return kBadArgument;
  PeerPtrs fl;
  for (int i = 0; i < kMaxRanks; ++i) fl.p[i] = (world > 1 && i < world) ? flag_ptrs[i] : nullptr;
  const long long cap = max_ctas > 0 ? max_ctas : static_cast<long long>(sm_count()) * 8;
  const int grid = static_cast<int>(total_tiles < cap ? total_tiles : cap);
  const long long rot = n_src > 1 ? (total_tiles / n_src) * src_rank : 0;
  sync_weights_table_kernel<<<grid, 256, 0, s>>>(static_cast<const SyncSeg*>(segs), n_seg, total_tiles, rot,
                                                 to_peers(src_ptrs, n_src), src_rank, fl, rank, world > 1 ? world : 1,
                                                 epoch, static_cast<__nv_bfloat16*>(dst_bf16),
                                                 static_cast<uint8_t*>(dst_q), dst_scale, status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}

// Size of one table record, so that the host side can lay the records out without sharing a header.
int apb_sync_seg_bytes() { return static_cast<int>(sizeof(apb::SyncSeg)); }

// ---- device pointers shared between processes (split placement: the sampler's process reads the trainer's
// parameter buffer over NVLink).  `handle` is an opaque 64-byte record to send to the other process.
int apb_ipc_export(const void* ptr, void* handle64, long long* offset_out) {
  if (!ptr || !handle64 || !offset_out) return apb::kBadArgument;
  CUdeviceptr base = 0;
  size_t size = 0;
  // the handle names the allocation; the pointer may sit inside it (a caching allocator's block)
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (!range_fn) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -1;
    range_fn = reinterpret_cast<RangeFn>(fp);
  }
  if (range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return -2;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  *offset_out = static_cast<long long>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return 0;
}

int apb_ipc_open(const void* handle64, long long offset, void** ptr_out) {
  if (!handle64 || !ptr_out) return apb::kBadArgument;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  *ptr_out = static_cast<char*>(base) + offset;
  return 0;
}

int apb_ipc_close(void* ptr, long long offset) {
  if (!ptr) return 0;
  return static_cast<int>(cudaIpcCloseMemHandle(static_cast<char*>(ptr) - offset));
}
}

// ---------------------------------------------------------------------------
// Expert-parallel dispatch / return: rows moved between ranks by P2P stores
// ---------------------------------------------------------------------------
namespace apb {

// For every routed pair e: copy row src[src_row[e]] (H bf16) into dst_ptrs[dst_rank[e]] at row dst_row[e]
// and, when meta_ptrs is given, write (this rank, tag[e]) beside it so the receiver can send the result back.
// One warp per pair.  dst_rank[e] < 0 skips the pair.
__global__ void __launch_bounds__(256)
ep_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, const int* __restrict__ src_row,
                       const int* __restrict__ dst_rank, const int* __restrict__ dst_row, const int* __restrict__ tag,
                       PeerPtrs dst_ptrs, long long ld_dst, PeerPtrs meta_ptrs, int rank, int world, int n_pairs,
                       int H, int* status) {
  const int lane = threadIdx.x & 31;
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nw = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long e = wid; e < n_pairs; e += nw) {
    const int dr = dst_rank[e];
    if (dr < 0) continue;
    if (dr >= world || dst_row[e] < 0) {  // corrupt routing table: record it and skip the store
      if (lane == 0) atomicCAS(status, 0, kBadRouting);
      continue;
    }
    const __nv_bfloat16* s = src + static_cast<long long>(src_row[e]) * ld_src;
    __nv_bfloat16* d = static_cast<__nv_bfloat16*>(dst_ptrs.p[dr]) + static_cast<long long>(dst_row[e]) * ld_dst;
    for (int i = lane * 8; i < H; i += 256) *reinterpret_cast<uint4*>(d + i) = *reinterpret_cast<const uint4*>(s + i);
    if (meta_ptrs.p[dr] != nullptr && lane == 0)
      static_cast<int2*>(meta_ptrs.p[dr])[dst_row[e]] = make_int2(rank, tag ? tag[e] : static_cast<int>(e));
  }
}

}  // namespace apb

extern "C" {

// dst_ptrs / meta_ptrs: per-rank base pointers (meta may be null).  H % 8 == 0.
int apb_ep_scatter_rows(const void* src, long long ld_src, const int* src_row, const int* dst_rank, const int* dst_row,
                        const int* tag, void* const* dst_ptrs, long long ld_dst, void* const* meta_ptrs, int rank,
                        int world, int n_pairs, int H, cudaStream_t s) {
  using namespace apb;
  if (n_pairs <= 0) return 0;
  if (world > kMaxRanks || (H % 8) || (ld_src % 8) || (ld_dst % 8)) return kBadArgument;
  PeerPtrs meta;
  for (int i = 0; i < kMaxRanks; ++i) meta.p[i] = (meta_ptrs && i < world) ? meta_ptrs[i] : nullptr;
  const long long g = (static_cast<long long>(n_pairs) * 32 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  const int grid = static_cast<int>(g < cap ? g : cap);
  ep_scatter_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), ld_src, src_row, dst_rank, dst_row,
                                              tag, to_peers(dst_ptrs, world), ld_dst, meta, rank, world, n_pairs, H,
                                              status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}
}
