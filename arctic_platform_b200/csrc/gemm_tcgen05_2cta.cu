// bf16 GEMM on CTA pairs: two SMs work on one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Why a pair.  With one CTA per 128 x 256 tile every MMA of 128 x 256 x 16 reads 4 KB of A and 8 KB of B
// from shared memory while TMA writes the same amount, which saturates the SM's shared-memory port at about
// three quarters of the tensor-core rate.  In a pair each CTA stages its own 128 rows of A and only HALF of
// the B tile (128 of the 256 columns); the instruction issued by the leader CTA multiplies the 256 x 16 A
// slab spread over both SMs with the 256 x 16 B slab spread over both SMs, so each SM reads 8 KB per
// 128 cycles instead of 12 KB and the tensor cores stay fed.
//
// Layout of the protocol (cluster of 2 CTAs, rank 0 = leader):
//   warp 0   TMA producer of ITS CTA: A rows [m0 + 128*rank, +128), B rows [n0 + 128*rank, +128) per k-block.
//            Loads are plain per-CTA copies (no multicast qualifier); the peer's copies signal the LEADER's
//            "full" barrier (cp.async.bulk.tensor ... cta_group::2), which expects the bytes of both CTAs.
//   warp 1   leader only: issues the MMAs, then commits to the "empty" barrier of the stage in BOTH CTAs and,
//            at the end of a tile, to the "accumulator full" barrier in both CTAs.  Owns the TMEM allocation
//            (both CTAs execute the paired alloc / dealloc).
//   warps 2-5 epilogue of ITS CTA: its 128 accumulator rows (TMEM lanes) x 256 columns -> registers -> global;
//            releases the accumulator buffer by arriving on the leader's barrier (8 arrivals: 4 warps x 2 CTAs).
// Two accumulator buffers (2 x 256 TMEM columns) overlap the epilogue of tile i with the main loop of tile i+1.
// Every mbarrier wait is bounded; a CTA whose wait runs out records a status code and unwinds, its partner's
// waits then run out as well, and both meet at the cluster barrier before TMEM is released.
//
// Stands in for the cuBLAS GEMMs behind every nn.Linear of the reference
// (arctic_platform/model/patches/liger.py:25-36 keeps them on cuBLAS).
#include "common.cuh"
#include "gemm_common.cuh"
#include "host_utils.cuh"

namespace apb {

constexpr int kPairBK = 64;
constexpr int kPairStages = 6;
constexpr int kPairABytes = 128 * kPairBK * 2;   // this CTA's 128 rows of A
constexpr int kPairBBytes = 128 * kPairBK * 2;   // this CTA's 128 of the tile's 256 columns of B
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr int kPairThreads = 192;
constexpr int kPairTmemCols = 512;               // two fp32 accumulators of 256 columns

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local_shared_addr` in the shared memory of CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_shared_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_shared_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Per-CTA tiled load whose completion bytes are counted on a barrier that may live in the partner CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on one mbarrier (cluster address: this CTA's or the partner's) once every MMA issued so far is done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__global__ void __launch_bounds__(kPairThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* empty_bar = full_bar + kPairStages;
  uint64_t* tfull_bar = empty_bar + kPairStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_cta_rank();      // 0 = leader
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 255) / 256;
  const int tiles_n = (p.N + 255) / 256;
  const int mn_tiles = tiles_m * tiles_n;
  const int total_tiles = mn_tiles * p.splits;   // work units: output tiles x K splits (split-K adds into C)
  const int k_blocks = (p.K + kPairBK - 1) / kPairBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);    // the leader's arrive.expect_tx; bytes come from both CTAs
      mbar_init(&empty_bar[s], 1);   // one commit by the leader's MMA thread
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);   // one commit by the leader's MMA thread
      mbar_init(&tempty_bar[b], 8);  // 4 epilogue warps of each CTA (used in the leader only)
    }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, kPairTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                // both CTAs' barriers are initialised before anybody signals the partner
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // Tile order: 8 m-tiles of one n-band at a time, so pairs running together share B in L2.
  auto decode = [&](int unit, int& m0, int& n0, int& kb0, int& kb1) {
    const int split = unit / mn_tiles;
    const int t = unit - split * mn_tiles;
    kb0 = static_cast<int>((static_cast<long long>(k_blocks) * split) / p.splits);
    kb1 = static_cast<int>((static_cast<long long>(k_blocks) * (split + 1)) / p.splits);
    constexpr int G = 8;
    const int per_group = G * tiles_n;
    const int g = t / per_group;
    const int first_m = g * G;
    const int gsize = min(tiles_m - first_m, G);
    const int r = t - g * per_group;
    m0 = (first_m + r % gsize) * 256;
    n0 = (r / gsize) * 256;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += num_pairs) {
        int m0, n0, kb0, kb1;
        decode(t, m0, n0, kb0, kb1);
        const int my_m = m0 + static_cast<int>(cta) * 128;
        const int my_n = n0 + static_cast<int>(cta) * 128;
        // All tiles walk K in the same order: pairs that share a row or a column of tiles in one wave then hit the
        // same operand tiles close together in time, which is what keeps them in L2 (starting every tile at a
        // different k-block was measured: it helps short K and costs up to 10 % at K >= 9728).
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kPairABytes;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tma_a, bar, kb * kPairBK, my_m);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sa + c * (64 * kPairBK * 2), &tma_a, bar, my_m + c * 64, kb * kPairBK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tma_b, bar, kb * kPairBK, my_n);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_2d_pair(sb + c * (64 * kPairBK * 2), &tma_b, bar, my_n + c * 64, kb * kPairBK);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give copies already issued time to land before shared memory is released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(256, 256, p.a_mn, p.b_mn);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
        int m0, n0, kb0, kb1;
        decode(t, m0, n0, kb0, kb1);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1, p.status, kTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * 256;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kPairStageBytes);
          const uint32_t sb = sa + kPairABytes;
#pragma unroll
          for (int k = 0; k < kPairBK / 16; ++k) {
            const uint64_t da = p.a_mn ? umma_smem_desc(sa + k * 2048, 64 * kPairBK * 2, 1024)
                                       : umma_smem_desc(sa + k * 32, 0, 1024);
            const uint64_t db = p.b_mn ? umma_smem_desc(sb + k * 2048, 64 * kPairBK * 2, 1024)
                                       : umma_smem_desc(sb + k * 32, 0, 1024);
            umma_bf16_ss_pair(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          tc_commit_pair(eb);
          tc_commit_pair(map_to_cta(eb, 1));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t tb = smem_u32(&tfull_bar[buf]);
          tc_commit_pair(tb);
          tc_commit_pair(map_to_cta(tb, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    int it = 0;
    bool ok = true;
    for (int t = pair; t < total_tiles && ok; t += num_pairs, ++it) {
      int m0, n0, kb0, kb1;
      decode(t, m0, n0, kb0, kb1);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tfull_bar[buf], acc_phase, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + static_cast<int>(cta) * 128 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * 256;
#pragma unroll 1
      for (int c = 0; c < 256 / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        gemm_store_chunk(p, row, col0, r);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[buf]), 0));
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nobody's shared memory or TMEM is still a target of the partner
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
}

}  // namespace apb

extern "C" {

// D[M,N] = alpha * op(A) * op(B)^T with the CTA-pair kernel.  Same operand conventions as apb_gemm_bf16
// (a_mn / b_mn, leading dimensions multiples of 8, 16-byte aligned bases).  Epilogues: bf16 (+bias), f32,
// f32 accumulate (split along K by the kernel's own choice when that fills the last wave), SwiGLU.  No tile table.  Returns kBadArgument for anything else so that the caller
// can fall back to the one-CTA kernel.
int apb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int a_mn, int b_mn, int epi, float alpha, const void* bias, void* C2,
                       long long ldc2, cudaStream_t stream) {
  using namespace apb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (epi != kEpiBf16 && epi != kEpiF32 && epi != kEpiF32Accum && epi != kEpiSwiGLU) return kBadArgument;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return kBadArgument;
  if (epi == kEpiBf16 || epi == kEpiSwiGLU) {
    if (C && (ldc % 8)) return kBadArgument;
    if (epi == kEpiBf16 && !C) return kBadArgument;
  } else if (!C || (ldc % 4)) {
    return kBadArgument;
  }
  if (epi == kEpiSwiGLU && (!C2 || (ldc2 % 8) || (N % 16))) return kBadArgument;

  CUtensorMap ta, tb;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&ta, A, 2, static_cast<uint64_t>(M), static_cast<uint64_t>(K), lda, 64, 128);
  else
    rc = make_tmap_2d(&ta, A, 2, static_cast<uint64_t>(K), static_cast<uint64_t>(M), lda, 64, 64);
  if (rc) return 1000 + rc;
  if (!b_mn)
    rc = make_tmap_2d(&tb, B, 2, static_cast<uint64_t>(N), static_cast<uint64_t>(K), ldb, 64, 128);
  else
    rc = make_tmap_2d(&tb, B, 2, static_cast<uint64_t>(K), static_cast<uint64_t>(N), ldb, 64, 64);
  if (rc) return 2000 + rc;

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.epi = epi;
  p.splits = 1;
  p.C = C;
  // Accumulating products (weight gradients: few output tiles, very long K) whose tile count leaves much of the
  // last wave of pairs idle are cut along K; the parts add into C with red.add, which is what "+=" asks for.
  if (epi == kEpiF32Accum) {
    const int k_blocks = (K + kPairBK - 1) / kPairBK;
    const long long tiles = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256);
    const int pairs_hint = sm_count() / 2;
    auto wave_eff = [&](int s) {
      const long long units = tiles * s;
      const long long waves = (units + pairs_hint - 1) / pairs_hint;
      return static_cast<double>(units) / static_cast<double>(waves * pairs_hint);
    };
    int best = 1;
    double best_eff = wave_eff(1);
    for (int s = 2; s <= 4; ++s) {
      if (k_blocks / s < 32) break;
      const double e = wave_eff(s);
      if (e > best_eff + 0.04) {
        best = s;
        best_eff = e;
      }
    }
    if (best > 1) {
      p.splits = best;
      p.epi = kEpiF32Atomic;
    }
  }
  p.ldc = ldc;
  p.C2 = C2;
  p.ldc2 = ldc2;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha;
  p.status = status_device_ptr();

  // How many pairs can be resident at once (SMs of a pair must sit in one cluster-capable group, so this can be
  // fewer than half the SM count).  The grid never exceeds it: a pair that had to wait for a second wave would
  // still take a full share of the tiles.
  static int resident_pairs[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!resident_pairs[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel, &cfg);
    if (e != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2 - 4;        // conservative when the query is unavailable
    }
    resident_pairs[dev & 63] = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const long long total = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) * p.splits;
  const int max_pairs = resident_pairs[dev & 63];
  const int pairs = static_cast<int>(total < max_pairs ? total : max_pairs);
  cfg.gridDim = dim3(2 * pairs);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel, ta, tb, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaGetLastError());
}
}
