// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), operands staged by TMA into a 128-byte-swizzled shared
// memory ring.  One persistent CTA per SM, three warp roles:
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer (one lane), owns the TMEM allocation
//   warps 2..5  epilogue: TMEM -> registers -> global, one accumulator row per thread
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main
// loop of tile i+1.  Every wait is bounded (see common.cuh).
//
// D[M,N] = A[M,K] * B[N,K]^T with either operand optionally "MN-major"
// (A stored as [K,M], B stored as [K,N]); this covers the forward, the
// data-gradient and the weight-gradient products of a linear layer without
// transposes in memory.  Stands in for the cuBLAS GEMMs behind every
// nn.Linear of the reference (arctic_platform/model/patches/liger.py:25-36
// keeps them on cuBLAS).
#include "common.cuh"
#include "gemm_common.cuh"
#include "host_utils.cuh"
#include "peer.cuh"
#include <stdlib.h>

namespace apb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

// ST = 0 picks the deepest ring that fits one CTA per SM; ST = 3 is the "two CTAs per SM" variant for skinny
// (decode) problems whose tile count falls between one and two waves of SMs.
template <int BN, int ST = 0>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // deepest ring that fits: widths 144 and 208 (one wave of SMs for column counts such as 19456 or 151936 that
  // 128- or 256-wide tiles cut into "one wave and a bit") are 16-column multiples between the power-of-two widths
  static constexpr int kStages = ST ? ST : (BN == 256) ? 4 : (BN > 144) ? 5 : (BN > 64) ? 6 : 8;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = BN <= 64 ? 128 : (BN <= 128 ? 256 : 512);   // a power of two, two accumulators
  static constexpr int kAccStride = kTmemCols / 2;
  static constexpr int kChunks = (BN + 31) / 32;                                // 32-column epilogue chunks
};

template <int BN, int ST = 0>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tma_a, const CUtensorMap& tma_b,
                                          const CUtensorMap* a_peer_maps, const GemmParams& p) {
  using Cfg = GemmCfg<BN, ST>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tfull_bar = empty_bar + Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int mn_tiles = p.tile_map ? (p.num_tiles_dev ? min(*p.num_tiles_dev, p.num_map_tiles) : p.num_map_tiles)
                                  : tiles_m * tiles_n;
  const int total_tiles = mn_tiles * p.splits;
  const int k_blocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4);
    }
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_launch_dependents();   // the next kernel of a chained launch may start its own set-up now

  // Tile decode shared by all roles.  Consecutive tile ids walk 8 m-tiles of
  // one n-band before moving on, so CTAs running at the same time share B in L2.
  // c_off / bk_off: see GemmParams::tile_ext (0 without it)
  int c_off = 0, bk_off = 0;
  auto decode = [&](int t, int& m0, int& m_end, int& b_row, int& n0, int& kb0, int& kb1) {
    const int split = t / mn_tiles;
    const int tt = t - split * mn_tiles;
    kb0 = static_cast<int>((static_cast<long long>(k_blocks) * split) / p.splits);
    kb1 = static_cast<int>((static_cast<long long>(k_blocks) * (split + 1)) / p.splits);
    if (p.tile_map) {
      const int4 e = p.tile_map[tt];
      m0 = e.x;
      m_end = e.y;
      n0 = e.w * BN;
      b_row = e.z + n0;
      if (p.tile_ext) {
        const int4 x = p.tile_ext[tt];
        c_off = x.x;
        bk_off = x.w;
        if (x.z >= 0) {
          kb0 = max(0, x.y);
          kb1 = min(k_blocks, x.z);
          if (kb1 < kb0) kb1 = kb0;
        }
      }
    } else {
      constexpr int G = 8;
      const int per_group = G * tiles_n;
      const int g = tt / per_group;
      const int first_m = g * G;
      const int gsize = min(tiles_m - first_m, G);
      const int r = tt - g * per_group;
      const int mi = first_m + r % gsize;
      const int ni = r / gsize;
      m0 = mi * kBM;
      m_end = p.M;
      n0 = ni * BN;
      b_row = n0;
    }
  };

  // Skinny problems (one row tile: decode) have every CTA read the SAME activation tile for the same k-block at the
  // same moment -- more than a hundred SMs queueing on the few L2 slices that hold those 16 KB.  Each output tile
  // therefore walks its K range from a different starting block (sums are order independent up to rounding), which
  // spreads the activation reads over the whole L2.
  auto k_rotation = [&](int tile, int nkb) -> int {
    return (tiles_m == 1 && !p.tile_map && nkb > 1) ? tile % nkb : 0;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // Chained launch: the B tiles (weights) of the first ring-full of k-blocks are requested BEFORE waiting for
      // the previous kernel, so the weight stream is already in flight when its output (A) becomes readable.
      int prefetched = 0;
      if (p.chained && blockIdx.x < total_tiles && !(a_peer_maps != nullptr && p.a_peer_rows > 0)) {
        int m0, m_end, b_row, n0, kb0, kb1;
        decode(blockIdx.x, m0, m_end, b_row, n0, kb0, kb1);
        prefetched = min(Cfg::kStages, kb1 - kb0);
        const int rot = k_rotation(blockIdx.x, kb1 - kb0);
        for (int i = 0; i < prefetched; ++i) {
          const int kb = kb0 + (i + rot) % (kb1 - kb0);
          uint8_t* sb = smem + i * Cfg::kStageBytes + Cfg::kABytes;
          mbar_expect_tx(&full_bar[i], Cfg::kStageBytes);
          if (!p.b_mn) {
            tma_load_2d(sb, &tma_b, &full_bar[i], kb * kBK, b_row);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * kBK * 2), &tma_b, &full_bar[i], b_row + c * 64, kb * kBK + bk_off);
          }
        }
      }
      pdl_wait();
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int m0, m_end, b_row, n0, kb0, kb1;
        decode(t, m0, m_end, b_row, n0, kb0, kb1);
        const int rot = k_rotation(t, kb1 - kb0);
        for (int it = 0; it < kb1 - kb0; ++it) {
          const int kb = kb0 + (it + rot) % (kb1 - kb0);
          const bool b_done = prefetched > 0;      // this stage's barrier is armed and its B tile requested already
          if (b_done) --prefetched;
          if (!b_done && !mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          if (!b_done) mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if (a_peer_maps != nullptr && p.a_peer_rows > 0) {
            // all-gather fused into the operand fetch: each slab of the A tile comes from the rank that owns
            // those rows, by a plain (non-multicast) TMA load from its peer mapping
            const int br = min(kBM, p.a_peer_rows);
            for (int i = 0; i < kBM / br; ++i) {
              const int row = m0 + i * br;
              const int peer = min(row / p.a_peer_rows, p.world - 1);
              tma_load_2d(sa + i * br * 128, &a_peer_maps[peer], &full_bar[stage], kb * kBK,
                          row - peer * p.a_peer_rows);
            }
          } else if (!p.a_mn) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * kBK, m0);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_2d(sa + c * (64 * kBK * 2), &tma_a, &full_bar[stage], m0 + c * 64, kb * kBK);
          }
          if (b_done) {
            // requested before the wait
          } else if (!p.b_mn) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], kb * kBK, b_row);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (64 * kBK * 2), &tma_b, &full_bar[stage], b_row + c * 64, kb * kBK + bk_off);
          }
          if (++stage == Cfg::kStages) {
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
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      pdl_wait();
      const uint32_t idesc = umma_idesc_bf16(kBM, BN, p.a_mn, p.b_mn);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int m0, m_end, b_row, n0, kb0, kb1;
        decode(t, m0, m_end, b_row, n0, kb0, kb1);
        if (kb1 <= kb0) continue;              // a group without rows: no loads, no accumulator, nothing stored
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1, p.status, kTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * Cfg::kAccStride;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = p.a_mn ? umma_smem_desc(sa + k * 2048, 64 * kBK * 2, 1024)
                                       : umma_smem_desc(sa + k * 32, 0, 1024);
            const uint64_t db = p.b_mn ? umma_smem_desc(sb + k * 2048, 64 * kBK * 2, 1024)
                                       : umma_smem_desc(sb + k * 32, 0, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tfull_bar[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    int it = 0;
    bool ok = true;
    pdl_wait();                    // the output buffer may still be read (or cleared) by the previous kernel
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int m0, m_end, b_row, n0, kb0, kb1;
      decode(t, m0, m_end, b_row, n0, kb0, kb1);
      if (kb1 <= kb0) continue;
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tfull_bar[buf], acc_phase, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < m_end;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * Cfg::kAccStride;
      if (p.epi == kEpiLogprobPartial) {
        // BN == 128 here: one partial record per row and tile
        const float rs = p.alpha * ((p.row_scale && row_ok) ? p.row_scale[row] : 1.f);
        const int label = row_ok ? p.labels[row] : -1;
        float m_run = -INFINITY, s_run = 0.f, e_run = 0.f, lab = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          float z[32];
          float cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            z[j] = (col0 + j < p.N) ? __uint_as_float(r[j]) * rs : -INFINITY;
            cm = fmaxf(cm, z[j]);
            if (col0 + j == label) lab = z[j];
          }
          const float m_new = fmaxf(m_run, cm);
          const float corr = __expf(m_run - m_new);
          float cs = 0.f, ce = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float ex = (col0 + j < p.N) ? __expf(z[j] - m_new) : 0.f;
            cs += ex;
            ce += (col0 + j < p.N) ? ex * z[j] : 0.f;
          }
          s_run = s_run * corr + cs;
          e_run = e_run * corr + ce;
          m_run = m_new;
        }
        if (row_ok) {
          const int tiles_n_ = (p.N + BN - 1) / BN;
          float4* dst = reinterpret_cast<float4*>(p.partial) + static_cast<long long>(row) * tiles_n_ + n0 / BN;
          *dst = make_float4(m_run, s_run, e_run, lab);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        continue;
      }
      if (p.epi == kEpiDlogits) {
        const float it = (p.row_scale && row_ok) ? p.row_scale[row] : 1.f;
        const float rs = p.alpha * it;
        const int label = row_ok ? p.labels[row] : -1;
        const float lse = row_ok ? p.row_lse[row] : 0.f;
        const float ent = row_ok ? p.row_ent[row] : 0.f;
        const float glp = row_ok ? p.row_glp[row] : 0.f;
        const float gent = (row_ok && p.row_gent) ? p.row_gent[row] : 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (!row_ok) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float z = __uint_as_float(r[j]) * rs;
            const float pj = __expf(z - lse);
            float g = -glp * pj - gent * pj * (z - lse + ent);
            if (col0 + j == label) g += glp;
            v[j] = g * rs;
          }
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col0 + q * 8 < p.N) {
              uint4 o;
              o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
              o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
              o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
              o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
              *reinterpret_cast<uint4*>(dst + q * 8) = o;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[buf]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < Cfg::kChunks; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        const int ncols = min(32, BN - c * 32);   // 16 in the last chunk of a width that is not a multiple of 32
        if (BN % 32 != 0 && ncols == 16) {
          uint32_t h[16];
          tmem_ld_32x16(taddr + c * 32, h);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = h[j];
#pragma unroll
          for (int j = 16; j < 32; ++j) r[j] = 0u;
        } else {
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
        }
        if (!row_ok) continue;
        gemm_store_chunk(p, row + c_off, col0, r, ncols);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  gemm_body<BN>(tma_a, tma_b, nullptr, p);
}

// Two CTAs per SM with a 3-stage ring each (see GemmCfg).
template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_bf16_x2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  gemm_body<BN, 3>(tma_a, tma_b, nullptr, p);
}

// Variant whose A operand is gathered from the other ranks' memory tile by tile (all-gather -> GEMM).
template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_ag_kernel(const __grid_constant__ PeerTensorMaps a_maps, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  gemm_body<BN>(a_maps.m[0], tma_b, a_maps.m, p);
}

}  // namespace apb

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace apb {

template <int BN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_ctas,
                       cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int mn_tiles = p.tile_map ? p.num_map_tiles : tiles_m * tiles_n;
  const long long total = static_cast<long long>(mn_tiles) * p.splits;
  int grid = static_cast<int>(total < sm_count() ? total : sm_count());
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid <= 0) return 0;
  return static_cast<int>(launch_kernel(gemm_bf16_kernel<BN>, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream,
                                        ta, tb, p));
}

template <int BN>
static int launch_gemm_x2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, 3>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_x2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const int tiles_m = (p.M + kBM - 1) / kBM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int mn_tiles = p.tile_map ? p.num_map_tiles : tiles_m * tiles_n;
  const long long total = static_cast<long long>(mn_tiles) * p.splits;
  const int cap = 2 * sm_count();
  const int grid = static_cast<int>(total < cap ? total : cap);
  if (grid <= 0) return 0;
  return static_cast<int>(launch_kernel(gemm_bf16_x2_kernel<BN>, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes,
                                        stream, ta, tb, p));
}

}  // namespace apb

extern "C" int apb_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, int a_mn, int b_mn, int epi, float alpha,
                                  const void* bias, void* C2, long long ldc2, cudaStream_t stream);

namespace apb {
static bool pair_kernel_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("APB_GEMM_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}
}  // namespace apb

extern "C" {

// D = alpha * op(A) * op(B)^T (+ epilogue).  bf16 operands.
//   a_mn = 0: A is [M,K] row-major (lda >= K);  a_mn = 1: A is stored [K,M] (lda >= M)
//   b_mn = 0: B is [N,K] row-major (ldb >= K);  b_mn = 1: B is stored [K,N] (ldb >= N)
// All leading dimensions and N must be multiples of 8; bases 16-byte aligned.
// tile_map (device, optional) has `num_map_tiles` int4 {m0, m_end, b_row_offset, n_tile}
// entries and turns the launch into a grouped GEMM over row ranges of A/C with
// per-group B row offsets (b_rows = total rows of the stacked B).
// bn = 0 picks the tile width; splits > 1 needs an atomic fp32 epilogue.
// max_ctas > 0 caps the grid (leaves SMs free for a concurrent kernel).
static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int a_mn, int b_mn, int epi, int splits, float alpha, const void* bias,
                         void* C2, long long ldc2, const void* tile_map, int num_map_tiles, const int* num_tiles_dev,
                         long long b_rows, int bn, int max_ctas, cudaStream_t stream, const void* tile_ext = nullptr,
                         long long b_k_rows = 0) {
  using namespace apb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tile_ext && (!tile_map || splits > 1)) return kBadArgument;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return kBadArgument;
  if (epi == kEpiBf16 || epi == kEpiSwiGLU) {
    if (C && (ldc % 8)) return kBadArgument;
  } else if (ldc % 4) {
    return kBadArgument;
  }
  if (epi == kEpiSwiGLU && (!C2 || (ldc2 % 8) || (N % 16))) return kBadArgument;
  const int k_blocks = (K + kBK - 1) / kBK;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks;
  if (splits > 1 && epi != kEpiF32Atomic) return kBadArgument;
  // Large plain problems go to the CTA-pair kernel (256 x 256 tiles, half of B per SM): at least one full wave
  // of pairs, automatic tile choice, no grid cap.  APB_GEMM_PAIR=0 keeps everything on the one-CTA kernel.
  if (bn == 0 && splits == 1 && !tile_map && max_ctas <= 0 && pair_kernel_enabled() &&
      (epi == kEpiBf16 || epi == kEpiF32 || epi == kEpiF32Accum || epi == kEpiSwiGLU) &&
      !(epi == kEpiBf16 && !C) && M >= 512 &&
      static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) >= sm_count() / 2)
    return apb_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, alpha, bias, C2, ldc2, stream);
  if (bn == 0) {
    const long long tm = (M + kBM - 1) / kBM;
    const long long t256 = tm * ((N + 255) / 256) * splits;
    const long long t128 = tm * ((N + 127) / 128) * splits;
    bn = (N >= 256 && t256 >= sm_count()) ? 256 : 128;
    // skinny problems (decode): narrower tiles put more SMs on the weight stream
    if (bn == 128 && t128 * 10 < sm_count() * 7 && N >= 128) bn = 64;
    if (tile_map) bn = 128;
    // one row tile (decode): the width that covers N in the fewest waves of SMs, then the fewest idle SMs
    if (!tile_map && tm == 1 && splits == 1 && !b_mn && N >= 1024 && epi != kEpiLogprobPartial && epi != kEpiDlogits) {
      const int cand[5] = {256, 208, 144, 128, 64};
      long long best_cost = -1;
      for (int i = 0; i < 5; ++i) {
        const long long tiles = (N + cand[i] - 1) / cand[i];
        const long long waves = (tiles + sm_count() - 1) / sm_count();
        const long long cost = waves * cand[i];          // columns streamed by the busiest SM
        if (best_cost < 0 || cost < best_cost) {
          best_cost = cost;
          bn = cand[i];
        }
      }
    }
  }
  // bn = 1000 + width: the two-CTAs-per-SM variant (widths 64 and 128)
  const bool x2 = bn > 1000;
  if (x2) bn -= 1000;
  if (bn != 64 && bn != 128 && bn != 144 && bn != 208 && bn != 256) return kBadArgument;
  if (x2 && bn != 64 && bn != 128) return kBadArgument;
  // the in-between widths exist for skinny NT products (decode); they do not take the transposed-B layout (its
  // 64-column chunks), the tile table or the lm-head epilogues
  if ((bn == 144 || bn == 208) && (b_mn || tile_map || epi == kEpiLogprobPartial || epi == kEpiDlogits))
    return kBadArgument;

  CUtensorMap ta, tb;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&ta, A, 2, static_cast<uint64_t>(M), static_cast<uint64_t>(K), lda, 64, kBM);
  else
    rc = make_tmap_2d(&ta, A, 2, static_cast<uint64_t>(K), static_cast<uint64_t>(M), lda, 64, 64);
  if (rc) return 1000 + rc;
  const uint64_t brows = b_rows > 0 ? static_cast<uint64_t>(b_rows) : static_cast<uint64_t>(N);
  if (!b_mn)
    rc = make_tmap_2d(&tb, B, 2, brows, static_cast<uint64_t>(K), ldb, 64, bn);
  else
    rc = make_tmap_2d(&tb, B, 2, static_cast<uint64_t>(b_k_rows > 0 ? b_k_rows : K), brows, ldb, 64, 64);
  if (rc) return 2000 + rc;

  GemmParams p{};  // zero: the peer-mode fields must read 0 in the plain path
  p.M = M;
  p.N = N;
  p.K = K;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.epi = epi;
  p.splits = splits;
  p.C = C;
  p.ldc = ldc;
  p.C2 = C2;
  p.ldc2 = ldc2;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha;
  p.tile_map = static_cast<const int4*>(tile_map);
  p.num_map_tiles = num_map_tiles;
  p.num_tiles_dev = tile_map ? num_tiles_dev : nullptr;
  p.tile_ext = static_cast<const int4*>(tile_ext);
  p.status = status_device_ptr();
  p.row_scale = nullptr;
  p.labels = nullptr;
  p.partial = nullptr;
  p.row_lse = p.row_ent = p.row_glp = p.row_gent = nullptr;
  p.chained = chained_launch_on() ? 1 : 0;
  if (x2) return bn == 64 ? launch_gemm_x2<64>(ta, tb, p, stream) : launch_gemm_x2<128>(ta, tb, p, stream);
  if (bn == 64) return launch_gemm<64>(ta, tb, p, max_ctas, stream);
  if (bn == 144) return launch_gemm<144>(ta, tb, p, max_ctas, stream);
  if (bn == 208) return launch_gemm<208>(ta, tb, p, max_ctas, stream);
  return bn == 256 ? launch_gemm<256>(ta, tb, p, max_ctas, stream) : launch_gemm<128>(ta, tb, p, max_ctas, stream);
}

int apb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                  long long ldc, int a_mn, int b_mn, int epi, int splits, float alpha, const void* bias,
                  void* C2, long long ldc2, const void* tile_map, int num_map_tiles, long long b_rows, int bn,
                  int max_ctas, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, splits, alpha, bias, C2, ldc2, tile_map,
                        num_map_tiles, nullptr, b_rows, bn, max_ctas, stream);
}

// Grouped GEMM whose tile table was written by a kernel: `tile_map` has room for `max_tiles` entries, the number in
// use is read from `*num_tiles_dev` when the GEMM runs (no host round trip between routing and the expert GEMMs).
int apb_gemm_bf16_grouped_dev(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                              long long ldc, int epi, float alpha, void* C2, long long ldc2, const void* tile_map,
                              int max_tiles, const int* num_tiles_dev, long long b_rows, cudaStream_t stream) {
  if (!tile_map || !num_tiles_dev || max_tiles <= 0) return apb::kBadArgument;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, epi, 1, alpha, nullptr, C2, ldc2, tile_map, max_tiles,
                        num_tiles_dev, b_rows, 128, 0, stream);
}

// The grouped backward passes of an expert layer, tables written by a kernel (apb_moe_plan):
//   data gradient    dX[rows of e] = dY[rows of e] @ W[e],  W stacked [E * K, N] (b_mn = 1, bk_off = e * K per tile);
//   weight gradient  dW[e] (+)= dY[rows of e]^T @ X[rows of e]: a_mn = b_mn = 1, K = the row axis, every tile walks
//                    the k-blocks of its expert's rows (64-row aligned, padding rows zero) and writes the e-th slab of
//                    the stacked dW (c_row_off = e * M).
// `tile_ext` holds one {c_row_off, kb0, kb1, bk_off} record per tile of `tile_map`.  b_k_rows: rows of the stacked
// [K, N] B (0: K).  b_n_rows: rows of a stacked [N, K] B (0: N).  num_tiles_dev may be null (all max_tiles live).
int apb_gemm_bf16_grouped_ext(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                              long long ldc, int a_mn, int b_mn, int epi, float alpha, const void* tile_map,
                              const void* tile_ext, int max_tiles, const int* num_tiles_dev, long long b_n_rows,
                              long long b_k_rows, cudaStream_t stream) {
  if (!tile_map || !tile_ext || max_tiles <= 0) return apb::kBadArgument;
  if (epi != apb::kEpiBf16 && epi != apb::kEpiF32 && epi != apb::kEpiF32Accum) return apb::kBadArgument;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, 1, alpha, nullptr, nullptr, 0, tile_map,
                        max_tiles, num_tiles_dev, b_n_rows, 128, 0, stream, tile_ext, b_k_rows);
}
}

// ---------------------------------------------------------------------------
// lm_head + log-softmax + label gather + entropy
// ---------------------------------------------------------------------------
namespace apb {

// Combines the per-tile partials of one row: lse, log-prob of the label, entropy = lse - E[z].
__global__ void lmhead_combine_kernel(const float4* __restrict__ partial, int tiles, float* __restrict__ lp,
                                      float* __restrict__ ent, float* __restrict__ lse_out, int M) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float4* pr = partial + static_cast<long long>(row) * tiles;
  float m = -INFINITY, s = 0.f, e = 0.f, lab = -INFINITY;
  for (int t = lane; t < tiles; t += 32) {
    const float4 v = pr[t];
    const float mn = fmaxf(m, v.x);
    const float c0 = (m == -INFINITY) ? 0.f : __expf(m - mn);
    const float c1 = (v.x == -INFINITY) ? 0.f : __expf(v.x - mn);
    s = s * c0 + v.y * c1;
    e = e * c0 + v.z * c1;
    m = mn;
    lab = fmaxf(lab, v.w);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float e2 = __shfl_xor_sync(0xffffffffu, e, o);
    const float l2 = __shfl_xor_sync(0xffffffffu, lab, o);
    const float mn = fmaxf(m, m2);
    const float c0 = (m == -INFINITY) ? 0.f : __expf(m - mn);
    const float c1 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
    s = s * c0 + s2 * c1;
    e = e * c0 + e2 * c1;
    m = mn;
    lab = fmaxf(lab, l2);
  }
  if (lane == 0) {
    const float lse = m + logf(s);
    lse_out[row] = lse;
    lp[row] = lab - lse;
    ent[row] = lse - e / s;
  }
}

static int lmhead_launch(const void* hidden, const void* weight, int M, int V, int H, long long ldh, long long ldw,
                         GemmParams& p, int bn, cudaStream_t stream) {
  if ((ldh % 8) || (ldw % 8) || (V % 8)) return kBadArgument;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, hidden, 2, M, H, ldh, 64, kBM);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tb, weight, 2, V, H, ldw, 64, bn);
  if (rc) return 2000 + rc;
  p.M = M;
  p.N = V;
  p.K = H;
  p.a_mn = 0;
  p.b_mn = 0;
  p.splits = 1;
  p.C2 = nullptr;
  p.ldc2 = 0;
  p.bias = nullptr;
  p.tile_map = nullptr;
  p.num_map_tiles = 0;
  p.status = status_device_ptr();
  return bn == 256 ? launch_gemm<256>(ta, tb, p, 0, stream) : launch_gemm<128>(ta, tb, p, 0, stream);
}

}  // namespace apb

extern "C" {

// hidden [M,H] bf16, weight [V,H] bf16, labels [M] int32, row_scale [M] fp32 or null (then `scale` applies).
// partial: fp32 scratch [M][ceil(V/128)][4].  Outputs lp/ent/lse fp32 [M].
int apb_lmhead_logprob_fwd(const void* hidden, const void* weight, const int* labels, const float* row_scale,
                           float* partial, float* lp, float* ent, float* lse, int M, int V, int H, long long ldh,
                           long long ldw, float scale, cudaStream_t stream) {
  using namespace apb;
  if (M <= 0) return 0;
  if (!hidden || !weight || !labels || !partial || !lp || !ent || !lse) return kBadArgument;
  GemmParams p{};
  p.epi = kEpiLogprobPartial;
  p.alpha = scale;
  p.C = nullptr;
  p.ldc = 0;
  p.row_scale = row_scale;
  p.labels = labels;
  p.partial = partial;
  int rc = lmhead_launch(hidden, weight, M, V, H, ldh, ldw, p, 128, stream);
  if (rc) return rc;
  const int tiles = (V + 127) / 128;
  const int grid = (M * 32 + 255) / 256;
  lmhead_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(partial), tiles, lp, ent, lse, M);
  return static_cast<int>(cudaGetLastError());
}

// dlogits [M,V] bf16 (row stride ldd) = d loss / d (hidden @ weight^T) given upstream g_lp, g_ent (null = 0).
int apb_lmhead_dlogits(const void* hidden, const void* weight, const int* labels, const float* row_scale,
                       const float* lse, const float* ent, const float* g_lp, const float* g_ent, void* dlogits,
                       int M, int V, int H, long long ldh, long long ldw, long long ldd, float scale,
                       cudaStream_t stream) {
  using namespace apb;
  if (M <= 0) return 0;
  if (ldd % 8) return kBadArgument;
  GemmParams p{};
  p.epi = kEpiDlogits;
  p.alpha = scale;
  p.C = dlogits;
  p.ldc = ldd;
  p.row_scale = row_scale;
  p.labels = labels;
  p.row_lse = lse;
  p.row_ent = ent;
  p.row_glp = g_lp;
  p.row_gent = g_ent;
  return lmhead_launch(hidden, weight, M, V, H, ldh, ldw, p, 256, stream);
}
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the fused lm-head log-prob forward (see apb_noalloc.h)
// ---------------------------------------------------------------------------
#include "apb_noalloc.h"

namespace apb {
// Per-tile reduction records (max, sum-exp, sum exp*z, label logit) for the no-alloc entry point.
// File-scope device storage: its size is fixed at build time and every device that loads the
// library carries it.  In host code this name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) float4 g_noalloc_partials[APB_NOALLOC_MAX_TILE_RECORDS];
}  // namespace apb

extern "C" int apb_lmhead_logprob_fwd_noalloc(const void* hidden, const void* weight, const int* labels,
                                               const float* row_scale, float* lp, float* ent, float* lse, int M,
                                               int V, int H, long long ldh, long long ldw, float scale,
                                               cudaStream_t stream) {
  using namespace apb;
  if (M <= 0) return 0;
  if (V <= 0 || H <= 0 || !hidden || !weight || !labels || !lp || !ent || !lse) return kBadArgument;
  const long long tiles = (static_cast<long long>(V) + 127) / 128;
  if (static_cast<long long>(M) * tiles > APB_NOALLOC_MAX_TILE_RECORDS) return APB_NOALLOC_TOO_LARGE;
  // One-time set-up per device (with that device current): resolve the device address of the scratch.
  // The cache below is filled without a lock: two host threads that make the first call together both
  // look the address up and store the same value, which is harmless.
  static float4* scratch_ptr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return APB_NOALLOC_SETUP_FAILED;
  if (!scratch_ptr[dev]) {
    float4* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials) != cudaSuccess || !p)
      return APB_NOALLOC_SETUP_FAILED;
    scratch_ptr[dev] = p;
  }
  float* partial = reinterpret_cast<float*>(scratch_ptr[dev]);
  GemmParams p{};
  p.epi = kEpiLogprobPartial;
  p.alpha = scale;
  p.C = nullptr;
  p.ldc = 0;
  p.row_scale = row_scale;
  p.labels = labels;
  p.partial = partial;
  int rc = lmhead_launch(hidden, weight, M, V, H, ldh, ldw, p, 128, stream);
  if (rc) return rc;
  const int grid = (M * 32 + 255) / 256;
  lmhead_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(partial), static_cast<int>(tiles),
                                                  lp, ent, lse, M);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Tensor-parallel fused GEMM + collective entry points
// ---------------------------------------------------------------------------
namespace apb {

// After a GEMM -> reduce-scatter: wait until every rank has finished adding into this rank's fp32 slice,
// then convert the slice to bf16 and clear it for its next use.
__global__ void __launch_bounds__(256)
tp_finalize_kernel(PeerPtrs flags, int rank, int world, int epoch, float* __restrict__ acc,
                   __nv_bfloat16* __restrict__ out, long long n, int* status) {
  if (!epoch_barrier(flags, rank, world, epoch, status)) return;
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4* a = reinterpret_cast<float4*>(acc + i * 8);
    const float4 x = a[0], y = a[1];
    uint4 o;
    o.x = pack_bf16x2(x.x, x.y);
    o.y = pack_bf16x2(x.z, x.w);
    o.z = pack_bf16x2(y.x, y.y);
    o.w = pack_bf16x2(y.z, y.w);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
    a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <int BN>
static int launch_gemm_ag(const PeerTensorMaps& maps, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_ag_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const long long total = static_cast<long long>((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN);
  const int grid = static_cast<int>(total < sm_count() ? total : sm_count());
  gemm_bf16_ag_kernel<BN><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(maps, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace apb

extern "C" {

// All-gather -> GEMM.  The activation is row-sharded: rank r holds rows [r*rows, (r+1)*rows) of A in its own
// buffer a_ptrs[r] ([rows, K] bf16, row stride lda, all mapped into this process).  Computes
// C[M = world*rows, N] = A_full @ B[N,K]^T on this rank; every A tile is fetched from its owner's memory by
// plain TMA loads while earlier tiles are multiplied.  The caller orders this launch after the peers' writes
// (apb_epoch_wait).  rows must be a multiple of 8 and either >= 128 with rows % 128 == 0, or a divisor of 128.
int apb_gemm_ag(void* const* a_ptrs, int world, int rows, const void* B, void* C, int N, int K, long long lda,
                long long ldb, long long ldc, int bn, cudaStream_t stream) {
  using namespace apb;
  if (world < 1 || world > 8 || rows <= 0 || (rows % 8)) return kBadArgument;
  if (rows >= kBM ? (rows % kBM) : (kBM % rows)) return kBadArgument;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return kBadArgument;
  PeerTensorMaps maps;
  const int br = rows < kBM ? rows : kBM;
  for (int r = 0; r < 8; ++r) {
    const int src = r < world ? r : 0;
    int rc = make_tmap_2d(&maps.m[r], a_ptrs[src], 2, rows, K, lda, 64, br);
    if (rc) return 1000 + rc;
  }
  if (bn == 0) bn = 128;
  if (bn != 64 && bn != 128 && bn != 256) return kBadArgument;
  CUtensorMap tb;
  int rc = make_tmap_2d(&tb, B, 2, N, K, ldb, 64, bn);
  if (rc) return 2000 + rc;
  GemmParams p{};
  p.M = world * rows;
  p.N = N;
  p.K = K;
  p.epi = kEpiBf16;
  p.splits = 1;
  p.C = C;
  p.ldc = ldc;
  p.alpha = 1.f;
  p.status = status_device_ptr();
  p.a_peer_rows = rows;
  p.world = world;
  if (bn == 64) return launch_gemm_ag<64>(maps, tb, p, stream);
  return bn == 256 ? launch_gemm_ag<256>(maps, tb, p, stream) : launch_gemm_ag<128>(maps, tb, p, stream);
}

// GEMM -> reduce-scatter.  Every rank computes its partial P = A[M,K_local] @ B[N,K_local]^T and adds each
// row into the fp32 accumulator of the rank that owns it (acc_ptrs[r]: [M/world, N] fp32, zero on entry),
// straight from the GEMM epilogue over the NVLink peer mappings.  Follow with apb_tp_finalize.
int apb_gemm_rs(const void* A, const void* B, void* const* acc_ptrs, int world, int M, int N, int K, long long lda,
                long long ldb, long long ld_acc, int bn, int splits, cudaStream_t stream) {
  using namespace apb;
  if (world < 1 || world > 8 || M % world || (lda % 8) || (ldb % 8) || (ld_acc % 4) || (N % 8)) return kBadArgument;
  if (bn == 0) bn = 128;
  // the epilogue adds into the owners' accumulators anyway, so the product may also be cut along K: skinny
  // (decode) problems then put every SM on the weight stream
  const int k_blocks = (K + kBK - 1) / kBK;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, 2, M, K, lda, 64, kBM);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tb, B, 2, N, K, ldb, 64, bn);
  if (rc) return 2000 + rc;
  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.epi = kEpiF32AtomicPeer;
  p.splits = splits;
  p.ldc = ld_acc;
  p.chained = chained_launch_on() ? 1 : 0;
  p.alpha = 1.f;
  p.status = status_device_ptr();
  p.rows_per_rank = M / world;
  p.world = world;
  for (int r = 0; r < 8; ++r) p.c_peers[r] = r < world ? acc_ptrs[r] : nullptr;
  if (bn == 64) return launch_gemm<64>(ta, tb, p, 0, stream);
  return bn == 256 ? launch_gemm<256>(ta, tb, p, 0, stream) : launch_gemm<128>(ta, tb, p, 0, stream);
}

// Grouped GEMM whose output rows are scattered to other ranks: row m of the result goes to
// out_ptrs[row_map[m].x] + row_map[m].y * ldc (bf16).  Used as the fused "expert GEMM 2 + combine" of
// expert-parallel MoE.  tile_map as in apb_gemm_bf16.
static int gemm_scatter_impl(const void* A, const void* B, void* const* out_ptrs, int world, const void* row_map, int M,
                             int N, int K, long long lda, long long ldb, long long ldc, const void* tile_map,
                             int num_map_tiles, const int* num_tiles_dev, long long b_rows, cudaStream_t stream) {
  using namespace apb;
  if (M <= 0) return 0;
  if (world < 1 || world > 8 || (lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return kBadArgument;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, 2, M, K, lda, 64, kBM);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tb, B, 2, b_rows > 0 ? b_rows : N, K, ldb, 64, 128);
  if (rc) return 2000 + rc;
  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.epi = kEpiBf16ScatterPeer;
  p.splits = 1;
  p.ldc = ldc;
  p.alpha = 1.f;
  p.tile_map = static_cast<const int4*>(tile_map);
  p.num_map_tiles = num_map_tiles;
  p.num_tiles_dev = num_tiles_dev;
  p.status = status_device_ptr();
  p.row_map = static_cast<const int2*>(row_map);
  p.world = world;
  for (int r = 0; r < 8; ++r) p.c_peers[r] = r < world ? out_ptrs[r] : nullptr;
  return launch_gemm<128>(ta, tb, p, 0, stream);
}

int apb_gemm_scatter(const void* A, const void* B, void* const* out_ptrs, int world, const void* row_map, int M, int N,
                     int K, long long lda, long long ldb, long long ldc, const void* tile_map, int num_map_tiles,
                     long long b_rows, cudaStream_t stream) {
  return gemm_scatter_impl(A, B, out_ptrs, world, row_map, M, N, K, lda, ldb, ldc, tile_map, num_map_tiles, nullptr,
                           b_rows, stream);
}

// The same with a tile table written by a kernel: room for `max_tiles` records, the live count read from
// `*num_tiles_dev` when the GEMM runs.
int apb_gemm_scatter_dev(const void* A, const void* B, void* const* out_ptrs, int world, const void* row_map, int M,
                         int N, int K, long long lda, long long ldb, long long ldc, const void* tile_map, int max_tiles,
                         const int* num_tiles_dev, long long b_rows, cudaStream_t stream) {
  if (!tile_map || !num_tiles_dev || max_tiles <= 0) return apb::kBadArgument;
  return gemm_scatter_impl(A, B, out_ptrs, world, row_map, M, N, K, lda, ldb, ldc, tile_map, max_tiles, num_tiles_dev,
                           b_rows, stream);
}

int apb_tp_finalize(void* const* flag_ptrs, int rank, int world, int epoch, float* acc, void* out, long long n,
                    cudaStream_t stream) {
  using namespace apb;
  if (world > kMaxRanks || (n % 8)) return kBadArgument;
  if (n <= 0) return 0;
  PeerPtrs f;
  for (int i = 0; i < kMaxRanks; ++i) f.p[i] = i < world ? flag_ptrs[i] : nullptr;
  long long g = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  const int grid = static_cast<int>(g < 1 ? 1 : (g < cap ? g : cap));
  tp_finalize_kernel<<<grid, 256, 0, stream>>>(f, rank, world, epoch, acc, static_cast<__nv_bfloat16*>(out), n,
                                               status_device_ptr());
  return static_cast<int>(cudaGetLastError());
}
}
