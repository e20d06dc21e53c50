// Declarations shared by the bf16 GEMM kernels of this package (the one-CTA kernel in gemm_tcgen05.cu and the
// CTA-pair kernel in gemm_tcgen05_2cta.cu): the parameter block, the epilogue kinds and the per-chunk epilogue
// (32 accumulator columns of one output row, already in registers) that both kernels run after reading TMEM.
#pragma once
#include "common.cuh"

namespace apb {

enum GemmEpilogue : int {
  kEpiBf16 = 0,        // C(bf16) = alpha * acc (+ bias[n])
  kEpiF32 = 1,         // C(f32)  = alpha * acc
  kEpiF32Atomic = 2,   // C(f32) += alpha * acc  (red.add; split-K or shared accumulation)
  kEpiF32Accum = 3,    // C(f32) += alpha * acc  (plain read-modify-write, one writer)
  kEpiSwiGLU = 4,      // columns interleaved (gate, up): C2(bf16)[m, n/2] = silu(g) * u; C(bf16) = acc if C != null
  kEpiLogprobPartial = 5,  // per row and 128-column tile: (max, sum exp, sum exp*z, label z) of z = acc*alpha*row_scale
  kEpiDlogits = 6,         // C(bf16) = d loss / d acc for log-prob / entropy heads (see lm-head section below)
  kEpiF32AtomicPeer = 7,   // GEMM -> reduce-scatter: red.add of the partial row into the fp32 buffer of the rank
                           // that owns the row (owner = row / rows_per_rank), over its NVLink peer mapping
  kEpiBf16ScatterPeer = 8, // GEMM -> all-to-all: bf16 row stored to (peer, row) = row_map[m] (MoE combine)
};

struct PeerTensorMaps {
  CUtensorMap m[8];
};

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int epi;
  int splits;
  void* C;
  long long ldc;
  void* C2;
  long long ldc2;
  const __nv_bfloat16* bias;
  float alpha;
  // Optional tile table for grouped problems: {m0, m_end, b_row_offset, n_tile}.
  const int4* tile_map;
  int num_map_tiles;         // entries of tile_map (an upper bound when num_tiles_dev is set)
  const int* num_tiles_dev;  // optional: the live entry count, written by a kernel (a routing plan built on the device)
  // Optional second record per tile (grouped backward passes): {c_row_off, kb0, kb1, bk_off}.  The tile's output rows
  // are written at row + c_row_off (per-group slabs of a stacked C), its K walk is the k-block range [kb0, kb1)
  // (kb1 < 0: all of K; an empty range skips the tile -- a group without rows), and B's K coordinate is shifted
  // by bk_off rows (per-group slabs of a stacked [K, N] B).
  const int4* tile_ext;
  int* status;
  // log-prob epilogues
  const float* row_scale;  // [M] per-row multiplier of the logits (inverse temperature) or null
  const int* labels;       // [M]
  float* partial;          // [M][tiles_n][4]
  const float* row_lse;    // [M] log-sum-exp of the scaled logits
  const float* row_ent;    // [M] entropy
  const float* row_glp;    // [M] upstream gradient of the log-prob
  const float* row_gent;   // [M] upstream gradient of the entropy, or null
  // peer-aware modes
  void* c_peers[8];        // per-rank output base pointers (symmetric buffers)
  int rows_per_rank;       // kEpiF32AtomicPeer: rows owned by each rank
  const int2* row_map;     // kEpiBf16ScatterPeer: (rank, destination row) per output row, rank < 0 = drop
  int a_peer_rows;         // > 0: A is row-sharded over ranks, this many rows each, read through per-rank maps
  int world;
  int chained;             // 1: launched in chained mode -- B (weights nobody in the chain writes) is prefetched
                           // before the wait for the previous kernel, everything else after it
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// One output row, 32 consecutive accumulator columns starting at `col0` (raw fp32 bits in `r`).  Covers every
// epilogue except the two lm-head ones, which keep running state across the chunks of a tile.
// `ncols` (32, or 16 for the last chunk of a tile width that is not a multiple of 32) clips the chunk at the tile
// edge; columns at or beyond p.N are never written either.
__device__ __forceinline__ void gemm_store_chunk(const GemmParams& p, int row, int col0, const uint32_t (&r)[32],
                                                 int ncols = 32) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
  if (p.epi == kEpiBf16 || (p.epi == kEpiSwiGLU && p.C != nullptr)) {
    if (p.bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
    }
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q * 8 < ncols && col0 + q * 8 < p.N) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        *reinterpret_cast<uint4*>(dst + q * 8) = o;
      }
    }
  }
  if (p.epi == kEpiSwiGLU) {
    __nv_bfloat16* dst =
        static_cast<__nv_bfloat16*>(p.C2) + static_cast<long long>(row) * p.ldc2 + (col0 >> 1);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      if (q * 16 < ncols && col0 + q * 16 < p.N) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = silu_f(v[q * 16 + 2 * j]) * v[q * 16 + 2 * j + 1];
        uint4 o;
        o.x = pack_bf16x2(a[0], a[1]);
        o.y = pack_bf16x2(a[2], a[3]);
        o.z = pack_bf16x2(a[4], a[5]);
        o.w = pack_bf16x2(a[6], a[7]);
        *reinterpret_cast<uint4*>(dst + q * 8) = o;
      }
    }
  } else if (p.epi == kEpiF32 || p.epi == kEpiF32Accum) {
    float* dst = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q * 4 < ncols && col0 + q * 4 < p.N) {
        float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        if (p.epi == kEpiF32Accum) {
          const float4 old = *reinterpret_cast<const float4*>(dst + q * 4);
          o.x += old.x;
          o.y += old.y;
          o.z += old.z;
          o.w += old.w;
        }
        *reinterpret_cast<float4*>(dst + q * 4) = o;
      }
    }
  } else if (p.epi == kEpiF32AtomicPeer) {
    const int owner = min(row / p.rows_per_rank, p.world - 1);
    float* dst = static_cast<float*>(p.c_peers[owner]) +
                 static_cast<long long>(row - owner * p.rows_per_rank) * p.ldc + col0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q * 4 < ncols && col0 + q * 4 < p.N)
        atomicAdd(reinterpret_cast<float4*>(dst + q * 4),
                  make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
    }
  } else if (p.epi == kEpiBf16ScatterPeer) {
    const int2 to = p.row_map[row];
    if (to.x >= p.world || to.y < 0) {
      atomicCAS(p.status, 0, kBadRouting);
    } else if (to.x >= 0) {
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c_peers[to.x]) + static_cast<long long>(to.y) * p.ldc + col0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (q * 8 < ncols && col0 + q * 8 < p.N) {
          uint4 o;
          o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
          o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
          o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
          o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + q * 8) = o;
        }
      }
    }
  } else if (p.epi == kEpiF32Atomic) {
    float* dst = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (q * 4 < ncols && col0 + q * 4 < p.N)
        atomicAdd(reinterpret_cast<float4*>(dst + q * 4),
                  make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
    }
  }
}

}  // namespace apb
