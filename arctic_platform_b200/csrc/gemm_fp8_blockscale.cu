// Block-scaled fp8 (e4m3) GEMM for the sampler: C[M,N] (bf16) = (A_q * sa) (W_q * sw)^T.
//
//   A_q [M, K] e4m3 with one fp32 scale per (row, 128-wide K block):      sa [M, K/128]
//   W_q [N, K] e4m3 with one fp32 scale per (128 x 128) block:            sw [ceil(N/128), K/128]
//
// The weights are what the trainer -> sampler sync produces (quant_fp8_block128_kernel); activations are quantised
// per token by quant_act_fp8_kernel below.  One CTA per 128 x 128 output tile; per 128-wide K block the tensor
// core (tcgen05.mma kind::f8f6f4, 4 instructions of K = 32) produces the UNSCALED partial product in one of two
// TMEM accumulators, and the four epilogue warps fold it into fp32 registers with the product of the two block
// scales while the next block's MMAs run into the other accumulator.  Operands arrive by TMA (128-byte swizzle: a
// row of a K block is exactly 128 bytes of fp8).  Decode-shaped problems are bound by the weight stream, which
// this format halves.  The reference serves fp8 through vLLM (arctic_platform/common/ray_server.py:375).
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct Fp8GemmParams {
  int M, N, K;
  const float* sa;   // [M, KB]
  const float* sw;   // [ceil(N/128), KB]
  __nv_bfloat16* C;
  long long ldc;
  int* status;
};

constexpr int kF8Threads = 192;
constexpr int kF8Stages = 4;
constexpr int kF8Tile = 128 * 128;                       // bytes of one A or B stage (fp8)
constexpr int kF8Smem = kF8Stages * 2 * kF8Tile + 1024 + 256;

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_bs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const Fp8GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kF8Stages * 2 * kF8Tile);
  uint64_t* empty = full + kF8Stages;
  uint64_t* tfull = empty + kF8Stages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + 127) / 128;
  const int m0 = (blockIdx.x / tiles_n) * 128, nt = blockIdx.x % tiles_n, n0 = nt * 128;
  const int KB = p.K / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < KB && ok; ++kb) {
        const int s = kb % kF8Stages;
        if (!mbar_wait(&empty[s], ((kb / kF8Stages) & 1) ^ 1, p.status, kTimeoutEmpty)) {
          ok = false;
          break;
        }
        uint8_t* sa = smem + s * 2 * kF8Tile;
        mbar_expect_tx(&full[s], 2 * kF8Tile);
        tma_load_2d(sa, &tma_a, &full[s], kb * 128, m0);
        tma_load_2d(sa + kF8Tile, &tma_b, &full[s], kb * 128, n0);
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_e4m3(128, 128);
      bool ok = true;
      for (int kb = 0; kb < KB && ok; ++kb) {
        const int s = kb % kF8Stages, buf = kb & 1;
        if (!mbar_wait(&tempty[buf], ((kb >> 1) & 1) ^ 1, p.status, kTimeoutTmemEmpty) ||
            !mbar_wait(&full[s], (kb / kF8Stages) & 1, p.status, kTimeoutFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * 2 * kF8Tile), sb = sa + kF8Tile;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 32 fp8 elements = 32 bytes per step inside the 128-byte swizzled row
          umma_e4m3_ss(tmem_base + buf * 128, umma_smem_desc(sa + k * 32, 0, 1024), umma_smem_desc(sb + k * 32, 0, 1024),
                       idesc, k > 0 ? 1u : 0u);
        tc_commit(&empty[s]);
        tc_commit(&tfull[buf]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    const bool row_ok = row < p.M;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.f;
    bool ok = true;
    for (int kb = 0; kb < KB; ++kb) {
      const int buf = kb & 1;
      if (!mbar_wait(&tfull[buf], (kb >> 1) & 1, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float sc = (row_ok ? p.sa[static_cast<long long>(row) * KB + kb] : 0.f) * p.sw[static_cast<long long>(nt) * KB + kb];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + buf * 128 + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(v[i]) * sc;
      }
      tc_fence_before();
      mbar_arrive(&tempty[buf]);
    }
    if (ok && row_ok) {
      __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + n0;
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        if (n0 + q * 8 < p.N) {
          uint4 o;
          o.x = pack_bf16x2(acc[q * 8 + 0], acc[q * 8 + 1]);
          o.y = pack_bf16x2(acc[q * 8 + 2], acc[q * 8 + 3]);
          o.z = pack_bf16x2(acc[q * 8 + 4], acc[q * 8 + 5]);
          o.w = pack_bf16x2(acc[q * 8 + 6], acc[q * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + q * 8) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Per-token activation quantisation: x [M, K] bf16 -> q [M, K] e4m3, scales [M, K/128] (amax / 448 per 128 values).
// One warp per (row, K block); a lane handles four consecutive values.
__global__ void __launch_bounds__(256)
quant_act_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M, int K, uint8_t* __restrict__ q,
                     long long ldq, float* __restrict__ scales) {
  const int KB = K / 128;
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(M) * KB) return;
  const int row = static_cast<int>(gw / KB), kb = static_cast<int>(gw % KB);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + row * ldx + kb * 128 + lane * 4);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(a.y * inv), "f"(a.x * inv));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(b.y * inv), "f"(b.x * inv));
  *reinterpret_cast<uint32_t*>(q + row * ldq + kb * 128 + lane * 4) = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
  if (lane == 0) scales[static_cast<long long>(row) * KB + kb] = scale;
}

}  // namespace apb

extern "C" {

int apb_quant_act_fp8(const void* x, long long ldx, int M, int K, void* q, long long ldq, float* scales,
                      cudaStream_t s) {
  using namespace apb;
  if (M <= 0) return 0;
  if (K % 128 || ldx % 4 || ldq % 4) return kBadArgument;
  const long long warps = static_cast<long long>(M) * (K / 128);
  quant_act_fp8_kernel<<<static_cast<int>((warps * 32 + 255) / 256), 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, M, K, static_cast<uint8_t*>(q), ldq, scales);
  return static_cast<int>(cudaGetLastError());
}

// A_q [M, K] (row stride lda bytes = elements), W_q [N, K] (ldw), scales as described at the top, C [M, N] bf16.
// K % 128 == 0, N % 8 == 0, lda/ldw % 16 == 0, bases 16-byte aligned.
int apb_gemm_fp8_blockscale(const void* Aq, const float* sa, const void* Wq, const float* sw, void* C, int M, int N,
                            int K, long long lda, long long ldw, long long ldc, cudaStream_t stream) {
  using namespace apb;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 128 || N % 8 || lda % 16 || ldw % 16 || ldc % 8) return kBadArgument;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, Aq, 1, static_cast<uint64_t>(M), static_cast<uint64_t>(K), lda, 128, 128);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tb, Wq, 1, static_cast<uint64_t>(N), static_cast<uint64_t>(K), ldw, 128, 128);
  if (rc) return 2000 + rc;
  Fp8GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.sa = sa;
  p.sw = sw;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.status = status_device_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_bs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const int tiles = ((M + 127) / 128) * ((N + 127) / 128);
  gemm_fp8_bs_kernel<<<tiles, kF8Threads, kF8Smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}
}
