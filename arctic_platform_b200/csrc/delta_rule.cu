// Gated delta rule (the linear-attention layers of the Qwen3.5 / Qwen3-Next hybrids): the sequential part of the
// chunked algorithm as ONE kernel.
//
// The chunked form splits a sequence into chunks of C = 64 tokens.  Everything that does not depend on the carried
// state S [Dk, Dv] -- the decay matrices, the triangular solve of the in-chunk corrections and the operands below --
// is batched over all chunks at once by the caller (large matmuls).  What is left is a recurrence over the chunks,
//     u_n = U_n - W_n S                    [C, Dv]   value corrections given the carried state
//     o_n = Qd_n S + QK_n u_n              [C, Dv]   outputs of the chunk
//     S   = e_n S + Kd_n^T u_n             [Dk, Dv]  state after the chunk
// with small operands (W, Qd, Kd [C, Dk], QK [C, C], U [C, Dv], e scalar).  Issued as library calls it is five tiny
// launches per chunk (thousands per layer); here one CTA owns one (head, 32-column slice of Dv), keeps its slice of
// S in shared memory for the whole sequence and walks the chunks, so the recurrence costs one launch.  The columns of
// S evolve independently, which is what makes the Dv slices independent CTAs.  fp32 throughout (CUDA cores: the
// products are 64 x 128 x 32 -- latency, not throughput, decides).  The reference takes this recurrence from the
// `fla` kernels (arctic_platform/model/implementations/qwen35/models/qwen3_5_moe/modeling_qwen3_5_moe.py:247-349).
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

constexpr int kDrThreads = 256;
constexpr int kDrC = 64;    // chunk length
constexpr int kDrBV = 32;   // Dv columns per CTA (= lanes of a warp)

struct DeltaScanParams {
  const float* u_local;   // [H, N, C, Dv]
  const float* w_state;   // [H, N, C, Dk]
  const float* q_dec;     // [H, N, C, Dk]
  const float* qk;        // [H, N, C, C]
  const float* k_dec;     // [H, N, C, Dk]
  const float* e_end;     // [H, N]
  const float* s0;        // [H, Dk, Dv] or null (zeros)
  float* out;             // [H, N, C, Dv]
  float* s_out;           // [H, Dk, Dv]
  int H, N, Dk, Dv;
};

// rows [C or Dk] x k-extent products with one output column per lane; each warp owns every 8th row, four at a time
template <int kMaxDk>
__global__ void __launch_bounds__(kDrThreads)
delta_rule_scan_kernel(const DeltaScanParams p) {
  extern __shared__ float sm[];
  const int Dk = p.Dk;
  float* S = sm;                           // [Dk][32]
  float* A = S + kMaxDk * kDrBV;           // [64][Dk] staging: W, then Qd, then Kd
  float* QK = A + kDrC * kMaxDk;           // [64][64]
  float* U = QK + kDrC * kDrC;             // [64][32] u_local, then u
  const int h = blockIdx.x, v0 = blockIdx.y * kDrBV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = v0 + lane;
  const bool col_ok = col < p.Dv;
  for (int i = threadIdx.x; i < Dk * kDrBV; i += kDrThreads) {
    const int k = i >> 5, c = i & 31;
    S[i] = (p.s0 && v0 + c < p.Dv) ? p.s0[(static_cast<long long>(h) * Dk + k) * p.Dv + v0 + c] : 0.f;
  }
  __syncthreads();
  auto load_rows = [&](float* dst, const float* src, int n_floats) {      // contiguous [rows, width] block
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (int i = threadIdx.x; i < n_floats / 4; i += kDrThreads) d4[i] = s4[i];
  };
  for (int n = 0; n < p.N; ++n) {
    const long long cn = static_cast<long long>(h) * p.N + n;
    // ---- u = U - W S
    load_rows(A, p.w_state + cn * kDrC * Dk, kDrC * Dk);
    for (int i = threadIdx.x; i < kDrC * kDrBV; i += kDrThreads) {
      const int r = i >> 5, c = i & 31;
      U[i] = (v0 + c < p.Dv) ? p.u_local[(cn * kDrC + r) * p.Dv + v0 + c] : 0.f;
    }
    __syncthreads();
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < Dk; k += 4) {
      const float s0 = S[k * kDrBV + lane], s1 = S[(k + 1) * kDrBV + lane];
      const float s2 = S[(k + 2) * kDrBV + lane], s3 = S[(k + 3) * kDrBV + lane];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 a = *reinterpret_cast<const float4*>(&A[(warp + 8 * j) * Dk + k]);   // same address in all lanes
        acc[j] += a.x * s0 + a.y * s1 + a.z * s2 + a.w * s3;
      }
    }
    __syncthreads();                       // everybody has read W (A is reloaded next) and the old U rows
#pragma unroll
    for (int j = 0; j < 8; ++j) U[(warp + 8 * j) * kDrBV + lane] -= acc[j];
    // ---- o = Qd S + QK u
    load_rows(A, p.q_dec + cn * kDrC * Dk, kDrC * Dk);
    load_rows(QK, p.qk + cn * kDrC * kDrC, kDrC * kDrC);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < Dk; k += 4) {
      const float s0 = S[k * kDrBV + lane], s1 = S[(k + 1) * kDrBV + lane];
      const float s2 = S[(k + 2) * kDrBV + lane], s3 = S[(k + 3) * kDrBV + lane];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 a = *reinterpret_cast<const float4*>(&A[(warp + 8 * j) * Dk + k]);   // same address in all lanes
        acc[j] += a.x * s0 + a.y * s1 + a.z * s2 + a.w * s3;
      }
    }
    for (int k = 0; k < kDrC; k += 4) {
      const float u0 = U[k * kDrBV + lane], u1 = U[(k + 1) * kDrBV + lane];
      const float u2 = U[(k + 2) * kDrBV + lane], u3 = U[(k + 3) * kDrBV + lane];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 a = *reinterpret_cast<const float4*>(&QK[(warp + 8 * j) * kDrC + k]);
        acc[j] += a.x * u0 + a.y * u1 + a.z * u2 + a.w * u3;
      }
    }
    if (col_ok) {
#pragma unroll
      for (int j = 0; j < 8; ++j) p.out[(cn * kDrC + warp + 8 * j) * p.Dv + col] = acc[j];
    }
    __syncthreads();                       // Qd has been read by everybody
    // ---- S = e S + Kd^T u   (row k of S needs column k of Kd: Kd is staged as [64][Dk] and read transposed)
    load_rows(A, p.k_dec + cn * kDrC * Dk, kDrC * Dk);
    __syncthreads();
    const float e = p.e_end[cn];
    for (int k0 = warp * 4; k0 < Dk; k0 += 8 * 4) {      // four consecutive state rows per warp and pass
      float sa[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < kDrC; ++c) {
        const float u = U[c * kDrBV + lane];
        const float4 a = *reinterpret_cast<const float4*>(&A[c * Dk + k0]);
        sa[0] += a.x * u;
        sa[1] += a.y * u;
        sa[2] += a.z * u;
        sa[3] += a.w * u;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) S[(k0 + j) * kDrBV + lane] = S[(k0 + j) * kDrBV + lane] * e + sa[j];
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < Dk * kDrBV; i += kDrThreads) {
    const int k = i >> 5, c = i & 31;
    if (v0 + c < p.Dv) p.s_out[(static_cast<long long>(h) * Dk + k) * p.Dv + v0 + c] = S[i];
  }
}

}  // namespace apb

extern "C" {

// All tensors fp32, contiguous, 16-byte aligned.  Chunk length 64; Dk a multiple of 4 and at most 256; any Dv.
// s0 may be null (zero initial state).  One launch for the whole sequence of every head.
int apb_delta_rule_scan(const float* u_local, const float* w_state, const float* q_dec, const float* qk,
                        const float* k_dec, const float* e_end, const float* s0, float* out, float* s_out, int H,
                        int N, int Dk, int Dv, cudaStream_t s) {
  using namespace apb;
  if (H <= 0 || N < 0 || Dv <= 0) return 0;
  if (!u_local || !w_state || !q_dec || !qk || !k_dec || !e_end || !out || !s_out || Dk < 4 || Dk > 256 || (Dk % 4))
    return kBadArgument;
  DeltaScanParams p{u_local, w_state, q_dec, qk, k_dec, e_end, s0, out, s_out, H, N, Dk, Dv};
  const dim3 grid(H, (Dv + kDrBV - 1) / kDrBV);
  if (Dk <= 128) {
    constexpr int kMax = 128;
    const int smem = (kMax * kDrBV + kDrC * kMax + kDrC * kDrC + kDrC * kDrBV) * 4;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(delta_rule_scan_kernel<kMax>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[dev & 63] = true;
    }
    delta_rule_scan_kernel<kMax><<<grid, kDrThreads, smem, s>>>(p);
  } else {
    constexpr int kMax = 256;
    const int smem = (kMax * kDrBV + kDrC * kMax + kDrC * kDrC + kDrC * kDrBV) * 4;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(delta_rule_scan_kernel<kMax>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[dev & 63] = true;
    }
    delta_rule_scan_kernel<kMax><<<grid, kDrThreads, smem, s>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}
}
