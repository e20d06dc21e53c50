// Memory-bound kernels of the transformer block: RMSNorm (with fused residual
// add), per-head q/k RMSNorm + rotary embedding, SwiGLU backward, all with
// 16-byte vector accesses so that each byte of the activation crosses HBM once.
// They replace the Liger Triton kernels the reference patches in
// (arctic_platform/model/patches/liger.py:25-36: rope, rms_norm, swiglu).
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const Bf16x8 r = *reinterpret_cast<const Bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  Bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<Bf16x8*>(p) = r;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// y = (x [+ res]) * rstd * w ; optionally writes the sum back as the new
// residual stream and the per-row rstd for the backward.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // H <= 256 * 8 * 4 = 8192

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int T, int H, float eps,
                   float w_offset, float* __restrict__ x_f32) {
  pdl_entry();
  __shared__ float scratch[32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    float vals[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        if (x_f32) {
          // split-K accumulator: read the fp32 sums and leave zeros behind for the next GEMM
          float4* xp = reinterpret_cast<float4*>(x_f32 + base + v * 8);
          const float4 a = xp[0], b = xp[1];
          vals[i][0] = a.x; vals[i][1] = a.y; vals[i][2] = a.z; vals[i][3] = a.w;
          vals[i][4] = b.x; vals[i][5] = b.y; vals[i][6] = b.z; vals[i][7] = b.w;
          xp[0] = make_float4(0.f, 0.f, 0.f, 0.f);
          xp[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          load8(x + base + v * 8, vals[i]);
        }
        if (res) {
          float r[8];
          load8(res + base + v * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r[j];
        }
        if (res_out) {
          store8(res_out + base + v * 8, vals[i]);
          // the normalised value is computed from the rounded residual so that
          // forward and backward see the same stream
          load8(res_out + base + v * 8, vals[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    ss = block_sum<kNormThreads>(ss, scratch);
    const float rstd = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float wv[8], o[8];
        load8(w + v * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * (wv[j] + w_offset);
        store8(y + base + v * 8, o);
      }
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)) [+ dres], g = dy * w ; dw += sum_t dy * xhat
// NV = 8-element vectors per thread (registers scale with it, so narrow rows keep more CTAs per SM).
template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 1 ? 3 : (NV <= 2 ? 2 : 1))
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int T, int H, float w_offset) {
  constexpr int kNormMaxVec = NV;  // shadows the file-level bound inside this kernel
  __shared__ float scratch[32];
  const int nvec = H / 8;
  float dw_acc[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;
  float wv[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      load8(w + v * 8, wv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[i][j] += w_offset;
    }
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float g[kNormMaxVec][8], xh[kNormMaxVec][8], rr[kNormMaxVec][8];
    float dot = 0.f;
    // all three inputs of the row are requested before the block-wide reduction: the upstream residual gradient
    // used to be loaded after it, a second full memory latency per row
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float d[8];
        load8(dy + base + v * 8, d);
        load8(x + base + v * 8, xh[i]);
        if (dres) load8(dres + base + v * 8, rr[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          g[i][j] = d[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
          dw_acc[i][j] += d[j] * xh[i][j];
        }
      }
    }
    dot = block_sum<kNormThreads>(dot, scratch) / H;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot) + (dres ? rr[i][j] : 0.f);
        store8(dx + base + v * 8, o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + v * 8 + j, dw_acc[i][j]);
      }
    }
  }
}

// N consecutive bf16 (N = 1, 2 or 4) as one 2-, 4- or 8-byte access.
template <int N>
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&out)[N]) {
  if constexpr (N == 1) {
    out[0] = __bfloat162float(p[0]);
  } else if constexpr (N == 2) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    out[0] = f.x;
    out[1] = f.y;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    out[0] = f0.x;
    out[1] = f0.y;
    out[2] = f1.x;
    out[3] = f1.y;
  }
}
template <int N>
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[N]) {
  if constexpr (N == 1) {
    p[0] = __float2bfloat16(v[0]);
  } else if constexpr (N == 2) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
  } else {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}

// ------------------------------------------------------- q/k norm + rotary
// One warp per (token, head); head_dim D in {64, 128, 256}; rotate-half RoPE on
// the first `rot` dims with cos/sin tables [max_pos, rot/2] fp32.
// Input rows: qkv[t] = [q heads | k heads | v heads]; outputs q_out[T,Hq,D],
// k_out[T,Hkv,D].  wq/wk may be null (no per-head norm, rstd := 1).
template <int D>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_qkv,
                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       const int* __restrict__ pos, __nv_bfloat16* __restrict__ q_out,
                       __nv_bfloat16* __restrict__ k_out, int T, int Hq, int Hkv, int rot, float eps) {
  constexpr int E = D / 32;  // elements per lane
  const int lane = threadIdx.x & 31;
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int heads = Hq + Hkv;
  if (gw >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int h = static_cast<int>(gw % heads);
  const bool is_q = h < Hq;
  const __nv_bfloat16* src = qkv + t * ld_qkv + static_cast<long long>(h) * D;
  const __nv_bfloat16* w = is_q ? wq : wk;
  __nv_bfloat16* dst = is_q ? q_out + (static_cast<long long>(t) * Hq + h) * D
                            : k_out + (static_cast<long long>(t) * Hkv + (h - Hq)) * D;
  // lane owns elements [lane*E/2 .. ) of the first half and the matching ones of the second half,
  // so a rotate-half pair (i, i + D/2) sits in one lane.
  constexpr int E2 = E / 2;
  float a[E2], b[E2];
#pragma unroll
  for (int j = 0; j < E2; ++j) {
    a[j] = __bfloat162float(src[lane * E2 + j]);
    b[j] = __bfloat162float(src[D / 2 + lane * E2 + j]);
  }
  float rstd = 1.f;
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < E2; ++j) ss += a[j] * a[j] + b[j] * b[j];
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + eps);
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      a[j] *= rstd * __bfloat162float(w[lane * E2 + j]);
      b[j] *= rstd * __bfloat162float(w[D / 2 + lane * E2 + j]);
    }
  }
  const int p = pos[t];
  const int half = rot / 2;
#pragma unroll
  for (int j = 0; j < E2; ++j) {
    const int i = lane * E2 + j;  // index inside the first half of the head
    float oa = a[j], ob = b[j];
    if (rot == D) {
      const float c = cos_t[static_cast<long long>(p) * half + i], s = sin_t[static_cast<long long>(p) * half + i];
      oa = a[j] * c - b[j] * s;
      ob = b[j] * c + a[j] * s;
    }
    dst[i] = __float2bfloat16(oa);
    dst[D / 2 + i] = __float2bfloat16(ob);
  }
}

// Backward of the above: dq/dk (post-rotary grads) -> d(raw q/k) written into
// dqkv rows (same layout as qkv), dwq/dwk accumulated in fp32.
// D / 16 lanes share one (token, head) item, so a warp works on 32 / (D / 16) items at a time with 16-byte loads
// (8 elements of each half of the head per lane): four times the bytes in flight per warp of a one-item-per-warp
// walk, whose 4-byte loads and position -> cos/sin load chain left the kernel at an eighth of the memory bandwidth.
// Weight gradients are summed over the lane groups, then over the CTA in shared memory, before one atomic per
// element and CTA.
template <int D>
__global__ void __launch_bounds__(256, 2)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_qkv,
                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                       const int* __restrict__ pos, const __nv_bfloat16* __restrict__ dq,
                       const __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dqkv, long long ld_dqkv,
                       float* __restrict__ dwq, float* __restrict__ dwk, int T, int Hq, int Hkv, int rot,
                       float eps) {
  constexpr int LPI = D / 16;       // lanes per item
  constexpr int IPW = 32 / LPI;     // items per warp and pass
  __shared__ float dw_s[2][D];
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPI, grp = lane / LPI;
  const int heads = Hq + Hkv;
  const long long nwarps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&dw_s[0][0])[i] = 0.f;
  __syncthreads();
  const bool has_w = wq != nullptr;
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int half = rot / 2;
  auto group_sum = [&](float v) {
#pragma unroll
    for (int o = LPI / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  };
  // The q heads first, then the k heads: each pass spreads its own items evenly over all warps (balanced whatever
  // the GQA ratio) and needs only its own weight and weight-gradient registers.
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    const int nh = c == 0 ? Hq : Hkv;
    const int h0 = c == 0 ? 0 : Hq;
    const __nv_bfloat16* w = c == 0 ? wq : wk;
    const __nv_bfloat16* gsrc = c == 0 ? dq : dk;
    float dwa[8], dwb[8], wa[8], wb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dwa[j] = dwb[j] = 0.f;
      wa[j] = wb[j] = 1.f;
    }
    if (w) {
      load8(w + sub * 8, wa);
      load8(w + D / 2 + sub * 8, wb);
    }
    const long long items = static_cast<long long>(T) * nh;
    for (long long base = gw * IPW; base < items; base += nwarps_total * IPW) {
      const long long it = base + grp;
      const bool valid = it < items;                     // the shuffles below need every lane of the warp
      const long long itc = valid ? it : items - 1;
      const int t = static_cast<int>(itc / nh);
      const int h = static_cast<int>(itc % nh);
      const __nv_bfloat16* src = qkv + t * ld_qkv + static_cast<long long>(h0 + h) * D;
      const __nv_bfloat16* g = gsrc + (static_cast<long long>(t) * nh + h) * D;
      __nv_bfloat16* dst = dqkv + t * ld_dqkv + static_cast<long long>(h0 + h) * D;
      const int p = pos[t];
      float ga[8], gb[8], xa[8], xb[8];
      load8(g + sub * 8, ga);
      load8(g + D / 2 + sub * 8, gb);
      load8(src + sub * 8, xa);
      load8(src + D / 2 + sub * 8, xb);
      if (rot == D) {
        const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<long long>(p) * half + sub * 8);
        const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<long long>(p) * half + sub * 8);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float da = ga[j], db = gb[j];
          ga[j] = da * cs[j] + db * sn[j];  // transpose of the rotation
          gb[j] = db * cs[j] - da * sn[j];
        }
      }
      if (has_w) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += xa[j] * xa[j] + xb[j] * xb[j];
        ss = group_sum(ss);
        const float rstd = rsqrtf(ss / D + eps);
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xa[j] *= rstd;
          xb[j] *= rstd;
          if (valid) {
            dwa[j] += ga[j] * xa[j];
            dwb[j] += gb[j] * xb[j];
          }
          ga[j] *= wa[j];
          gb[j] *= wb[j];
          dot += ga[j] * xa[j] + gb[j] * xb[j];
        }
        dot = group_sum(dot) / D;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ga[j] = rstd * (ga[j] - xa[j] * dot);
          gb[j] = rstd * (gb[j] - xb[j] * dot);
        }
      }
      if (valid) {
        store8(dst + sub * 8, ga);
        store8(dst + D / 2 + sub * 8, gb);
      }
    }
    if (has_w) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = dwa[j], b2 = dwb[j];
#pragma unroll
        for (int o = LPI; o < 32; o <<= 1) {             // over the lane groups of the warp
          a += __shfl_xor_sync(0xffffffffu, a, o);
          b2 += __shfl_xor_sync(0xffffffffu, b2, o);
        }
        if (grp == 0) {
          atomicAdd(&dw_s[c][sub * 8 + j], a);
          atomicAdd(&dw_s[c][D / 2 + sub * 8 + j], b2);
        }
      }
    }
  }
  if (has_w) {
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
      float* dwp = i < D ? dwq : dwk;
      if (dwp) atomicAdd(dwp + (i % D), (&dw_s[0][0])[i]);
    }
  }
}

// SwiGLU on fp32 split-K sums: acc [T, 2I] interleaved (gate, up) -> act [T, I] bf16; acc is reset to zero.
// One thread handles four outputs (eight inputs, two 16-byte loads).
__global__ void swiglu_f32in_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ act, long long n_quads) {
  pdl_entry();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_quads;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4* p = reinterpret_cast<float4*>(acc + i * 8);
    const float4 x = p[0], y = p[1];
    p[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    p[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float o0 = x.x / (1.f + __expf(-x.x)) * x.y;
    const float o1 = x.z / (1.f + __expf(-x.z)) * x.w;
    const float o2 = y.x / (1.f + __expf(-y.x)) * y.y;
    const float o3 = y.z / (1.f + __expf(-y.z)) * y.w;
    uint2 out;
    *reinterpret_cast<__nv_bfloat162*>(&out.x) = __floats2bfloat162_rn(o0, o1);
    *reinterpret_cast<__nv_bfloat162*>(&out.y) = __floats2bfloat162_rn(o2, o3);
    *reinterpret_cast<uint2*>(act + i * 4) = out;
  }
}

// --------------------------------------------------------------- SwiGLU
// Interleaved layout: gu[t, 2j] = gate_j, gu[t, 2j+1] = up_j.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                  long long n_pairs8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_pairs8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], b[8], o[8];
    load8(gu + i * 16, a);
    load8(gu + i * 16 + 8, b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j] = a[2 * j] / (1.f + __expf(-a[2 * j])) * a[2 * j + 1];
      o[4 + j] = b[2 * j] / (1.f + __expf(-b[2 * j])) * b[2 * j + 1];
    }
    store8(act + i * 8, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, long long n_pairs8) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_pairs8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float a[8], b[8], d[8], oa[8], ob[8];
    load8(gu + i * 16, a);
    load8(gu + i * 16 + 8, b);
    load8(dact + i * 8, d);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      {
        const float g = a[2 * j], u = a[2 * j + 1], s = 1.f / (1.f + __expf(-g));
        oa[2 * j] = d[j] * u * s * (1.f + g * (1.f - s));
        oa[2 * j + 1] = d[j] * g * s;
      }
      {
        const float g = b[2 * j], u = b[2 * j + 1], s = 1.f / (1.f + __expf(-g));
        ob[2 * j] = d[4 + j] * u * s * (1.f + g * (1.f - s));
        ob[2 * j + 1] = d[4 + j] * g * s;
      }
    }
    store8(dgu + i * 16, oa);
    store8(dgu + i * 16 + 8, ob);
  }
}

}  // namespace apb

// ---------------------------------------------------------------------------
extern "C" {
using namespace apb;

int apb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd, int T,
                    int H, float eps, float w_offset, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || H > kNormThreads * 8 * kNormMaxVec) return kBadArgument;
  const int grid = T < apb::sm_count() * 8 ? T : apb::sm_count() * 8;
  return static_cast<int>(launch_kernel(rmsnorm_fwd_kernel, dim3(grid), dim3(kNormThreads), 0, s,
                                        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
                                        static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
                                        static_cast<__nv_bfloat16*>(res_out), rstd, T, H, eps, w_offset,
                                        static_cast<float*>(nullptr)));
}

// Same as apb_rmsnorm_fwd with the input taken from an fp32 buffer (split-K GEMM sums) that is reset to
// zero as it is read; res_out is required (it receives x + res in bf16, or x alone when res is null).
int apb_rmsnorm_fwd_f32in(float* x_f32, const void* res, const void* w, void* y, void* res_out, int T, int H, float eps,
                          float w_offset, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || H > kNormThreads * 8 * kNormMaxVec || !res_out) return kBadArgument;
  const int grid = T < apb::sm_count() * 8 ? T : apb::sm_count() * 8;
  return static_cast<int>(launch_kernel(rmsnorm_fwd_kernel, dim3(grid), dim3(kNormThreads), 0, s,
                                        static_cast<const __nv_bfloat16*>(nullptr),
                                        static_cast<const __nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(w),
                                        static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(res_out),
                                        static_cast<float*>(nullptr), T, H, eps, w_offset, x_f32));
}

// dw (fp32 [H]) is accumulated into; the caller zeroes it.
int apb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw, int T, int H, float w_offset, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || H > kNormThreads * 8 * kNormMaxVec) return kBadArgument;
  const int nv = (H / 8 + kNormThreads - 1) / kNormThreads;
  const int per_sm = nv <= 1 ? 3 : (nv <= 2 ? 2 : 1);
  const int grid = T < apb::sm_count() * per_sm ? T : apb::sm_count() * per_sm;
#define APB_NORM_BWD(NV)                                                                                     \
  rmsnorm_bwd_kernel<NV><<<grid, kNormThreads, 0, s>>>(                                                       \
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),                            \
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),                    \
      static_cast<__nv_bfloat16*>(dx), dw, T, H, w_offset)
  if (nv <= 1) APB_NORM_BWD(1);
  else if (nv <= 2) APB_NORM_BWD(2);
  else APB_NORM_BWD(4);
#undef APB_NORM_BWD
  return static_cast<int>(cudaGetLastError());
}

int apb_qknorm_rope_fwd(const void* qkv, long long ld_qkv, const void* wq, const void* wk, const float* cos_t,
                        const float* sin_t, const int* pos, void* q_out, void* k_out, int T, int Hq, int Hkv,
                        int D, int rot, float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  if (rot != 0 && rot != D) return kBadArgument;
  const long long warps = static_cast<long long>(T) * (Hq + Hkv);
  const int grid = static_cast<int>((warps * 32 + 255) / 256);
#define APB_LAUNCH_QK(DD)                                                                                   \
  qknorm_rope_fwd_kernel<DD><<<grid, 256, 0, s>>>(                                                          \
      static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<const __nv_bfloat16*>(wq),               \
      static_cast<const __nv_bfloat16*>(wk), cos_t, sin_t, pos, static_cast<__nv_bfloat16*>(q_out),        \
      static_cast<__nv_bfloat16*>(k_out), T, Hq, Hkv, rot, eps)
  if (D == 128) APB_LAUNCH_QK(128);
  else if (D == 64) APB_LAUNCH_QK(64);
  else if (D == 256) APB_LAUNCH_QK(256);
  else return kBadArgument;
#undef APB_LAUNCH_QK
  return static_cast<int>(cudaGetLastError());
}

// dwq/dwk (fp32 [D]) are accumulated into; the caller zeroes them.  The v part
// of dqkv is not touched (the attention backward writes dv there directly).
int apb_qknorm_rope_bwd(const void* qkv, long long ld_qkv, const void* wq, const void* wk, const float* cos_t,
                        const float* sin_t, const int* pos, const void* dq, const void* dk, void* dqkv,
                        long long ld_dqkv, float* dwq, float* dwk, int T, int Hq, int Hkv, int D, int rot,
                        float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  if (rot != 0 && rot != D) return kBadArgument;
  const int grid = apb::sm_count() * 2;       // two resident CTAs per SM, each walks its share of the items
#define APB_LAUNCH_QKB(DD)                                                                                  \
  qknorm_rope_bwd_kernel<DD><<<grid, 256, 0, s>>>(                                                          \
      static_cast<const __nv_bfloat16*>(qkv), ld_qkv, static_cast<const __nv_bfloat16*>(wq),               \
      static_cast<const __nv_bfloat16*>(wk), cos_t, sin_t, pos, static_cast<const __nv_bfloat16*>(dq),     \
      static_cast<const __nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dqkv), ld_dqkv, dwq, dwk, T, Hq,  \
      Hkv, rot, eps)
  if (D == 128) APB_LAUNCH_QKB(128);
  else if (D == 64) APB_LAUNCH_QKB(64);
  else if (D == 256) APB_LAUNCH_QKB(256);
  else return kBadArgument;
#undef APB_LAUNCH_QKB
  return static_cast<int>(cudaGetLastError());
}

int apb_swiglu_f32in(float* acc, void* act, long long T, long long I, cudaStream_t s) {
  if (I % 4) return kBadArgument;
  const long long n = T * I / 4;
  if (n <= 0) return 0;
  const int grid = static_cast<int>(n / 256 + 1 < apb::sm_count() * 16 ? n / 256 + 1 : apb::sm_count() * 16);
  return static_cast<int>(launch_kernel(swiglu_f32in_kernel, dim3(grid), dim3(256), 0, s, acc,
                                        static_cast<__nv_bfloat16*>(act), n));
}
int apb_swiglu_fwd(const void* gu, void* act, long long T, long long I, cudaStream_t s) {
  if (I % 8) return kBadArgument;
  const long long n = T * I / 8;
  if (n <= 0) return 0;
  const int grid = static_cast<int>(n / 256 + 1 < apb::sm_count() * 16 ? n / 256 + 1 : apb::sm_count() * 16);
  swiglu_fwd_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(act), n);
  return static_cast<int>(cudaGetLastError());
}
int apb_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long T, long long I, cudaStream_t s) {
  if (I % 8) return kBadArgument;
  const long long n = T * I / 8;
  if (n <= 0) return 0;
  const int grid = static_cast<int>(n / 256 + 1 < apb::sm_count() * 16 ? n / 256 + 1 : apb::sm_count() * 16);
  swiglu_bwd_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gu),
                                         static_cast<const __nv_bfloat16*>(dact),
                                         static_cast<__nv_bfloat16*>(dgu), n);
  return static_cast<int>(cudaGetLastError());
}
}
