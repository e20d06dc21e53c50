// Sampler-side kernels: paged KV cache writes, paged (split-KV) decode attention with
// an LSE-weighted merge that also serves forest-cascade decode, and token sampling.
// These take the place of the vLLM / ArcticInference kernels the reference drives
// through ReplicaPool (arctic_platform/common/ray_server.py:197-201,921-933; forest
// cascade attention is switched on by `use_fca`, common/utils/server_models.py:123-132).
//
// KV cache layout: [num_pages, Hkv, 16, D] bf16 -- the 16 tokens of one (page, head)
// are one contiguous 4 KB tile (D = 128).
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

constexpr int kPage = 16;

// k, v: [T, Hkv, D] (row stride ld elements); slots[t] = page * 16 + offset, or < 0 to skip.
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ k, long long ldk,
                                      const __nv_bfloat16* __restrict__ v, long long ldv,
                                      const int* __restrict__ slots, __nv_bfloat16* __restrict__ kcache,
                                      __nv_bfloat16* __restrict__ vcache, int T, int Hkv, int D) {
  pdl_entry();
  const int vec_per_row = Hkv * D / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
       i < static_cast<long long>(T) * vec_per_row; i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int e = static_cast<int>(i % vec_per_row) * 8;
    const int slot = slots[t];
    if (slot < 0) continue;
    const int h = e / D, d = e % D;
    const long long dst = ((static_cast<long long>(slot / kPage) * Hkv + h) * kPage + slot % kPage) * D + d;
    *reinterpret_cast<uint4*>(kcache + dst) = *reinterpret_cast<const uint4*>(k + t * ldk + e);
    *reinterpret_cast<uint4*>(vcache + dst) = *reinterpret_cast<const uint4*>(v + t * ldv + e);
  }
}

// Paged decode attention.  One CTA = (query group, kv head, kv split); a query group is
// `nq` consecutive query rows that share one page list (nq = 1: ordinary decode; nq > 1:
// one node of the prefix forest, whose KV is read ONCE for all descendant sequences).
//   q        [Bq, Hq, D]
//   q_start  [G]        first query row of group g;  q_count [G] rows in the group (<= kMaxNq)
//   pages    [G, max_pages]  page ids of the group's KV range;  kv_len [G] tokens in it
//   out_o    [Bq, Hq, splits, D] fp32 partial numerators (un-normalised), out_ml [Bq,Hq,splits,2] (max, sum)
// Scores use base-2 exponentials with scale_log2 = softmax_scale * log2(e).
constexpr int kDecThreads = 128;
constexpr int kMaxNq = 16;

template <int R, int D>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const int* __restrict__ q_start,
                    const int* __restrict__ q_count, const int* __restrict__ pages, int max_pages,
                    const int* __restrict__ kv_len, const __nv_bfloat16* __restrict__ kcache,
                    const __nv_bfloat16* __restrict__ vcache, float* __restrict__ out_o, float* __restrict__ out_ml,
                    int Hq, int Hkv, int splits, float scale_log2) {
  pdl_entry();
  static_assert(D == 128, "head_dim 128");
  const int g = blockIdx.x / Hkv;
  const int kvh = blockIdx.x % Hkv;
  const int split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = q_count[g];
  const int qs = q_start[g];
  const int len = kv_len[g];
  const int n_pages = (len + kPage - 1) / kPage;
  const int per = (n_pages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(n_pages, p0 + per);

  __shared__ float q_s[R][D];
  __shared__ __align__(16) float p_s[4][R][kPage];
  __shared__ float red_m[4][R], red_l[4][R];
  __shared__ float red_o[4][R][D];

  const int tok = lane & 15, half = lane >> 4;
  for (int qi = 0; qi < nq; ++qi) {
    const int row = qs + qi;
    __syncthreads();
    for (int i = threadIdx.x; i < R * D; i += kDecThreads) {
      const int r = i / D, d = i % D;
      q_s[r][d] = __bfloat162float(q[(static_cast<long long>(row) * Hq + kvh * R + r) * D + d]) * scale_log2;
    }
    __syncthreads();
    float m[R], l[R], acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      m[r] = -INFINITY;
      l[r] = 0.f;
      acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    }
    // K of the page being processed sits in registers; the next page's K and this page's V are
    // requested before the arithmetic so that three pages of loads are in flight per warp.
    uint4 kreg[8];
    {
      const int pi0 = p0 + warp;
      if (pi0 < p1) {
        const int page = pages[static_cast<long long>(g) * max_pages + pi0];
        const __nv_bfloat16* kp = kcache + ((static_cast<long long>(page) * Hkv + kvh) * kPage + tok) * D + half * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) kreg[i] = *reinterpret_cast<const uint4*>(kp + i * 8);
      }
    }
#pragma unroll 1
    for (int pi = p0 + warp; pi < p1; pi += 4) {
      const int page = pages[static_cast<long long>(g) * max_pages + pi];
      uint4 knext[8];
      if (pi + 4 < p1) {
        const int pn = pages[static_cast<long long>(g) * max_pages + pi + 4];
        const __nv_bfloat16* kp = kcache + ((static_cast<long long>(pn) * Hkv + kvh) * kPage + tok) * D + half * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) knext[i] = *reinterpret_cast<const uint4*>(kp + i * 8);
      }
      uint2 vreg[kPage];
      {
        const __nv_bfloat16* vp = vcache + ((static_cast<long long>(page) * Hkv + kvh) * kPage) * D + lane * 4;
#pragma unroll
        for (int t = 0; t < kPage; ++t) vreg[t] = *reinterpret_cast<const uint2*>(vp + t * D);
      }
      float dot[R];
#pragma unroll
      for (int r = 0; r < R; ++r) dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&kreg[i]);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          kf[2 * e] = f.x;
          kf[2 * e + 1] = f.y;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float* qr = &q_s[r][half * 64 + i * 8];
#pragma unroll
          for (int e = 0; e < 8; ++e) dot[r] += kf[e] * qr[e];
        }
      }
      const bool valid = pi * kPage + tok < len;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float s = dot[r] + __shfl_xor_sync(0xffffffffu, dot[r], 16);
        if (!valid) s = -INFINITY;
        float mx = s;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m[r], mx);
        const float pv = valid ? exp2f(s - m_new) : 0.f;
        float ps = pv;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        const float alpha = (m[r] == -INFINITY) ? 0.f : exp2f(m[r] - m_new);
        l[r] = l[r] * alpha + ps;
        m[r] = m_new;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] *= alpha;
        if (half == 0) p_s[warp][r][tok] = pv;
      }
      __syncwarp();
#pragma unroll
      for (int t4 = 0; t4 < kPage / 4; ++t4) {
        float4 pw4[R];  // probabilities of four tokens per head, one 16-byte shared load each
#pragma unroll
        for (int r = 0; r < R; ++r) pw4[r] = *reinterpret_cast<const float4*>(&p_s[warp][r][t4 * 4]);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
          const int t = t4 * 4 + tt;
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vreg[t].x));
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vreg[t].y));
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float pw = tt == 0 ? pw4[r].x : tt == 1 ? pw4[r].y : tt == 2 ? pw4[r].z : pw4[r].w;
            acc[r][0] += pw * a.x;
            acc[r][1] += pw * a.y;
            acc[r][2] += pw * b.x;
            acc[r][3] += pw * b.y;
          }
        }
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 8; ++i) kreg[i] = knext[i];
    }
    // merge the four warps
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (lane == 0) {
        red_m[warp][r] = m[r];
        red_l[warp][r] = l[r];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) red_o[warp][r][lane * 4 + e] = acc[r][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * D; i += kDecThreads) {
      const int r = i / D, d = i % D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_m[w][r]);
      float o = 0.f, ll = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float sc = (red_m[w][r] == -INFINITY) ? 0.f : exp2f(red_m[w][r] - mm);
        o += red_o[w][r][d] * sc;
        ll += red_l[w][r] * sc;
      }
      const long long base = (static_cast<long long>(row) * Hq + kvh * R + r) * splits + split;
      out_o[base * D + d] = o;
      if (d == 0) {
        out_ml[base * 2] = mm;
        out_ml[base * 2 + 1] = ll;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Paged decode on warp-level tensor-core MMAs (m16n8k16): the per-sequence pass.
//
// A decode query group has at most a handful of rows per KV head (R query heads of ONE token), far below the
// 64/128-row tile of the tcgen05 path used for shared prefixes, and the kernel is bound by streaming KV pages, not
// by math.  So: each warp owns every 4th page of the CTA's range, copies K and V pages with cp.async into a
// 3-deep shared-memory ring (XOR-swizzled 16-byte chunks), reads fragments with ldmatrix and runs S = Q K^T and
// O += P V as m16n8k16 MMAs whose 16 rows hold up to 16 / R queries x R heads.  Per page that is 32 MMAs and 16
// ldmatrix instead of ~850 scalar instructions, which leaves the load pipeline as the only limiter.
// Output format is the same un-normalised (numerator, max, sum) partial as the scalar kernel.
// ---------------------------------------------------------------------------
constexpr int kMmaStages = 3;
constexpr int kMmaPageBytes = kPage * 128 * 2;                    // one K or V page of one head
constexpr int kMmaWarpBytes = kMmaStages * 2 * kMmaPageBytes;     // K+V ring of one warp
constexpr int kMmaSmem = 4 * kMmaWarpBytes;                       // 96 KB

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One page (K and V, 4 KB each, contiguous in the cache) -> one ring stage; chunk c of row t lands at
// t * 256 + ((c ^ (t & 7)) * 16) so that the 8 rows of an ldmatrix tile hit 8 different bank groups.
__device__ __forceinline__ void decode_issue_page(uint32_t stage_addr, const __nv_bfloat16* kpage,
                                                  const __nv_bfloat16* vpage, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 32 + lane;  // 16-byte chunk 0..255 of the page
    const int t = c >> 4, col = c & 15;
    const uint32_t off = static_cast<uint32_t>(t * 256 + ((col ^ (t & 7)) << 4));
    cp_async16(stage_addr + off, reinterpret_cast<const uint8_t*>(kpage) + c * 16);
    cp_async16(stage_addr + kMmaPageBytes + off, reinterpret_cast<const uint8_t*>(vpage) + c * 16);
  }
}

__global__ void __launch_bounds__(kDecThreads)
paged_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const int* __restrict__ q_start,
                        const int* __restrict__ q_count, const int* __restrict__ pages, int max_pages,
                        const int* __restrict__ kv_len, const __nv_bfloat16* __restrict__ kcache,
                        const __nv_bfloat16* __restrict__ vcache, float* __restrict__ out_o, float* __restrict__ out_ml,
                        int Hq, int Hkv, int splits, float scale_log2) {
  pdl_entry();
  constexpr int D = 128;
  extern __shared__ __align__(128) uint8_t dec_smem[];
  const int g = blockIdx.x / Hkv;
  const int kvh = blockIdx.x % Hkv;
  const int split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = Hq / Hkv;
  const int nq = q_count[g];
  const int qs = q_start[g];
  const int len = kv_len[g];
  const int n_pages = (len + kPage - 1) / kPage;
  const int per = (n_pages + splits - 1) / splits;
  const int p0 = split * per, p1 = min(n_pages, p0 + per);
  const int* my_pages = pages + static_cast<long long>(g) * max_pages;
  const uint32_t ring = smem_u32(dec_smem) + warp * kMmaWarpBytes;
  const int n_my = (p1 - p0 - warp + 3) / 4;  // pages p0 + warp, p0 + warp + 4, ... (<= 0: none)
  const int q_per_pass = 16 / R;              // queries whose R heads fit the 16 MMA rows
  const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;

  for (int q0 = 0; q0 < nq; q0 += q_per_pass) {
    const int rows_valid = min(q_per_pass, nq - q0) * R;
    // ---- Q fragments (A operand), rows >= rows_valid are zero
    uint32_t qa[8][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int rr = quad_row + 8 * h;
      const bool ok = rr < rows_valid;
      const long long qrow = qs + q0 + rr / R;
      const __nv_bfloat16* qp = q + (qrow * Hq + kvh * R + rr % R) * D + quad_col;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa[ks][h] = ok ? *reinterpret_cast<const uint32_t*>(qp + ks * 16) : 0u;
        qa[ks][2 + h] = ok ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8) : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // ---- prologue: first kMmaStages-1 pages of this warp
#pragma unroll
    for (int j = 0; j < kMmaStages - 1; ++j) {
      if (j < n_my) {
        const long long page = my_pages[p0 + warp + 4 * j];
        const __nv_bfloat16* kp = kcache + (page * Hkv + kvh) * (kPage * D);
        const __nv_bfloat16* vp = vcache + (page * Hkv + kvh) * (kPage * D);
        decode_issue_page(ring + (j % kMmaStages) * 2 * kMmaPageBytes, kp, vp, lane);
      }
      cp_async_commit();
    }
#pragma unroll 1
    for (int j = 0; j < n_my; ++j) {
      {
        const int jn = j + kMmaStages - 1;
        if (jn < n_my) {
          const long long page = my_pages[p0 + warp + 4 * jn];
          const __nv_bfloat16* kp = kcache + (page * Hkv + kvh) * (kPage * D);
          const __nv_bfloat16* vp = vcache + (page * Hkv + kvh) * (kPage * D);
          decode_issue_page(ring + (jn % kMmaStages) * 2 * kMmaPageBytes, kp, vp, lane);
        }
        cp_async_commit();
      }
      cp_async_wait<kMmaStages - 1>();
      __syncwarp();
      const uint32_t ks_addr = ring + (j % kMmaStages) * 2 * kMmaPageBytes;
      const uint32_t vs_addr = ks_addr + kMmaPageBytes;
      // ---- S = Q K^T : two 8-token tiles
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      {
        const int mat = lane >> 3, rowin = lane & 7;
        const int tok = rowin + 8 * (mat >> 1);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int chunk = ks * 2 + (mat & 1);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(ks_addr + tok * 256 + ((chunk ^ (tok & 7)) << 4), b0, b1, b2, b3);
          mma_16816(sc[0], qa[ks], b0, b1);
          mma_16816(sc[1], qa[ks], b2, b3);
        }
      }
      // ---- online softmax for rows quad_row (h = 0) and quad_row + 8 (h = 1)
      const int tok_base = (p0 + warp + 4 * j) * kPage + quad_col;
      uint32_t pa[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && rows_valid <= 8) {  // uniform: the upper 8 rows are padding
          pa[1] = pa[3] = 0u;
          continue;
        }
        float sv[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool valid = tok_base + nt * 8 + e < len;
            sv[nt * 2 + e] = valid ? sc[nt][2 * h + e] * scale_log2 : -INFINITY;
          }
        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[h], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run[h] - m_use);  // m_run = -inf -> 0
        float pv[4], ps = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pv[i] = exp2f(sv[i] - m_use);  // masked: exp2(-inf) = 0
          ps += pv[i];
        }
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run[h] = l_run[h] * alpha + ps;
        m_run[h] = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          o[i][2 * h] *= alpha;
          o[i][2 * h + 1] *= alpha;
        }
        pa[h] = pack_bf16x2(pv[0], pv[1]);
        pa[2 + h] = pack_bf16x2(pv[2], pv[3]);
      }
      // ---- O += P V : sixteen 8-dim tiles, V fragments via transposed ldmatrix
      {
        const int mat = lane >> 3, rowin = lane & 7;
        const int tok = rowin + 8 * (mat & 1);
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          const int chunk = dp * 2 + (mat >> 1);
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(vs_addr + tok * 256 + ((chunk ^ (tok & 7)) << 4), b0, b1, b2, b3);
          mma_16816(o[2 * dp], pa, b0, b1);
          mma_16816(o[2 * dp + 1], pa, b2, b3);
        }
      }
      __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring: reuse it for the cross-warp merge
    float* red_o = reinterpret_cast<float*>(dec_smem);                 // [4][16][D]
    float* red_m = red_o + 4 * 16 * D;                                 // [4][16]
    float* red_l = red_m + 4 * 16;                                     // [4][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int rr = quad_row + 8 * h;
      if ((lane & 3) == 0) {
        red_m[warp * 16 + rr] = m_run[h];
        red_l[warp * 16 + rr] = l_run[h];
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float2 v2 = make_float2(o[i][2 * h], o[i][2 * h + 1]);
        *reinterpret_cast<float2*>(&red_o[(warp * 16 + rr) * D + i * 8 + quad_col]) = v2;
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows_valid * D; i += kDecThreads) {
      const int rr = i / D, d = i % D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red_m[w * 16 + rr]);
      float ov = 0.f, ll = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = red_m[w * 16 + rr];
        const float scw = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
        ov += red_o[(w * 16 + rr) * D + d] * scw;
        ll += red_l[w * 16 + rr] * scw;
      }
      const long long qrow = qs + q0 + rr / R;
      const long long base = ((qrow * Hq + kvh * R + rr % R) * splits + split);
      out_o[base * D + d] = ov;
      if (d == 0) {
        out_ml[base * 2] = mm;
        out_ml[base * 2 + 1] = ll;
      }
    }
    __syncthreads();  // the ring is written again by the next pass
  }
}

// Merges `n_src` sets of partials per (row, head): sets s = 0..n_src-1 are [rows, Hq, splits_s, D] blocks
// given by pointer tables (cascade levels: shared prefix nodes + per-sequence suffix), producing
// normalised bf16 output [rows, Hq, D].  One warp per (row, head).
struct MergeSrc {
  const float* o[4];
  const float* ml[4];
  int splits[4];
  int n;
};
__global__ void decode_merge_kernel(MergeSrc src, const int* __restrict__ row_mask, __nv_bfloat16* __restrict__ out,
                                    float* __restrict__ lse_out, int rows, int Hq, int D) {
  pdl_entry();
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(rows) * Hq) return;
  // bit s of row_mask[row]: source s holds partials of this row (a sequence without a node at some level of the
  // forest has stale data there); null = every source is valid for every row
  const int valid = row_mask ? row_mask[gw / Hq] : 0xF;
  float mm = -INFINITY;
  for (int s = 0; s < src.n; ++s) {
    if (!((valid >> s) & 1)) continue;
    for (int k = 0; k < src.splits[s]; ++k) mm = fmaxf(mm, src.ml[s][(gw * src.splits[s] + k) * 2]);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float ll = 0.f;
  for (int s = 0; s < src.n; ++s)
    for (int k = 0; k < src.splits[s]; ++k) {
      if (!((valid >> s) & 1)) break;
      const long long b = gw * src.splits[s] + k;
      const float m = src.ml[s][b * 2];
      const float sc = (m == -INFINITY) ? 0.f : exp2f(m - mm);
      ll += src.ml[s][b * 2 + 1] * sc;
      const float4 v = *reinterpret_cast<const float4*>(src.o[s] + b * D + lane * 4);
      acc[0] += v.x * sc;
      acc[1] += v.y * sc;
      acc[2] += v.z * sc;
      acc[3] += v.w * sc;
    }
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  uint2 o;
  o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(out + gw * D + lane * 4) = o;
  if (lse_out && lane == 0) lse_out[gw] = ll > 0.f ? (mm + log2f(ll)) * 0.6931471805599453f : -INFINITY;
}

// Decode-step epilogue of the split-K qkv projection: reads the fp32 sums [B, (Hq + 2 Hkv) * D] (and resets them to
// zero for the next step), applies the per-head RMSNorm and rotate-half RoPE to q and k, writes q as bf16 and puts k
// and v straight into their KV-cache slots -- one kernel instead of (bf16 store in the GEMM, norm+RoPE, cache write).
// One warp per (token, head).
template <int D>
__global__ void __launch_bounds__(256)
decode_qkv_post_kernel(float* __restrict__ acc, long long ld_acc, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, const int* __restrict__ pos, const int* __restrict__ slots,
                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kcache,
                       __nv_bfloat16* __restrict__ vcache, int B, int Hq, int Hkv, float eps) {
  pdl_entry();
  constexpr int E2 = D / 64;
  const int lane = threadIdx.x & 31;
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int heads = Hq + 2 * Hkv;
  if (gw >= static_cast<long long>(B) * heads) return;
  const int t = static_cast<int>(gw / heads);
  const int h = static_cast<int>(gw % heads);
  float* src = acc + t * ld_acc + static_cast<long long>(h) * D;
  float a[E2], b[E2];
#pragma unroll
  for (int j = 0; j < E2; ++j) {
    a[j] = src[lane * E2 + j];
    b[j] = src[D / 2 + lane * E2 + j];
    src[lane * E2 + j] = 0.f;
    src[D / 2 + lane * E2 + j] = 0.f;
  }
  const int slot = slots[t];
  const bool is_q = h < Hq, is_k = !is_q && h < Hq + Hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* w = is_q ? wq : wk;
    if (w) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < E2; ++j) ss += a[j] * a[j] + b[j] * b[j];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
      for (int j = 0; j < E2; ++j) {
        a[j] *= rstd * __bfloat162float(w[lane * E2 + j]);
        b[j] *= rstd * __bfloat162float(w[D / 2 + lane * E2 + j]);
      }
    }
    const int p = pos[t];
#pragma unroll
    for (int j = 0; j < E2; ++j) {
      const int i = lane * E2 + j;
      const float c = cos_t[static_cast<long long>(p) * (D / 2) + i], sn = sin_t[static_cast<long long>(p) * (D / 2) + i];
      const float oa = a[j] * c - b[j] * sn, ob = b[j] * c + a[j] * sn;
      a[j] = oa;
      b[j] = ob;
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<long long>(t) * Hq + h) * D;
  } else {
    if (slot < 0) return;  // inactive sequence: nothing enters the cache
    const int hh = is_k ? h - Hq : h - Hq - Hkv;
    __nv_bfloat16* cache = is_k ? kcache : vcache;
    dst = cache + ((static_cast<long long>(slot / kPage) * Hkv + hh) * kPage + slot % kPage) * D;
  }
#pragma unroll
  for (int j = 0; j < E2; ++j) {
    dst[lane * E2 + j] = __float2bfloat16(a[j]);
    dst[D / 2 + lane * E2 + j] = __float2bfloat16(b[j]);
  }
}

// ---------------------------------------------------------------------------- step bookkeeping
// Start of a decode step, one block per slot: the cache slot of the token being fed (page table look-up; -1 for
// an inactive slot) and the token's embedding row copied into the activation buffer.
__global__ void __launch_bounds__(128)
decode_begin_kernel(const int* __restrict__ tokens, const int* __restrict__ pos, const int* __restrict__ active,
                    const int* __restrict__ page_table, int max_pages, const __nv_bfloat16* __restrict__ embed,
                    long long ld_embed, int H, int vocab, int* __restrict__ slots, __nv_bfloat16* __restrict__ x) {
  pdl_entry();
  const int b = blockIdx.x;
  const int ps = pos[b];
  if (threadIdx.x == 0) {
    int slot = -1;
    if (active[b] > 0 && ps >= 0 && ps / kPage < max_pages)
      slot = page_table[static_cast<long long>(b) * max_pages + ps / kPage] * kPage + ps % kPage;
    slots[b] = slot;
  }
  int tok = tokens[b];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const uint4* src = reinterpret_cast<const uint4*>(embed + static_cast<long long>(tok) * ld_embed);
  uint4* dst = reinterpret_cast<uint4*>(x + static_cast<long long>(b) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

struct DecodeAdvanceArgs {
  const int* new_tok;
  const float* new_lp;
  int* active;
  int* finished;
  int* tokens;
  int* pos;
  int* len;
  int* priv_len;
  const int* max_len;
  const int* stop;       // 8 stop token ids, -1 = unused
  long long* out_idx;    // [B] tokens emitted so far
  int* out_tokens;       // [B, out_cap]
  float* out_lps;        // [B, out_cap]
  int out_cap;
  int* step;             // global decode step (random stream)
  int B;
};

// End of a decode step: store the sampled token and its log-prob, decide which sequences end (stop token or length
// limit), and advance positions / lengths of those that go on.  One thread per slot.
__global__ void __launch_bounds__(256) decode_advance_kernel(const DecodeAdvanceArgs a) {
  pdl_entry();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0) *a.step += 1;
  if (b >= a.B) return;
  const bool act = a.active[b] > 0;
  if (!act) return;
  const int tok = a.new_tok[b];
  long long idx = a.out_idx[b];
  if (idx > a.out_cap - 1) idx = a.out_cap - 1;
  a.out_tokens[static_cast<long long>(b) * a.out_cap + idx] = tok;
  a.out_lps[static_cast<long long>(b) * a.out_cap + idx] = a.new_lp[b];
  a.out_idx[b] += 1;
  const int newlen = a.len[b] + 1;
  bool stop = false;
#pragma unroll
  for (int i = 0; i < 8; ++i) stop |= (a.stop[i] == tok);
  if (stop || newlen >= a.max_len[b]) {
    a.finished[b] = 1;
    a.active[b] = 0;
    return;
  }
  a.tokens[b] = tok;
  a.pos[b] += 1;
  a.len[b] = newlen;
  a.priv_len[b] += 1;
}

// ---------------------------------------------------------------------------- sampling
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
// Order-preserving map float -> uint32 (larger float = larger key) and back.
__device__ __forceinline__ uint32_t float_key(float z) {
  const uint32_t u = __float_as_uint(z);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// top-k / top-p cut-off per row: thr[b] = smallest scaled logit that stays in the distribution (-inf: no filter).
// Exact radix select on the 32-bit keys, 11 + 11 + 10 bits per pass; every pass builds a histogram of counts (top-k)
// or of softmax mass (top-p) over the keys that match the prefix found so far, then walks it from the top.
// One block per row; the row stays in L2 between passes.
constexpr int kSelBins = 2048;
__global__ void __launch_bounds__(1024)
sample_threshold_kernel(const float* __restrict__ logits, long long ldl, const float* __restrict__ temperature, int V,
                        const int* __restrict__ top_k, const float* __restrict__ top_p, float* __restrict__ thr) {
  pdl_entry();
  const int b = blockIdx.x;
  const float T = temperature[b];
  const int k_lim = top_k ? top_k[b] : 0;
  const float p_lim = top_p ? top_p[b] : 1.f;
  const bool use_k = k_lim > 0 && k_lim < V, use_p = p_lim < 1.f;
  if (!(T > 0.f) || (!use_k && !use_p)) {
    if (threadIdx.x == 0) thr[b] = -INFINITY;
    return;
  }
  const float invT = 1.f / T;
  const float* row = logits + b * ldl;
  __shared__ float hist[kSelBins];
  __shared__ float red[32];
  __shared__ float sh_m, sh_s, sh_above;
  __shared__ uint32_t sh_prefix;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // row maximum and softmax denominator (top-p needs the mass scale)
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, row[i] * invT);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
  if (warp == 0) {
    m = red[lane];
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) sh_m = m;
  }
  __syncthreads();
  m = sh_m;
  float ssum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) ssum += __expf(row[i] * invT - m);
  for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
  __syncthreads();
  if (lane == 0) red[warp] = ssum;
  __syncthreads();
  if (warp == 0) {
    ssum = red[lane];
    for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
    if (lane == 0) sh_s = ssum;
  }
  __syncthreads();
  float best_thr = -INFINITY;
  uint32_t kcut = 0u;  // key of the k-th largest logit once top-k has run: top-p then works inside that set
#pragma unroll 1
  for (int mode = 0; mode < 2; ++mode) {  // 0: top-k (weights 1), 1: top-p (weights = softmax mass)
    if ((mode == 0 && !use_k) || (mode == 1 && !use_p)) continue;
    if (mode == 1 && kcut != 0u) {
      // top-p applies to the distribution renormalised over the top-k set: its mass replaces the full sum
      float part = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * invT;
        if (float_key(z) >= kcut) part += __expf(z - m);
      }
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      __syncthreads();
      if (lane == 0) red[warp] = part;
      __syncthreads();
      if (warp == 0) {
        part = red[lane];
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) sh_s = part;
      }
      __syncthreads();
    }
    const float target = mode == 0 ? static_cast<float>(k_lim) : p_lim * sh_s;
    if (threadIdx.x == 0) {
      sh_prefix = 0u;
      sh_above = 0.f;
    }
    int shift = 32;
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      const int bits = pass < 2 ? 11 : 10;
      shift -= bits;
      const int nb = 1 << bits;
      for (int i = threadIdx.x; i < nb; i += blockDim.x) hist[i] = 0.f;
      __syncthreads();
      const uint32_t prefix = sh_prefix;
      const uint32_t hi_mask = pass == 0 ? 0u : ~((1u << (shift + bits)) - 1u);
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * invT;
        const uint32_t key = float_key(z);
        if ((key & hi_mask) != prefix || key < kcut) continue;
        atomicAdd(&hist[(key >> shift) & (nb - 1)], mode == 0 ? 1.f : __expf(z - m));
      }
      __syncthreads();
      if (warp == 0) {
        // walk the bins from the top: lane l owns bins [nb - (l+1)*per, nb - l*per)
        const int per = nb / 32;
        float mine = 0.f;
        for (int j = 0; j < per; ++j) mine += hist[nb - 1 - (lane * per + j)];
        float incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        const float above = sh_above;
        const float before = above + incl - mine;              // weight above this lane's bins
        const bool crosses = before < target && before + mine >= target;
        const unsigned vote = __ballot_sync(0xffffffffu, crosses);
        // no lane crosses only through rounding at the very end: take the last non-empty lane
        const int owner = vote ? __ffs(vote) - 1 : 31;
        if (lane == owner) {
          float acc = before;
          int chosen = nb - 1 - (lane * per + per - 1);
          for (int j = 0; j < per; ++j) {
            const int bin = nb - 1 - (lane * per + j);
            if (acc + hist[bin] >= target) {
              chosen = bin;
              break;
            }
            acc += hist[bin];
          }
          sh_above = acc;
          sh_prefix = prefix | (static_cast<uint32_t>(chosen) << shift);
        }
      }
      __syncthreads();
    }
    best_thr = fmaxf(best_thr, key_float(sh_prefix));
    if (mode == 0) kcut = sh_prefix;
    __syncthreads();
  }
  if (threadIdx.x == 0) thr[b] = best_thr;
}

// One block per row.  logits [B, V] fp32 (row stride ldl).  temperature[b] <= 0 -> greedy.
// Gumbel-max sampling: argmax(z + g), z = logit / T, over the tokens with z >= thr[b] when a cut-off is given.
// Also returns log softmax(z)[token] under the UNFILTERED distribution (what the trainer's old_log_probs expect).
__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, long long ldl, const float* __restrict__ temperature, int V,
              uint32_t seed, const int* __restrict__ step_dev, const float* __restrict__ thr,
              int* __restrict__ tokens, float* __restrict__ logprobs) {
  pdl_entry();
  const int b = blockIdx.x;
  const uint32_t step = step_dev ? static_cast<uint32_t>(*step_dev) : 0u;
  const float T = temperature[b];
  const bool greedy = !(T > 0.f);
  const float invT = greedy ? 1.f : 1.f / T;
  const float* row = logits + b * ldl;
  const float cut = (thr && !greedy) ? thr[b] : -INFINITY;
  float best = -INFINITY, best_z = 0.f;
  int best_i = 0;
  float m = -INFINITY, s = 0.f;
  // one hash per element: the per-(seed, step, row) part is mixed once, the column enters by a Weyl step
  const uint32_t base = hash_u32(seed ^ (step * 0x9E3779B9u)) ^ hash_u32(static_cast<uint32_t>(b) * 0x85ebca6bU + 1u);
  auto consider = [&](float raw, int i) {
    const float z = raw * invT;
    // running softmax statistics with ONE exponential per element (the rescaling branch is taken only when a new
    // maximum appears, which becomes rare after the first few elements of a thread)
    if (z > m) {
      s = s * __expf(m - z) + 1.f;
      m = z;
    } else if (z > -INFINITY) {
      s += __expf(z - m);
    }
    float key = z;
    if (!greedy) {
      if (z >= cut) {
        const uint32_t h = hash_u32(base + static_cast<uint32_t>(i) * 0x9E3779B9u);
        const float u = (static_cast<float>(h >> 8) + 0.5f) * (1.f / 16777216.f);
        key = z - __logf(-__logf(u));
      } else {
        key = -INFINITY;  // outside the top-k / top-p set
      }
    }
    if (key > best) {
      best = key;
      best_i = i;
      best_z = z;
    }
  };
  if ((ldl & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
    for (int i4 = threadIdx.x; i4 < n4; i4 += blockDim.x) {
      const float4 v = row4[i4];
      consider(v.x, 4 * i4);
      consider(v.y, 4 * i4 + 1);
      consider(v.z, 4 * i4 + 2);
      consider(v.w, 4 * i4 + 3);
    }
    for (int i = 4 * n4 + threadIdx.x; i < V; i += blockDim.x) consider(row[i], i);
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) consider(row[i], i);
  }
  __shared__ float sb[32], sz[32], sm[32], ss[32];
  __shared__ int si[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    const float oz = __shfl_xor_sync(0xffffffffu, best_z, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
      best_z = oz;
    }
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (om == -INFINITY ? 0.f : os * __expf(om - mn));
    m = mn;
  }
  if (lane == 0) {
    sb[warp] = best;
    si[warp] = best_i;
    sz[warp] = best_z;
    sm[warp] = m;
    ss[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sb[lane] : -INFINITY;
    best_i = lane < nw ? si[lane] : 0x7fffffff;
    best_z = lane < nw ? sz[lane] : 0.f;
    m = lane < nw ? sm[lane] : -INFINITY;
    s = lane < nw ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      const float oz = __shfl_xor_sync(0xffffffffu, best_z, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
        best_z = oz;
      }
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mn)) + (om == -INFINITY ? 0.f : os * __expf(om - mn));
      m = mn;
    }
    if (lane == 0) {
      tokens[b] = best_i;
      logprobs[b] = best_z - (m + __logf(s));
    }
  }
}

}  // namespace apb

extern "C" {
using namespace apb;

int apb_kv_cache_write(const void* k, long long ldk, const void* v, long long ldv, const int* slots, void* kcache,
                       void* vcache, int T, int Hkv, int D, cudaStream_t s) {
  if (T <= 0) return 0;
  if ((D % 8) || (ldk % 8) || (ldv % 8)) return kBadArgument;
  const long long n = static_cast<long long>(T) * Hkv * D / 8;
  const int grid = static_cast<int>((n + 255) / 256 < apb::sm_count() * 8 ? (n + 255) / 256 : apb::sm_count() * 8);
  return static_cast<int>(launch_kernel(kv_cache_write_kernel, dim3(grid), dim3(256), 0, s,
                                        static_cast<const __nv_bfloat16*>(k), ldk, static_cast<const __nv_bfloat16*>(v),
                                        ldv, slots, static_cast<__nv_bfloat16*>(kcache),
                                        static_cast<__nv_bfloat16*>(vcache), T, Hkv, D));
}

int apb_decode_qkv_post(float* acc, long long ld_acc, const void* wq, const void* wk, const float* cos_t,
                        const float* sin_t, const int* pos, const int* slots, void* q_out, void* kcache, void* vcache,
                        int B, int Hq, int Hkv, int D, float eps, cudaStream_t s) {
  if (B <= 0) return 0;
  const long long warps = static_cast<long long>(B) * (Hq + 2 * Hkv);
  const int grid = static_cast<int>((warps * 32 + 255) / 256);
#define APB_QKV_POST(DD)                                                                                       \
  return static_cast<int>(launch_kernel(decode_qkv_post_kernel<DD>, dim3(grid), dim3(256), 0, s, acc, ld_acc,  \
                                        static_cast<const __nv_bfloat16*>(wq),                                \
                                        static_cast<const __nv_bfloat16*>(wk), cos_t, sin_t, pos, slots,      \
                                        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(kcache), \
                                        static_cast<__nv_bfloat16*>(vcache), B, Hq, Hkv, eps))
  if (D == 128) APB_QKV_POST(128);
  if (D == 64) APB_QKV_POST(64);
  if (D == 256) APB_QKV_POST(256);
#undef APB_QKV_POST
  return kBadArgument;
}

// Selects the scalar (CUDA-core) paged decode kernel instead of the MMA one: numerics cross-check and A/B timing.
static int g_decode_scalar = 0;
void apb_decode_use_scalar(int on) { g_decode_scalar = on; }

// Partial attention of G query groups (see paged_decode_kernel).  out_o / out_ml are fp32 scratch
// [Bq, Hq, splits, D] and [Bq, Hq, splits, 2].
int apb_paged_decode_partial(const void* q, const int* q_start, const int* q_count, const int* pages, int max_pages,
                             const int* kv_len, const void* kcache, const void* vcache, float* out_o, float* out_ml,
                             int G, int Hq, int Hkv, int D, int splits, float scale, cudaStream_t s) {
  if (G <= 0) return 0;
  if (D != 128 || Hq % Hkv || splits < 1) return kBadArgument;
  const int R = Hq / Hkv;
  const dim3 grid(G * Hkv, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (16 % R == 0 && !g_decode_scalar) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMmaSmem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[dev & 63] = true;
    }
    return static_cast<int>(launch_kernel(paged_decode_mma_kernel, grid, dim3(kDecThreads), kMmaSmem, s,
                                          static_cast<const __nv_bfloat16*>(q), q_start, q_count, pages, max_pages,
                                          kv_len, static_cast<const __nv_bfloat16*>(kcache),
                                          static_cast<const __nv_bfloat16*>(vcache), out_o, out_ml, Hq, Hkv, splits,
                                          sl2));
  }
#define APB_DEC(RR)                                                                                           \
  paged_decode_kernel<RR, 128><<<grid, kDecThreads, 0, s>>>(                                                  \
      static_cast<const __nv_bfloat16*>(q), q_start, q_count, pages, max_pages, kv_len,                      \
      static_cast<const __nv_bfloat16*>(kcache), static_cast<const __nv_bfloat16*>(vcache), out_o, out_ml, Hq, \
      Hkv, splits, sl2)
  if (R == 1) APB_DEC(1);
  else if (R == 2) APB_DEC(2);
  else if (R == 4) APB_DEC(4);
  else if (R == 8) APB_DEC(8);
  else return kBadArgument;
#undef APB_DEC
  return static_cast<int>(cudaGetLastError());
}

// Merges up to 4 partial sets into out [rows, Hq, D] bf16 (+ optional natural-log LSE [rows, Hq]).
// row_mask [rows] (or null): bit s set = source s is valid for the row.
int apb_decode_merge(const float* const* o_ptrs, const float* const* ml_ptrs, const int* splits, int n_src,
                     const int* row_mask, void* out, float* lse, int rows, int Hq, int D, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (n_src < 1 || n_src > 4 || D != 128) return kBadArgument;
  MergeSrc src;
  src.n = n_src;
  for (int i = 0; i < 4; ++i) {
    src.o[i] = i < n_src ? o_ptrs[i] : nullptr;
    src.ml[i] = i < n_src ? ml_ptrs[i] : nullptr;
    src.splits[i] = i < n_src ? splits[i] : 0;
  }
  const long long warps = static_cast<long long>(rows) * Hq;
  const int grid = static_cast<int>((warps * 32 + 255) / 256);
  return static_cast<int>(launch_kernel(decode_merge_kernel, dim3(grid), dim3(256), 0, s, src, row_mask,
                                        static_cast<__nv_bfloat16*>(out), lse, rows, Hq, D));
}

// Step bookkeeping of the rollout engine (see decode_begin_kernel / decode_advance_kernel).  All arrays are
// device buffers of the engine; x [B, H] bf16 receives the embedding rows, slots [B] the cache slots.
int apb_decode_begin(const int* tokens, const int* pos, const int* active, const int* page_table, int max_pages,
                     const void* embed, long long ld_embed, int H, int vocab, int* slots, void* x, int B,
                     cudaStream_t s) {
  if (B <= 0) return 0;
  if ((H % 8) || (ld_embed % 8) || !tokens || !pos || !active || !page_table || !embed || !slots || !x)
    return kBadArgument;
  return static_cast<int>(launch_kernel(decode_begin_kernel, dim3(B), dim3(128), 0, s, tokens, pos, active, page_table,
                                        max_pages, static_cast<const __nv_bfloat16*>(embed), ld_embed, H, vocab, slots,
                                        static_cast<__nv_bfloat16*>(x)));
}

int apb_decode_advance(const int* new_tok, const float* new_lp, int* active, int* finished, int* tokens, int* pos,
                       int* len, int* priv_len, const int* max_len, const int* stop, long long* out_idx,
                       int* out_tokens, float* out_lps, int out_cap, int* step, int B, cudaStream_t s) {
  if (B <= 0) return 0;
  if (!new_tok || !new_lp || !active || !finished || !tokens || !pos || !len || !priv_len || !max_len || !stop ||
      !out_idx || !out_tokens || !out_lps || !step || out_cap < 1)
    return kBadArgument;
  DecodeAdvanceArgs a{new_tok, new_lp, active, finished, tokens, pos, len, priv_len, max_len, stop, out_idx,
                      out_tokens, out_lps, out_cap, step, B};
  return static_cast<int>(launch_kernel(decode_advance_kernel, dim3((B + 255) / 256), dim3(256), 0, s, a));
}

// step_dev: device int holding the decode step (read by the kernel, so a captured graph sees new values).
int apb_sample(const float* logits, long long ldl, const float* temperature, int B, int V, unsigned seed,
               const int* step_dev, int* tokens, float* logprobs, cudaStream_t s) {
  if (B <= 0) return 0;
  return static_cast<int>(launch_kernel(sample_kernel, dim3(B), dim3(1024), 0, s, logits, ldl, temperature, V,
                                        static_cast<uint32_t>(seed), step_dev, static_cast<const float*>(nullptr),
                                        tokens, logprobs));
}

// Sampling restricted to the top-k tokens and to the smallest set of tokens with probability mass >= top_p.
// top_k [B] (<= 0: off), top_p [B] (>= 1: off), thr [B] fp32 scratch for the per-row cut-off.
int apb_sample_filtered(const float* logits, long long ldl, const float* temperature, int B, int V, unsigned seed,
                        const int* step_dev, const int* top_k, const float* top_p, float* thr, int* tokens,
                        float* logprobs, cudaStream_t s) {
  if (B <= 0) return 0;
  if (!thr) return kBadArgument;
  cudaError_t e = launch_kernel(sample_threshold_kernel, dim3(B), dim3(1024), 0, s, logits, ldl, temperature, V, top_k,
                                top_p, thr);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_kernel(sample_kernel, dim3(B), dim3(1024), 0, s, logits, ldl, temperature, V,
                                        static_cast<uint32_t>(seed), step_dev, static_cast<const float*>(thr), tokens,
                                        logprobs));
}
}
