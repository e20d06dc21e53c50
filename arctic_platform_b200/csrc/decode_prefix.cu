// Forest-cascade decode, shared-prefix pass on tcgen05 tensor cores.
//
// All decode queries that share one node of the prefix forest (the rollouts of one prompt, or all rollouts of
// all prompts under a common header) attend to the node's KV pages TOGETHER: the query rows of up to 128/R sequences x R query heads of one KV head form one
// 128-row UMMA tile, the node's K/V pages are streamed once by TMA (one 16-token page per copy, straight out
// of the paged cache), S = Q K^T and P V run on the tensor core with S/P in tensor memory, and the result is
// left as an un-normalised partial (max, sum, numerator) per query row and KV split, in the same format as
// the per-sequence pass, so one LSE merge joins the two levels.  KV of a shared prompt is therefore read once
// per step for all of its rollouts instead of once per rollout.  A forest with several shared levels (header ->
// prompt -> rollout) is one launch: every node names its level, partials of level l go to buffer l, and the merge
// joins the levels a sequence takes part in with its private pass.  The reference obtains this behaviour from
// ArcticInference's forest cascade attention (`use_fca`, arctic_platform/common/utils/server_models.py:123-132).
//
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 softmax (one row each).
//
// The KV blocks of a node are software-pipelined: tensor memory holds TWO score buffers, the MMA warp issues Q K^T of
// block j+1 before it waits for the probabilities of block j, and P V accumulates over all blocks in ONE output
// buffer in tensor memory that the softmax warps read only once, at the end.  The running maximum is therefore a
// REFERENCE maximum: a row rescales its output (read, multiply, write back -- after the previous P V has landed)
// only when its true maximum has moved more than 2^8 above the reference; otherwise the probabilities are taken
// against the stale reference (at most 256, harmless in bf16 / fp32) and nothing is rescaled.  Per block a softmax
// thread thus reads its 128 scores once, takes 128 exponentials and writes 64 packed words -- the per-block read-out
// and fold of the output (and the second pass over the scores) of the earlier versions set the pace of the kernel.
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct DecPrefixParams {
  const int* q_start;   // [G] first sequence (query row) of the group
  const int* q_count;   // [G] sequences in the group (R * count <= 128)
  const int* pages;     // [G, max_pages]
  int max_pages;
  const int* kv_len;    // [G] tokens in the node
  const int* level;     // [G] tree level of the node (selects the output buffer) or null (all level 0)
  float* out_o[3];      // per level: [Bq, Hq, splits, D] fp32 un-normalised numerators
  float* out_ml[3];     // per level: [Bq, Hq, splits, 2] (max in base-2 scaled units, sum)
  int Hq, Hkv, splits;
  float scale_log2;
  int* status;
};

constexpr int kDpThreads = 192;
constexpr int kDpSlots = 4;
constexpr int kDpTile = 128 * 128 * 2;  // one Q / K / V tile (D = 128)
constexpr int kDpSmem = kDpTile + kDpSlots * kDpTile + 1024 + 256;
constexpr int kDpTmemCols = 512;        // S0 | S1 | O (128 fp32 columns each); 384 used, the allocation is a power of 2
constexpr float kDpRescaleSlack = 8.f;  // log2 units the true row maximum may exceed the reference before a rescale

__global__ void __launch_bounds__(kDpThreads, 1)
decode_prefix_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const DecPrefixParams p) {
  constexpr int D = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;
  uint8_t* smem_kv = smem + kDpTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_kv + kDpSlots * kDpTile);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + kDpSlots;
  uint64_t* q_full = bars + 2 * kDpSlots;
  uint64_t* s_full = q_full + 1;    // [2] MMA -> softmax: scores of block j are in S[j & 1]
  uint64_t* p_full = s_full + 2;    // [2] softmax -> MMA: probabilities of block j are in S[j & 1]
  uint64_t* o_full = p_full + 2;    // [1] MMA -> softmax: P V of block j has been added to O (one phase per block)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_full + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x / p.Hkv;
  const int kvh = blockIdx.x % p.Hkv;
  const int split = blockIdx.y;
  const int R = p.Hq / p.Hkv;
  const int nq = p.q_count[g];
  const int qs = p.q_start[g];
  const int len = p.kv_len[g];
  const int n_blocks_all = (len + 127) / 128;
  const int per = (n_blocks_all + p.splits - 1) / p.splits;
  const int b0 = split * per;
  const int b1 = min(n_blocks_all, b0 + per);
  const int n_blocks = max(0, b1 - b0);
  const int last_page = (len + 15) / 16 - 1;
  if (nq <= 0) {        // uniform across the CTA, nothing allocated yet
    pdl_entry();        // a chained kernel never ends before its predecessor has: later kernels rely on that order
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDpSlots; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(q_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 128);
      mbar_init(&o_full[b], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kDpTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // chained launch: barriers and TMEM are set up.  The pages of a shared node are never written while its
  // sequences decode (new tokens go to private pages), so the first K and V tiles are requested BEFORE
  // the wait for the previous kernel; q, which that kernel produces, is loaded after it.
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0 && n_blocks > 0) {
      bool ok = true;
      const int early = min(2, 2 * n_blocks);       // the first K and V tiles; q must not queue behind a full ring
      for (int n = 0; n < 2 * n_blocks && ok; ++n) {
        if (n == early) {
          pdl_wait();
          mbar_expect_tx(q_full, kDpTile);
          for (int c = 0; c < 2; ++c) tma_load_4d(smem_q + c * 16384, &tma_q, q_full, c * 64, 0, kvh, qs);
        }
        const int slot = n % kDpSlots;
        const uint32_t phase = (n / kDpSlots) & 1;
        if (n >= early && !mbar_wait(&kv_empty[slot], phase ^ 1, p.status, kTimeoutEmpty)) {
          ok = false;
          break;
        }
        const int b = b0 + (n >> 1);
        uint8_t* dst = smem_kv + slot * kDpTile;
        mbar_expect_tx(&kv_full[slot], kDpTile);
        const CUtensorMap* map = (n & 1) ? &tma_v : &tma_k;
        for (int pg = 0; pg < 8; ++pg) {
          // pages past the end of the node are replaced by its last page: finite data, masked by `limit`
          const int pi = min(b * 8 + pg, last_page);
          const int page = p.pages[static_cast<long long>(g) * p.max_pages + pi];
          const int row = (page * p.Hkv + kvh) * 16;
          for (int c = 0; c < 2; ++c) tma_load_2d(dst + c * 16384 + pg * 2048, map, &kv_full[slot], c * 64, row);
        }
      }
      if (2 * n_blocks <= early) {         // every tile fitted into the first ring-full: q is still to come
        pdl_wait();
        mbar_expect_tx(q_full, kDpTile);
        for (int c = 0; c < 2; ++c) tma_load_4d(smem_q + c * 16384, &tma_q, q_full, c * 64, 0, kvh, qs);
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) {
        }
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutFull);
      const uint32_t qa = smem_u32(smem_q);
      // S(j) = Q K(j)^T into score buffer j & 1
      auto issue_qk = [&](int j) -> bool {
        const int nk = 2 * j;
        if (!mbar_wait(&kv_full[nk % kDpSlots], (nk / kDpSlots) & 1, p.status, kTimeoutFull)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(smem_kv + (nk % kDpSlots) * kDpTile);
        const uint32_t t_s = tmem_base + (j & 1) * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * 16384 + (k % 4) * 32;
          umma_bf16_ss(t_s, umma_smem_desc(qa + off, 0, 1024), umma_smem_desc(ka + off, 0, 1024), idesc_s,
                       k > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[j & 1]);
        tc_commit(&kv_empty[nk % kDpSlots]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        // the scores of the NEXT block first: they are ready when the softmax warps finish this one.  Its buffer
        // held the probabilities of block j-1, whose P V was issued before this point (the pipe runs in order).
        if (j + 1 < n_blocks && !issue_qk(j + 1)) {
          ok = false;
          break;
        }
        const int nv = 2 * j + 1, b = j & 1;
        if (!mbar_wait(&kv_full[nv % kDpSlots], (nv / kDpSlots) & 1, p.status, kTimeoutFull) ||
            !mbar_wait(&p_full[b], (j >> 1) & 1, p.status, kTimeoutTmemEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t va = smem_u32(smem_kv + (nv % kDpSlots) * kDpTile);
        const uint32_t t_p = tmem_base + b * 128, t_o = tmem_base + 256;
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k)
          umma_bf16_ts(t_o, t_p + k * 8, umma_smem_desc(va + k * 2048, 16384, 1024), idesc_o,
                       (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(&o_full[0]);
        tc_commit(&kv_empty[nv % kDpSlots]);
      }
    }
  } else {
    pdl_wait();                    // the partial buffers may still be read by the previous step's merge
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    // m_ref: the maximum the exponentials are taken against (see the header); l_run: row sum in the same units
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    const uint32_t t_o = tmem_base + lane_off + 256;
    for (int j = 0; j < n_blocks; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_s = tmem_base + lane_off + b * 128;
      const int limit = max(0, min(128, len - (b0 + j) * 128));
      uint32_t sc[4][32];
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sc[c]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i < limit) mx = fmaxf(mx, __uint_as_float(sc[c][i]));
      const float m_new = fmaxf(m_ref, mx * p.scale_log2);
      if (m_new > m_ref + kDpRescaleSlack || m_ref == -INFINITY) {
        // move the reference.  Everything accumulated so far is in the old units: the row sum here, the output
        // row in tensor memory (once the previous block's P V has landed; block 0 has nothing to rescale)
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {
          if (!mbar_wait(&o_full[0], (j - 1) & 1, p.status, kTimeoutTmemFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_o + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, r);
          }
        }
        l_run *= alpha;
        m_ref = m_new;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rowsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = exp2f(__uint_as_float(sc[c][2 * i]) * p.scale_log2 - m_use);
          float p1 = exp2f(__uint_as_float(sc[c][2 * i + 1]) * p.scale_log2 - m_use);
          if (c * 32 + 2 * i >= limit) p0 = 0.f;
          if (c * 32 + 2 * i + 1 >= limit) p1 = 0.f;
          rowsum += p0 + p1;
          pk[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(t_s + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[b]);
      l_run += rowsum;
    }
    // the output row: one read after the last P V
    float o_acc[D];
    if (ok && n_blocks > 0) {
      ok = mbar_wait(&o_full[0], (n_blocks - 1) & 1, p.status, kTimeoutTmemFull);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_o + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = __uint_as_float(r[i]);
        }
        tc_fence_before();
      }
    } else {
#pragma unroll
      for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    }
    const float m_run = m_ref;
    if (ok && row < nq * R) {
      const int seq = qs + row / R;
      const int head = kvh * R + row % R;
      const long long base = (static_cast<long long>(seq) * p.Hq + head) * p.splits + split;
      int lvl = p.level ? p.level[g] : 0;
      lvl = lvl < 0 ? 0 : (lvl > 2 ? 2 : lvl);
      float* out_o = lvl == 0 ? p.out_o[0] : (lvl == 1 ? p.out_o[1] : p.out_o[2]);
      float* out_ml = lvl == 0 ? p.out_ml[0] : (lvl == 1 ? p.out_ml[1] : p.out_ml[2]);
      float4* dst = reinterpret_cast<float4*>(out_o + base * D);
#pragma unroll
      for (int q = 0; q < D / 4; ++q)
        dst[q] = make_float4(o_acc[q * 4], o_acc[q * 4 + 1], o_acc[q * 4 + 2], o_acc[q * 4 + 3]);
      out_ml[base * 2] = m_run;
      out_ml[base * 2 + 1] = l_run;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kDpTmemCols);
  }
}

}  // namespace apb

extern "C" {

// Shared-prefix pass of cascade decode on the tensor cores.  Same node tables and output format as
// apb_paged_decode_partial, plus `level` [G] (or null): the partials of a node go to out_o[level] / out_ml[level]
// (up to 3 shared levels; unused entries may be null).  q [Bq, Hq, D] bf16 contiguous; caches
// [num_pages, Hkv, 16, D] bf16.  Requires D == 128 and R * max(q_count) <= 128.
int apb_decode_prefix_tc(const void* q, int Bq, const int* q_start, const int* q_count, const int* pages,
                         int max_pages, const int* kv_len, const int* level, const void* kcache, const void* vcache,
                         long long num_pages, float* const* out_o, float* const* out_ml, int n_levels, int G, int Hq,
                         int Hkv, int D, int splits, float scale, cudaStream_t s) {
  using namespace apb;
  if (G <= 0) return 0;
  if (D != 128 || Hq % Hkv || splits < 1 || n_levels < 1 || n_levels > 3 || !out_o || !out_ml) return kBadArgument;
  const int R = Hq / Hkv;
  if (R > 128 || 128 % R) return kBadArgument;
  for (int l = 0; l < n_levels; ++l)
    if (!out_o[l] || !out_ml[l]) return kBadArgument;
  if (n_levels > 1 && !level) return kBadArgument;
  CUtensorMap tq, tk, tv;
  {
    const uint64_t dims[4] = {128, static_cast<uint64_t>(R), static_cast<uint64_t>(Hkv), static_cast<uint64_t>(Bq)};
    const uint64_t strides[3] = {128 * 2ull, static_cast<uint64_t>(R) * 128 * 2ull, static_cast<uint64_t>(Hq) * 128 * 2ull};
    const uint32_t box[4] = {64, static_cast<uint32_t>(R), 1, static_cast<uint32_t>(128 / R)};
    int rc = make_tmap_nd(&tq, q, 2, 4, dims, strides, box);
    if (rc) return 1000 + rc;
  }
  const uint64_t rows = static_cast<uint64_t>(num_pages) * Hkv * 16;
  int rc = make_tmap_2d(&tk, kcache, 2, rows, 128, 128, 64, 16);
  if (rc) return 2000 + rc;
  rc = make_tmap_2d(&tv, vcache, 2, rows, 128, 128, 64, 16);
  if (rc) return 3000 + rc;
  DecPrefixParams p;
  p.q_start = q_start;
  p.q_count = q_count;
  p.pages = pages;
  p.max_pages = max_pages;
  p.kv_len = kv_len;
  p.level = level;
  for (int l = 0; l < 3; ++l) {
    // levels beyond n_levels alias the last valid buffer: a level id out of range can never reach a null pointer
    p.out_o[l] = out_o[l < n_levels ? l : n_levels - 1];
    p.out_ml[l] = out_ml[l < n_levels ? l : n_levels - 1];
  }
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_device_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(decode_prefix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDpSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const dim3 grid(G * Hkv, splits);
  return static_cast<int>(launch_kernel(decode_prefix_kernel, grid, dim3(kDpThreads), kDpSmem, s, tq, tk, tv, p));
}
}
