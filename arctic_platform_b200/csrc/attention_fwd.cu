// Segment attention forward on tcgen05 tensor cores.
//
// One kernel covers plain packed varlen causal attention, ZoRRo prompt-to-prompt
// attention and ZoRRo response-to-(shared prompt + own response) attention: every
// query tile attends to a "prefix" key range that is fully visible (the group's
// shared prompt, stored ONCE in the packed K/V) followed by its "own" key range
// under a bottom-right aligned causal mask.  The reference reaches the same result
// by materialising per-sample [prompt || response] K/V copies with torch.cat and
// two flash_attn_varlen calls per layer
// (arctic_platform/rl/zorro_train/qwen_attention_patcher.py:1197-1231,
//  arctic_platform/rl/zorro_train/zorro_train.py:857-912); here the key tile index
// is resolved in the kernel and nothing is replicated.
//
// CTA = 320 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 and 6-9 two
// softmax groups.  The two groups hold two query heads of the same KV head (same
// 128 query rows), so they walk the same K/V tiles and ping-pong on the tensor
// core: while one group does softmax on S_j the other group's P*V and next S run.
// S (fp32) lives in TMEM, P (bf16) overwrites it in place and feeds the P*V MMA as
// the TMEM A operand, the P*V product is read back and accumulated in registers
// with the usual online-softmax rescale.
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct AttnFwdParams {
  const int* work;  // [num_work][8]: q_row0, q_valid, pre_start, pre_len, own_start, own_len, diag, head|(pair<<16)
  int num_work;
  int Hq, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* O;  // [T, Hq*D]
  long long ldo;
  float* lse;        // [Hq, T] natural-log LSE
  int T;
  int* status;
};

constexpr int kAttnThreads = 320;
constexpr int kKvBlock = 128;

template <int D>
struct AttnCfg {
  static constexpr int kChunks = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;      // one Q, K or V tile
  static constexpr int kSlots = 4;                    // K/V ring
  static constexpr int kSmemBytes = 2 * kTileBytes + kSlots * kTileBytes + 1024 + 256;
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const AttnFwdParams p) {
  using Cfg = AttnCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_q = smem;                              // 2 tiles
  uint8_t* smem_kv = smem + 2 * Cfg::kTileBytes;       // ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_kv + Cfg::kSlots * Cfg::kTileBytes);
  uint64_t* kv_full = bars;                 // [kSlots]
  uint64_t* kv_empty = bars + Cfg::kSlots;  // [kSlots]
  uint64_t* q_full = bars + 2 * Cfg::kSlots;
  uint64_t* s_full = q_full + 1;  // [2]
  uint64_t* p_full = s_full + 2;  // [2]
  uint64_t* o_full = p_full + 2;  // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_full + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int* w = p.work + static_cast<long long>(blockIdx.x) * 8;
  const int q_row0 = w[0], q_valid = w[1], pre_start = w[2], pre_len = w[3], own_start = w[4], own_len = w[5],
            diag = w[6];
  const int head0 = w[7] & 0xFFFF;
  const int n_groups = (w[7] >> 16) ? 2 : 1;
  const int kvh = head0 / (p.Hq / p.Hkv);
  const int n_pre = (pre_len + kKvBlock - 1) / kKvBlock;
  const int n_own = (own_len + kKvBlock - 1) / kKvBlock;
  const int n_blocks = n_pre + n_own;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kSlots; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(q_full, 1);
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&p_full[g], 128);
      mbar_init(&o_full[g], 1);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // TMEM map: S/P of group g at columns [g*128, g*128+128), P*V of group g at [256 + g*128, ...+D)

  auto block_row = [&](int b) { return b < n_pre ? pre_start + b * kKvBlock : own_start + (b - n_pre) * kKvBlock; };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && n_blocks > 0) {
      mbar_expect_tx(q_full, n_groups * Cfg::kTileBytes);
      for (int g = 0; g < n_groups; ++g)
        for (int c = 0; c < Cfg::kChunks; ++c)
          tma_load_2d(smem_q + g * Cfg::kTileBytes + c * 16384, &tma_q, q_full, (head0 + g) * D + c * 64, q_row0);
      bool ok = true;
      for (int n = 0; n < 2 * n_blocks && ok; ++n) {
        const int slot = n % Cfg::kSlots;
        const uint32_t phase = (n / Cfg::kSlots) & 1;
        if (!mbar_wait(&kv_empty[slot], phase ^ 1, p.status, kTimeoutEmpty)) {
          ok = false;
          break;
        }
        const int row = block_row(n >> 1);
        uint8_t* dst = smem_kv + slot * Cfg::kTileBytes;
        mbar_expect_tx(&kv_full[slot], Cfg::kTileBytes);
        const CUtensorMap* map = (n & 1) ? &tma_v : &tma_k;
        for (int c = 0; c < Cfg::kChunks; ++c)
          tma_load_2d(dst + c * 16384, map, &kv_full[slot], kvh * D + c * 64, row);
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_blocks > 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, kKvBlock, 0, 0);
      const uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutFull);
      auto issue_s = [&](int g, int slot) {
        const uint32_t qa = smem_u32(smem_q + g * Cfg::kTileBytes);
        const uint32_t ka = smem_u32(smem_kv + slot * Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * 16384 + (k % 4) * 32;
          umma_bf16_ss(tmem_base + g * 128, umma_smem_desc(qa + off, 0, 1024), umma_smem_desc(ka + off, 0, 1024),
                       idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[g]);
      };
      auto issue_o = [&](int g, int slot) {
        const uint32_t va = smem_u32(smem_kv + slot * Cfg::kTileBytes);
#pragma unroll
        for (int k = 0; k < kKvBlock / 16; ++k) {
          umma_bf16_ts(tmem_base + 256 + g * 128, tmem_base + g * 128 + k * 8,
                       umma_smem_desc(va + k * 2048, 16384, 1024), idesc_o, k > 0 ? 1u : 0u);
        }
        tc_commit(&o_full[g]);
      };
      // K_j sits in ring position 2j, V_j in 2j+1.
      auto wait_slot = [&](int n) {
        return mbar_wait(&kv_full[n % Cfg::kSlots], (n / Cfg::kSlots) & 1, p.status, kTimeoutFull);
      };
      if (ok) ok = wait_slot(0);
      if (ok) {
        tc_fence_after();
        for (int g = 0; g < n_groups; ++g) issue_s(g, 0);
        // K_0 is released once both S_0 are done; later K_j are released after the second group's S_j.
        tc_commit(&kv_empty[0]);
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int nv = 2 * j + 1;
        const int nk = 2 * j + 2;
        if (!wait_slot(nv)) {
          ok = false;
          break;
        }
        const bool more = j + 1 < n_blocks;
        if (more && !wait_slot(nk)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int g = 0; g < n_groups; ++g) {
          if (!mbar_wait(&p_full[g], j & 1, p.status, kTimeoutTmemEmpty)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_o(g, nv % Cfg::kSlots);
          if (more) issue_s(g, nk % Cfg::kSlots);
        }
        if (!ok) break;
        tc_commit(&kv_empty[nv % Cfg::kSlots]);
        if (more) tc_commit(&kv_empty[nk % Cfg::kSlots]);
      }
    }
  } else if (n_blocks > 0) {
    // ---------------------------------------------------------------- softmax groups
    const int g = (warp - 2) >> 2;
    if (g < n_groups) {
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;  // row inside the query tile
      const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t t_s = tmem_base + lane_off + g * 128;
      const uint32_t t_o = tmem_base + lane_off + 256 + g * 128;
      float o_acc[D];
#pragma unroll
      for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < n_blocks; ++j) {
        if (!mbar_wait(&s_full[g], j & 1, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        int limit;  // number of visible key columns of this block for this row
        if (j < n_pre) {
          limit = pre_len - j * kKvBlock;
        } else {
          const int b0 = (j - n_pre) * kKvBlock;
          limit = min(own_len - b0, row + diag - b0 + 1);
        }
        limit = max(0, min(limit, kKvBlock));
        // pass 1: row maximum
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < kKvBlock / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < limit) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(m_run - m_use);  // m_run = -inf -> 0
        // pass 2: probabilities, written over S as packed bf16 (two per 32-bit column)
        float rowsum = 0.f;
#pragma unroll 1
        for (int c = 0; c < kKvBlock / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float p0 = exp2f(__uint_as_float(r[2 * i]) * p.scale_log2 - m_use);
            float p1 = exp2f(__uint_as_float(r[2 * i + 1]) * p.scale_log2 - m_use);
            if (c * 32 + 2 * i >= limit) p0 = 0.f;
            if (c * 32 + 2 * i + 1 >= limit) p1 = 0.f;
            rowsum += p0 + p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x16(t_s + c * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&p_full[g]);
        l_run = l_run * alpha + rowsum;
        m_run = m_new;
        // accumulate P*V of this block
        if (!mbar_wait(&o_full[g], j & 1, p.status, kTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_o + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha + __uint_as_float(r[i]);
        }
        tc_fence_before();
      }
      if (ok && row < q_valid) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const long long t = static_cast<long long>(q_row0) + row;
        __nv_bfloat16* dst = p.O + t * p.ldo + static_cast<long long>(head0 + g) * D;
#pragma unroll
        for (int q = 0; q < D / 8; ++q) {
          uint4 o;
          o.x = pack_bf16x2(o_acc[q * 8 + 0] * inv, o_acc[q * 8 + 1] * inv);
          o.y = pack_bf16x2(o_acc[q * 8 + 2] * inv, o_acc[q * 8 + 3] * inv);
          o.z = pack_bf16x2(o_acc[q * 8 + 4] * inv, o_acc[q * 8 + 5] * inv);
          o.w = pack_bf16x2(o_acc[q * 8 + 6] * inv, o_acc[q * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + q * 8) = o;
        }
        if (p.lse)
          p.lse[static_cast<long long>(head0 + g) * p.T + t] =
              l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace apb

extern "C" {

// q [T, Hq*D] (row stride ldq), k/v [T, Hkv*D] (ldk/ldv), o [T, Hq*D] (ldo), lse [Hq, T] fp32 or null.
// work: device int32 [num_work][8] (see AttnFwdParams).  scale is the softmax scale (1/sqrt(D)).
int apb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* work, int num_work,
                 int T, int Hq, int Hkv, int D, long long ldq, long long ldk, long long ldv, long long ldo,
                 float scale, cudaStream_t stream) {
  using namespace apb;
  if (num_work <= 0) return 0;
  if ((D != 128 && D != 64) || (ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || Hq % Hkv) return kBadArgument;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d(&tq, q, 2, T, static_cast<uint64_t>(Hq) * D, ldq, 64, 128);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tk, k, 2, T, static_cast<uint64_t>(Hkv) * D, ldk, 64, 128);
  if (rc) return 2000 + rc;
  rc = make_tmap_2d(&tv, v, 2, T, static_cast<uint64_t>(Hkv) * D, ldv, 64, 128);
  if (rc) return 3000 + rc;
  AttnFwdParams p;
  p.work = work;
  p.num_work = num_work;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = lse;
  p.T = T;
  p.status = status_device_ptr();
  static bool configured[2][64] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (D == 128) {
    if (!configured[0][dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           AttnCfg<128>::kSmemBytes);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[0][dev & 63] = true;
    }
    attn_fwd_kernel<128><<<num_work, kAttnThreads, AttnCfg<128>::kSmemBytes, stream>>>(tq, tk, tv, p);
  } else {
    if (!configured[1][dev & 63]) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           AttnCfg<64>::kSmemBytes);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[1][dev & 63] = true;
    }
    attn_fwd_kernel<64><<<num_work, kAttnThreads, AttnCfg<64>::kSmemBytes, stream>>>(tq, tk, tv, p);
  }
  return static_cast<int>(cudaGetLastError());
}
}
