// Segment attention backward on tcgen05 tensor cores (see attention_fwd.cu for
// the segment model).  One CTA owns one key block (128 rows of one KV head) and
// walks every 64-row query tile that can see it -- all query heads of the KV
// head, and under ZoRRo all rollouts that share the prompt the block belongs to
// -- so dK and dV of a shared prompt are accumulated in tensor memory and written
// once.  The reference gets these sums from autograd through torch.cat copies of
// the prompt K/V (arctic_platform/rl/zorro_train/zorro_train.py:857-912).
//
// Per query tile, with everything transposed so that TMEM lanes are key rows:
//   S^T  = K  Q^T          dP^T = V dO^T                     (tensor core)
//   P^T  = exp2(S^T*c - lse[q])     dS^T = P^T*(dP^T - delta[q])*scale   (128 threads)
//   dV  += P^T dO          dK  += dS^T Q        dQ^T = K^T dS^T          (tensor core)
// P^T overwrites S^T in TMEM and is the TMEM A operand of the dV product; dS^T goes
// to shared memory once and is read by two products (K-major for dK, MN-major for
// dQ^T).  dQ^T is added to an fp32 accumulator in global memory with coalesced
// red.add (lanes = head-dim index).
//
// Two gradient warpgroups take alternate query tiles, so the tensor core works on tile i+1 while the other group is
// still in the exponentials / dS of tile i.  Tensor memory (512 columns): per group one 64-column slot that holds
// S^T, then P^T, then dQ^T of its tile, and one 64-column slot for dP^T; dK and dV take 128 columns each.
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct AttnBwdParams {
  const int* cta;   // [n_cta][8]  kv_row0, kv_valid, kvh, list_off, list_cnt
  const int* list;  // [n_list][4] q_row0, q_valid, diag_rel
  int Hq, Hkv, T;
  float scale, scale_log2;
  const float* lse;    // [Hq, T]
  const float* delta;  // [Hq, T]
  float* dq_acc;       // [T, Hq*D] fp32, zero-initialised by the caller
  long long ld_dq;
  __nv_bfloat16* dk;   // [T, Hkv*D]
  __nv_bfloat16* dv;
  long long ld_dk, ld_dv;
  int* status;
};

constexpr int kBwdThreads = 320;  // producer, MMA issuer, two gradient groups of four warps
constexpr int kBwdQTile = 64;
constexpr int kBwdStages = 3;
constexpr int kBigDiag = 1 << 27;

template <int D>
struct AttnBwdCfg {
  static constexpr int kKvTileBytes = 128 * D * 2;
  static constexpr int kQTileBytes = kBwdQTile * D * 2;
  static constexpr int kStageBytes = 2 * kQTileBytes + 512;  // Q, dO, lse[64], delta[64]
  static constexpr int kDsBytes = 128 * kBwdQTile * 2;
  static constexpr int kSmemBytes = 2 * kKvTileBytes + kBwdStages * (2 * kQTileBytes) + 2 * kDsBytes +
                                    kBwdStages * 512 + 1024 + 256;
};

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_do,
                const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                const AttnBwdParams p) {
  using Cfg = AttnBwdCfg<D>;
  constexpr int QCH = Cfg::kQTileBytes / (D / 64);  // bytes of one 64-wide chunk of a Q/dO tile (8192)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_k = smem;
  uint8_t* smem_v = smem_k + Cfg::kKvTileBytes;
  uint8_t* smem_qdo = smem_v + Cfg::kKvTileBytes;                       // [stage][Q | dO]
  uint8_t* smem_ds = smem_qdo + kBwdStages * 2 * Cfg::kQTileBytes;      // [2][128 x 64 bf16]
  float* smem_stat = reinterpret_cast<float*>(smem_ds + 2 * Cfg::kDsBytes);  // [stage][lse 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(smem_stat) + kBwdStages * 512);
  uint64_t* full = bars;                    // [stages]
  uint64_t* empty = full + kBwdStages;      // [stages]
  uint64_t* kv_full = empty + kBwdStages;   // 1
  uint64_t* s_full = kv_full + 1;           // [2]  S^T of a tile is in its group's slot
  uint64_t* dp_full = s_full + 2;           // [2]  dP^T likewise
  uint64_t* p_full = dp_full + 2;           // [2]  (128 arrivals) P^T written
  uint64_t* ds_full = p_full + 2;           // [2]  (128 arrivals) dS^T in shared memory, dP^T slot free
  uint64_t* dq_full = ds_full + 2;          // [2]  dQ^T of the tile is in the slot
  uint64_t* dq_read = dq_full + 2;          // [2]  (128 arrivals) slot free again
  uint64_t* dkv_full = dq_read + 2;         // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(dkv_full + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int* c = p.cta + static_cast<long long>(blockIdx.x) * 8;
  const int kv_row0 = c[0], kv_valid = c[1], kvh = c[2], list_off = c[3], list_cnt = c[4];
  const int ratio = p.Hq / p.Hkv;
  const int n_iter = list_cnt * ratio;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(kv_full, 1);
    for (int g = 0; g < 2; ++g) {
      mbar_init(&s_full[g], 1);
      mbar_init(&dp_full[g], 1);
      mbar_init(&p_full[g], 128);
      mbar_init(&ds_full[g], 128);
      mbar_init(&dq_full[g], 1);
      mbar_init(&dq_read[g], 128);
    }
    mbar_init(dkv_full, 1);
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
  constexpr uint32_t kColSlot = 0, kColDP = 128, kColDK = 256, kColDV = 384;  // slot / dP: + 64 * group

  if (warp == 0) {
    // ---------------------------------------------------------------- producer (whole warp)
    if (n_iter > 0) {
      if (lane == 0) {
        mbar_expect_tx(kv_full, 2 * Cfg::kKvTileBytes);
        for (int ch = 0; ch < D / 64; ++ch) {
          tma_load_2d(smem_k + ch * 16384, &tma_k, kv_full, kvh * D + ch * 64, kv_row0);
          tma_load_2d(smem_v + ch * 16384, &tma_v, kv_full, kvh * D + ch * 64, kv_row0);
        }
      }
      bool ok = true;
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % kBwdStages;
        const uint32_t ph = (it / kBwdStages) & 1;
        int okw = 1;
        if (lane == 0) okw = mbar_wait(&empty[s], ph ^ 1, p.status, kTimeoutEmpty) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) {
          ok = false;
          break;
        }
        const int* e = p.list + static_cast<long long>(list_off + it / ratio) * 4;
        const int q_row0 = e[0];
        const int head = kvh * ratio + it % ratio;
        float* st = smem_stat + s * 128;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int idx = lane + 32 * i;
          const long long t = static_cast<long long>(q_row0) + idx;
          const bool in = t < p.T;
          st[idx] = in ? p.lse[static_cast<long long>(head) * p.T + t] * 1.4426950408889634f : 0.f;
          st[64 + idx] = in ? p.delta[static_cast<long long>(head) * p.T + t] : 0.f;
        }
        __syncwarp();
        if (lane == 0) {
          uint8_t* sq = smem_qdo + s * 2 * Cfg::kQTileBytes;
          uint8_t* sdo = sq + Cfg::kQTileBytes;
          mbar_expect_tx(&full[s], 2 * Cfg::kQTileBytes);
          for (int ch = 0; ch < D / 64; ++ch) {
            tma_load_2d(sq + ch * QCH, &tma_q, &full[s], head * D + ch * 64, q_row0);
            tma_load_2d(sdo + ch * QCH, &tma_do, &full[s], head * D + ch * 64, q_row0);
          }
        }
      }
      if (!ok && lane == 0) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 100000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_st = umma_idesc_bf16(128, kBwdQTile, 0, 0);  // S^T, dP^T : A K-major, B K-major
      const uint32_t idesc_dv = umma_idesc_bf16(128, D, 0, 1);          // dV, dK    : A K-major, B MN-major
      const uint32_t idesc_dq = umma_idesc_bf16(128, kBwdQTile, 1, 1);  // dQ^T      : A MN-major, B MN-major
      const uint32_t ka = smem_u32(smem_k), va = smem_u32(smem_v);
      auto stage_q = [&](int s) { return smem_u32(smem_qdo + s * 2 * Cfg::kQTileBytes); };
      auto issue_st = [&](uint32_t a_base, uint32_t b_base, uint32_t tcol) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t aoff = (k / 4) * 16384 + (k % 4) * 32;
          const uint32_t boff = (k / 4) * QCH + (k % 4) * 32;
          umma_bf16_ss(tmem_base + tcol, umma_smem_desc(a_base + aoff, 0, 1024),
                       umma_smem_desc(b_base + boff, 0, 1024), idesc_st, k > 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutFull);
      // S^T and dP^T of the first tile of each group
      for (int j = 0; j < 2 && j < n_iter && ok; ++j) {
        ok = mbar_wait(&full[j % kBwdStages], 0, p.status, kTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        issue_st(ka, stage_q(j % kBwdStages), kColSlot + j * 64);
        tc_commit(&s_full[j]);
        issue_st(va, stage_q(j % kBwdStages) + Cfg::kQTileBytes, kColDP + j * 64);
        tc_commit(&dp_full[j]);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % kBwdStages;
        const int g = it & 1;
        const uint32_t par = (it >> 1) & 1;
        const uint32_t sq = stage_q(s), sdo = sq + Cfg::kQTileBytes;
        const uint32_t slot = tmem_base + kColSlot + g * 64;
        // dV += P^T dO
        if (!mbar_wait(&p_full[g], par, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBwdQTile / 16; ++k)
          umma_bf16_ts(tmem_base + kColDV, slot + k * 8, umma_smem_desc(sdo + k * 2048, QCH, 1024), idesc_dv,
                       (it > 0 || k > 0) ? 1u : 0u);
        // S^T and dP^T of the other group's next tile (its slot is free once dQ^T of tile it-1 has been read)
        if (it >= 1 && it + 1 < n_iter) {
          const int it1 = it + 1, g1 = g ^ 1, s1 = it1 % kBwdStages;
          if (!mbar_wait(&dq_read[g1], ((it - 1) >> 1) & 1, p.status, kTimeoutTmemEmpty) ||
              !mbar_wait(&full[s1], (it1 / kBwdStages) & 1, p.status, kTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          issue_st(ka, stage_q(s1), kColSlot + g1 * 64);
          tc_commit(&s_full[g1]);
          issue_st(va, stage_q(s1) + Cfg::kQTileBytes, kColDP + g1 * 64);
          tc_commit(&dp_full[g1]);
        }
        // dK += dS^T Q ; dQ^T = K^T dS^T (into the slot, whose P^T the dV product above has consumed: the
        // tensor core executes one CTA's MMAs in issue order)
        if (!mbar_wait(&ds_full[g], par, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dsa = smem_u32(smem_ds + g * Cfg::kDsBytes);
#pragma unroll
        for (int k = 0; k < kBwdQTile / 16; ++k)
          umma_bf16_ss(tmem_base + kColDK, umma_smem_desc(dsa + k * 32, 0, 1024),
                       umma_smem_desc(sq + k * 2048, QCH, 1024), idesc_dv, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k)
          umma_bf16_ss(slot, umma_smem_desc(ka + k * 2048, 16384, 1024), umma_smem_desc(dsa + k * 2048, 0, 1024),
                       idesc_dq, k > 0 ? 1u : 0u);
        tc_commit(&dq_full[g]);
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(dkv_full);
    }
  } else {
    // ---------------------------------------------------------------- softmax / gradient group
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;    // gradient group: tiles grp, grp + 2, ...
    const int r = quarter * 32 + lane;  // key row of the block (and head-dim index for dQ^T)
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_ok = r < kv_valid;
    bool ok = true;
    for (int it = grp; it < n_iter; it += 2) {
      const uint32_t par = (it >> 1) & 1;
      const int s = it % kBwdStages;
      const int* e = p.list + static_cast<long long>(list_off + it / ratio) * 4;
      const int q_row0 = e[0], q_valid = e[1], diag = e[2];
      const int head = kvh * ratio + it % ratio;
      const int c_min = (diag >= kBigDiag) ? 0 : max(0, r - diag);
      const float* st = smem_stat + s * 128;
      if (!mbar_wait(&full[s], (it / kBwdStages) & 1, p.status, kTimeoutFull) ||
          !mbar_wait(&s_full[grp], par, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_s = tmem_base + lane_off + kColSlot + grp * 64;
      float pr[kBwdQTile];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + h * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = h * 32 + i;
          const bool vis = row_ok && col >= c_min && col < q_valid;
          pr[col] = vis ? exp2f(__uint_as_float(v[i]) * p.scale_log2 - st[col]) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pr[h * 32 + 2 * i], pr[h * 32 + 2 * i + 1]);
        tmem_st_32x16(t_s + h * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[grp]);
      // dS^T
      if (!mbar_wait(&dp_full[grp], par, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint8_t* ds_row = smem_ds + grp * Cfg::kDsBytes + r * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_off + kColDP + grp * 64 + h * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = h * 32 + u * 8 + 2 * i;
            const float a = pr[col] > 0.f ? pr[col] * (__uint_as_float(v[u * 8 + 2 * i]) - st[64 + col]) * p.scale : 0.f;
            const float b = pr[col + 1] > 0.f
                                ? pr[col + 1] * (__uint_as_float(v[u * 8 + 2 * i + 1]) - st[64 + col + 1]) * p.scale
                                : 0.f;
            o[i] = pack_bf16x2(a, b);
          }
          const int unit = (h * 4 + u) ^ (r & 7);
          *reinterpret_cast<uint4*>(ds_row + unit * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[grp]);
      // dQ^T -> global accumulator (this thread holds head-dim index r for 64 query rows)
      if (!mbar_wait(&dq_full[grp], par, p.status, kTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float* dq = p.dq_acc + static_cast<long long>(q_row0) * p.ld_dq + static_cast<long long>(head) * D + r;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld_32x32(t_s + h * 32, v);
        tmem_ld_wait();
        if (r < D) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = h * 32 + i;
            if (col < q_valid) atomicAdd(dq + static_cast<long long>(col) * p.ld_dq, __uint_as_float(v[i]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&dq_read[grp]);
    }
    // dK / dV of this block.  The TMEM loads are warp collectives: every lane runs them, only the
    // global stores are predicated on the row being inside the block.
    ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    if (ok) {
      if (n_iter > 0) ok = mbar_wait(dkv_full, 0, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
      tc_fence_after();
      if (ok) {
        __nv_bfloat16* dkp = p.dk + (static_cast<long long>(kv_row0) + r) * p.ld_dk + static_cast<long long>(kvh) * D;
        __nv_bfloat16* dvp = p.dv + (static_cast<long long>(kv_row0) + r) * p.ld_dv + static_cast<long long>(kvh) * D;
        {
          const int which = grp;  // group 0 stores dK, group 1 stores dV
          __nv_bfloat16* dst = which ? dvp : dkp;
          const uint32_t col0 = which ? kColDV : kColDK;
#pragma unroll 1
          for (int h = 0; h < D / 32; ++h) {
            uint32_t v[32];
            if (n_iter > 0) {  // uniform across the CTA
              tmem_ld_32x32(tmem_base + lane_off + col0 + h * 32, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
                *reinterpret_cast<uint4*>(dst + h * 32 + q * 8) = o;
              }
            }
          }
        }
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

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]; one warp per (t, h).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                                  const __nv_bfloat16* __restrict__ d_o, long long lddo, float* __restrict__ delta,
                                  int T, int Hq, int D) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(T) * Hq) return;
  const int t = static_cast<int>(gw / Hq), h = static_cast<int>(gw % Hq);
  const __nv_bfloat16* a = o + t * ldo + static_cast<long long>(h) * D;
  const __nv_bfloat16* b = d_o + t * lddo + static_cast<long long>(h) * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    acc += x.x * y.x + x.y * y.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = acc;
}

}  // namespace apb

extern "C" {

// Backward of apb_attn_fwd for head_dim 128.
//   q/o/d_o [T, Hq*D], k/v [T, Hkv*D] bf16 with row strides ld*; lse [Hq,T] from the forward.
//   delta [Hq,T] fp32 scratch (written here); dq_acc [T, Hq*D] fp32 accumulator, zeroed by the caller;
//   dk/dv [T, Hkv*D] bf16 outputs.  cta/list are the tables of apb_rt_attn_bwd_work.
int apb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                 float* delta, float* dq_acc, void* dk, void* dv, const int* cta, int n_cta, const int* list, int T,
                 int Hq, int Hkv, int D, long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                 long long ld_dq, long long ld_dk, long long ld_dv, float scale, cudaStream_t stream) {
  using namespace apb;
  if (n_cta <= 0 || T <= 0) return 0;
  if (D != 128 || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (ld_dk % 8) || (ld_dv % 8) || Hq % Hkv)
    return kBadArgument;
  {
    const long long warps = static_cast<long long>(T) * Hq;
    const int grid = static_cast<int>((warps * 32 + 255) / 256);
    attn_delta_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(o), ldo,
                                                static_cast<const __nv_bfloat16*>(d_o), lddo, delta, T, Hq, D);
  }
  CUtensorMap tq, tdo, tk, tv;
  int rc = make_tmap_2d(&tq, q, 2, T, static_cast<uint64_t>(Hq) * D, ldq, 64, kBwdQTile);
  if (rc) return 1000 + rc;
  rc = make_tmap_2d(&tdo, d_o, 2, T, static_cast<uint64_t>(Hq) * D, lddo, 64, kBwdQTile);
  if (rc) return 2000 + rc;
  rc = make_tmap_2d(&tk, k, 2, T, static_cast<uint64_t>(Hkv) * D, ldk, 64, 128);
  if (rc) return 3000 + rc;
  rc = make_tmap_2d(&tv, v, 2, T, static_cast<uint64_t>(Hkv) * D, ldv, 64, 128);
  if (rc) return 4000 + rc;
  AttnBwdParams p;
  p.cta = cta;
  p.list = list;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.T = T;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.ld_dq = ld_dq;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.ld_dk = ld_dk;
  p.ld_dv = ld_dv;
  p.status = status_device_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         AttnBwdCfg<128>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  attn_bwd_kernel<128><<<n_cta, kBwdThreads, AttnBwdCfg<128>::kSmemBytes, stream>>>(tq, tdo, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}
}
