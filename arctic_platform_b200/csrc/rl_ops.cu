// Small fused kernels of the RL step that are not GEMM shaped:
//   * the token-mean GRPO / dual-clip PPO objective with its low-variance KL term: loss statistics AND the gradient
//     with respect to the log-probs in one pass over the tokens (the reference evaluates about thirty element-wise
//     torch kernels plus autograd, arctic_platform/integrations/verl/grpo_loss.py:93-210);
//   * the mixture-of-experts routing decision: scores (softmax or sigmoid, optional selection bias), top-k per token
//     and the tokens-per-expert histogram in one kernel (the reference: softmax + topk + bincount,
//     arctic_platform/model/implementations/qwen35/models/layers/moe.py:226-269).
// Both are memory bound: one read of their inputs, one write of their outputs.
#include "common.cuh"
#include "host_utils.cuh"

namespace apb {

struct GrpoArgs {
  const float* lp;        // [n] current log-probs
  const float* old_lp;    // [n]
  const float* adv;       // [n]
  const float* ref_lp;    // [n] or null (no KL term)
  const float* weight;    // [n] or null (per-token importance correction)
  const uint8_t* mask;    // [n] 0 / 1
  float* grad;            // [n] d loss / d lp for an upstream gradient of 1
  double* sums;           // [8]: tokens, clipped, sum(-log ratio), lower-clipped, sum(pg), sum(kl), 0, 0
  long long n;
  float clip_low, clip_high, clip_c, kl_coef, scale;
  int kl_kind;            // 0 none, 1 low_var_kl (k3), 2 kl (k1), 3 mse (k2), 4 abs
};

__global__ void __launch_bounds__(256) grpo_token_loss_kernel(const GrpoArgs a) {
  float s_tok = 0.f, s_clip = 0.f, s_kl_ratio = 0.f, s_lower = 0.f, s_pg = 0.f, s_kld = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < a.n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const bool on = a.mask[i] != 0;
    float g = 0.f;
    if (on) {
      const float lp = a.lp[i], adv = a.adv[i];
      const float raw = lp - a.old_lp[i];
      const float d = fminf(fmaxf(raw, -20.f), 20.f);
      const float dd = (raw >= -20.f && raw <= 20.f) ? 1.f : 0.f;     // derivative of the clamp
      const float ratio = __expf(d);
      const float l1 = -adv * ratio;
      const float rc = fminf(fmaxf(ratio, 1.f - a.clip_low), 1.f + a.clip_high);
      const float l2 = -adv * rc;
      const float g1 = -adv * ratio * dd;
      const float g2 = (ratio >= 1.f - a.clip_low && ratio <= 1.f + a.clip_high) ? g1 : 0.f;
      const float c1 = fmaxf(l1, l2);
      const float gc1 = (l1 > l2) ? g1 : ((l1 < l2) ? g2 : 0.5f * (g1 + g2));
      const float l3 = -adv * a.clip_c;
      float loss = c1, gl = gc1;
      bool lower = false;
      if (adv < 0.f) {
        lower = c1 > l3;
        loss = fminf(l3, c1);
        gl = (c1 < l3) ? gc1 : ((c1 > l3) ? 0.f : 0.5f * gc1);
      }
      const float w = a.weight ? a.weight[i] : 1.f;
      loss *= w;
      gl *= w;
      float kld = 0.f, gk = 0.f;
      if (a.kl_kind != 0 && a.ref_lp) {
        const float dk = lp - a.ref_lp[i];
        if (a.kl_kind == 1) {
          const float k = fminf(fmaxf(-dk, -20.f), 20.f);
          const float kin = (-dk >= -20.f && -dk <= 20.f) ? 1.f : 0.f;
          const float e = __expf(k);
          const float v = e - k - 1.f;
          kld = fminf(fmaxf(v, -10.f), 10.f);
          gk = (v >= -10.f && v <= 10.f) ? -(e - 1.f) * kin : 0.f;
        } else if (a.kl_kind == 2) {
          kld = dk;
          gk = 1.f;
        } else if (a.kl_kind == 3) {
          kld = 0.5f * dk * dk;
          gk = dk;
        } else {
          kld = fabsf(dk);
          gk = dk > 0.f ? 1.f : (dk < 0.f ? -1.f : 0.f);
        }
      }
      g = (gl + a.kl_coef * gk) * a.scale;
      s_tok += 1.f;
      s_clip += (l2 > l1) ? 1.f : 0.f;
      s_kl_ratio += -d;
      s_lower += lower ? 1.f : 0.f;
      s_pg += loss;
      s_kld += kld;
    }
    a.grad[i] = g;
  }
  __shared__ float red[6][8];
  float v[6] = {s_tok, s_clip, s_kl_ratio, s_lower, s_pg, s_kld};
#pragma unroll
  for (int k = 0; k < 6; ++k) v[k] = warp_sum(v[k]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < 6; ++k) red[k][warp] = v[k];
  }
  __syncthreads();
  if (threadIdx.x < 6) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[threadIdx.x][w];
    atomicAdd(a.sums + threadIdx.x, static_cast<double>(t));
  }
}

// One warp per token.  scores = softmax(logits) or sigmoid(logits); selection on scores + bias; k rounds of warp
// arg-max (ties go to the lower expert index, like a stable descending sort).  E <= 32 * kRouteMaxPerLane.
constexpr int kRouteMaxPerLane = 16;
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int T, int E, int k,
                 int sigmoid, long long* __restrict__ idx_out, int* __restrict__ counts) {
  const long long tok = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= T) return;
  const float* row = logits + tok * ld;
  float sc[kRouteMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kRouteMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    sc[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, sc[j]);
  }
  if (!sigmoid) {
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      sc[j] = e < E ? __expf(sc[j] - mx) : 0.f;
      s += sc[j];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) sc[j] *= inv;
  } else {
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) sc[j] = 1.f / (1.f + __expf(-sc[j]));
  }
#pragma unroll
  for (int j = 0; j < kRouteMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    sc[j] = e < E ? sc[j] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (sc[j] > best) {          // ascending e inside a lane: the first maximum is the lowest index
        best = sc[j];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) {
        best = ob;
        be = oe;
      }
    }
    if (lane == 0) {
      idx_out[tok * k + r] = be;
      if (counts) atomicAdd(counts + be, 1);
    }
    if ((be & 31) == lane) sc[be >> 5] = -INFINITY;   // taken
  }
}

// Tile tables of the two grouped expert GEMMs from the tokens-per-expert histogram, on the device: expert e owns
// counts[e] consecutive rows of the expert-sorted activations; every 128-row block of an expert times every 128-column
// block of the output is one tile {m0, m_end, b_row_offset, n_tile}.  One block; thread t handles expert t (+ stride).
__global__ void __launch_bounds__(256)
moe_group_tiles_kernel(const int* __restrict__ counts, int E, int n_out1, int n_out2, int4* __restrict__ tiles1,
                       int4* __restrict__ tiles2, int max_tiles1, int max_tiles2, int* __restrict__ n_tiles,
                       int* __restrict__ offsets) {
  __shared__ int row_off[513];
  __shared__ int blk_off[513];
  if (threadIdx.x == 0) {
    int r = 0, b = 0;
    for (int e = 0; e < E; ++e) {
      row_off[e] = r;
      blk_off[e] = b;
      r += counts[e];
      b += (counts[e] + 127) / 128;
    }
    row_off[E] = r;
    blk_off[E] = b;
  }
  __syncthreads();
  const int nt1 = (n_out1 + 127) / 128, nt2 = (n_out2 + 127) / 128;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (offsets) offsets[e] = row_off[e];
    const int c = counts[e], r0 = row_off[e];
    int b = blk_off[e];
    for (int m0 = r0; m0 < r0 + c; m0 += 128, ++b) {
      for (int nt = 0; nt < nt1; ++nt)
        if (b * nt1 + nt < max_tiles1) tiles1[b * nt1 + nt] = make_int4(m0, r0 + c, e * n_out1, nt);
      for (int nt = 0; nt < nt2; ++nt)
        if (b * nt2 + nt < max_tiles2) tiles2[b * nt2 + nt] = make_int4(m0, r0 + c, e * n_out2, nt);
    }
  }
  if (threadIdx.x == 0) {
    if (offsets) offsets[E] = row_off[E];
    n_tiles[0] = min(blk_off[E] * nt1, max_tiles1);
    n_tiles[1] = min(blk_off[E] * nt2, max_tiles2);
  }
}

// Routing plan of an expert layer whose rows are laid out expert-major with every expert's segment padded to a
// multiple of 64 rows (padding rows hold zeros), from the tokens-per-expert histogram, on the device.  Writes
//   seg_start [E + 1]: first padded row of every expert (seg_start[E] = rows in use);
//   row-block tables {m0, m_end, b_row_offset, n_tile} (+ extension records {c_row_off, kb0, kb1, bk_off}) for the
//   four GEMMs that walk 128-row blocks of the segments:
//     0 gate/up forward   (N = 2I, B = Wgu  stacked [E * 2I, H], b_row_offset = e * 2I)
//     1 down forward      (N = H,  B = Wdn  stacked [E * H, I],  b_row_offset = e * H)
//     2 d act = dY @ Wdn  (N = I,  B stacked [E * H, I] read K-major, bk_off = e * H)
//     3 d x = dGU @ Wgu   (N = H,  B stacked [E * 2I, H] read K-major, bk_off = e * 2I)
//   and the two weight-gradient tables, whose tile COUNT is static (every expert x every 128 x 128 block of its weight)
//   and whose K walk is the expert's 64-row blocks:
//     4 dWdn[e] [H, I]  += dY[seg]^T  @ act[seg]      5 dWgu[e] [2I, H] += dGU[seg]^T @ x[seg]
// n_tiles [4]: live sizes of tables 0-3.  One block; the prefix sums are serial over E <= 512 experts.
struct MoePlanOut {
  int4* map[6];
  int4* ext[6];
  int max_tiles[4];
};

__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ counts, int E, int H, int I, MoePlanOut out, int* __restrict__ seg_start,
                int* __restrict__ n_tiles) {
  __shared__ int row_off[513];
  __shared__ int blk_off[513];
  if (threadIdx.x == 0) {
    int r = 0, b = 0;
    for (int e = 0; e < E; ++e) {
      row_off[e] = r;
      blk_off[e] = b;
      const int padded = (max(counts[e], 0) + 63) / 64 * 64;
      r += padded;
      b += (padded + 127) / 128;
    }
    row_off[E] = r;
    blk_off[E] = b;
  }
  __syncthreads();
  const int I2 = 2 * I;
  const int nt[4] = {(I2 + 127) / 128, (H + 127) / 128, (I + 127) / 128, (H + 127) / 128};
  const int b_off_mul[4] = {I2, H, 0, 0};      // b_row_offset = e * this
  const int bk_mul[4] = {0, 0, H, I2};         // bk_off = e * this
  for (int e = threadIdx.x; e <= E; e += blockDim.x) seg_start[e] = row_off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int r0 = row_off[e], r1 = row_off[e + 1];
    int b = blk_off[e];
    for (int m0 = r0; m0 < r1; m0 += 128, ++b) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        for (int t = 0; t < nt[g]; ++t) {
          const int i = b * nt[g] + t;
          if (i < out.max_tiles[g]) {
            out.map[g][i] = make_int4(m0, r1, e * b_off_mul[g], t);
            out.ext[g][i] = make_int4(0, 0, -1, e * bk_mul[g]);
          }
        }
      }
    }
    // weight gradients: tile (e, mt, nt) at a fixed position
    const int kb0 = r0 / 64, kb1 = r1 / 64;
    const int mt_dn = (H + 127) / 128, nt_dn = (I + 127) / 128;
    for (int mt = 0; mt < mt_dn; ++mt)
      for (int t = 0; t < nt_dn; ++t) {
        const int i = (e * mt_dn + mt) * nt_dn + t;
        out.map[4][i] = make_int4(mt * 128, H, 0, t);
        out.ext[4][i] = make_int4(e * H, kb0, kb1, 0);
      }
    const int mt_gu = (I2 + 127) / 128, nt_gu = (H + 127) / 128;
    for (int mt = 0; mt < mt_gu; ++mt)
      for (int t = 0; t < nt_gu; ++t) {
        const int i = (e * mt_gu + mt) * nt_gu + t;
        out.map[5][i] = make_int4(mt * 128, I2, 0, t);
        out.ext[5][i] = make_int4(e * I2, kb0, kb1, 0);
      }
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int g = 0; g < 4; ++g) n_tiles[g] = min(blk_off[E] * nt[g], out.max_tiles[g]);
  }
}

}  // namespace apb

extern "C" {

// counts [E] int32 on the device (E <= 512), hidden size H, expert width I.  maps / exts: 6 device tables each (see
// moe_plan_kernel); max_tiles [4]: capacity of tables 0-3 (tables 4 and 5 hold E * ceil(H/128) * ceil(I/128) and
// E * ceil(2I/128) * ceil(H/128) records).  seg_start [E + 1], n_tiles [4]: device outputs.
int apb_moe_plan(const int* counts, int E, int H, int I, void* const* maps, void* const* exts, const int* max_tiles,
                 int* seg_start, int* n_tiles, cudaStream_t s) {
  using namespace apb;
  if (!counts || !maps || !exts || !max_tiles || !seg_start || !n_tiles || E < 1 || E > 512 || H < 1 || I < 1)
    return kBadArgument;
  MoePlanOut o;
  for (int g = 0; g < 6; ++g) {
    if (!maps[g] || !exts[g]) return kBadArgument;
    o.map[g] = static_cast<int4*>(maps[g]);
    o.ext[g] = static_cast<int4*>(exts[g]);
  }
  for (int g = 0; g < 4; ++g) o.max_tiles[g] = max_tiles[g];
  moe_plan_kernel<<<1, 256, 0, s>>>(counts, E, H, I, o, seg_start, n_tiles);
  return static_cast<int>(cudaGetLastError());
}

// counts [E] int32 (E <= 512) -> tile tables of the gate/up (n_out1 columns per expert) and down (n_out2) grouped
// GEMMs, their live sizes n_tiles[2] and, optionally, the row offset of every expert (offsets [E + 1]).
int apb_moe_group_tiles(const int* counts, int E, int n_out1, int n_out2, void* tiles1, void* tiles2, int max_tiles1,
                        int max_tiles2, int* n_tiles, int* offsets, cudaStream_t s) {
  using namespace apb;
  if (!counts || !tiles1 || !tiles2 || !n_tiles || E < 1 || E > 512) return kBadArgument;
  moe_group_tiles_kernel<<<1, 256, 0, s>>>(counts, E, n_out1, n_out2, static_cast<int4*>(tiles1),
                                           static_cast<int4*>(tiles2), max_tiles1, max_tiles2, n_tiles, offsets);
  return static_cast<int>(cudaGetLastError());
}

// Token-mean GRPO / dual-clip PPO loss terms with gradient.  All vectors fp32 [n] on the device except mask (bytes).
// sums: 8 doubles, ZEROED BY THE CALLER.  loss = (sums[4] + kl_coef * sums[5]) * scale.
int apb_grpo_token_loss(const float* lp, const float* old_lp, const float* adv, const float* ref_lp, const float* weight,
                        const void* mask, float* grad, double* sums, long long n, float clip_low, float clip_high,
                        float clip_c, int kl_kind, float kl_coef, float scale, cudaStream_t s) {
  using namespace apb;
  if (n <= 0) return 0;
  if (!lp || !old_lp || !adv || !mask || !grad || !sums || kl_kind < 0 || kl_kind > 4) return kBadArgument;
  if (kl_kind != 0 && !ref_lp) return kBadArgument;
  GrpoArgs a{lp, old_lp, adv, ref_lp, weight, static_cast<const uint8_t*>(mask), grad, sums, n,
             clip_low, clip_high, clip_c, kl_coef, scale, kl_kind};
  long long g = (n + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  grpo_token_loss_kernel<<<static_cast<int>(g < cap ? g : cap), 256, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// logits [T, E] fp32 (row stride ld); bias [E] fp32 or null; idx_out [T, k] int64; counts [E] int32 or null (added to).
int apb_moe_route(const float* logits, long long ld, const float* bias, int T, int E, int k, int sigmoid,
                  long long* idx_out, int* counts, cudaStream_t s) {
  using namespace apb;
  if (T <= 0) return 0;
  if (!logits || !idx_out || E < 1 || E > 32 * kRouteMaxPerLane || k < 1 || k > E) return kBadArgument;
  const long long threads = static_cast<long long>(T) * 32;
  moe_route_kernel<<<static_cast<int>((threads + 255) / 256), 256, 0, s>>>(logits, ld, bias, T, E, k, sigmoid, idx_out,
                                                                            counts);
  return static_cast<int>(cudaGetLastError());
}
}
