// Host-side AdamW for optimizer state that lives in (pinned) host memory.
//
// One pass over the shard: reads the fp32 gradient, updates both moments and the fp32 master weight in place and
// writes the bf16 parameter that goes back to the device.  The range is cut into contiguous chunks, one per worker
// thread; the loop body is branch-free so the compiler vectorises it.  The arithmetic is the same as the device
// kernel's (decoupled weight decay, bias-corrected moments, eps added after the square root).
//
// The reference gets this from DeepSpeed's CPU Adam when ``zero_optimization.offload_optimizer.device`` is ``cpu``
// (arctic_platform/integrations/verl/config/remote_backend/arctic.yaml:91, and the offload / reload fall-backs in
// arctic_platform/common/deepspeed_worker.py:955).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline uint16_t bf16_rne(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);   // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, inv_bias1, inv_bias2, gscale;
};

void adamw_range(float* __restrict__ w, float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g,
                 uint16_t* __restrict__ out, int64_t lo, int64_t hi, AdamArgs a) {
  const float decay = 1.0f - a.lr * a.wd;
  for (int64_t i = lo; i < hi; ++i) {
    const float gi = g[i] * a.gscale;
    const float mi = a.b1 * m[i] + (1.0f - a.b1) * gi;
    const float vi = a.b2 * v[i] + (1.0f - a.b2) * gi * gi;
    const float wi = w[i] * decay - a.lr * (mi * a.inv_bias1) / (std::sqrt(vi * a.inv_bias2) + a.eps);
    m[i] = mi;
    v[i] = vi;
    w[i] = wi;
    if (out) out[i] = bf16_rne(wi);
  }
}

}  // namespace

extern "C" {

// Returns 0, or -1 for bad arguments.  ``out_bf16`` may be null (no low-precision copy wanted).
int32_t apb_rt_cpu_adamw(float* w, float* m, float* v, const float* g, uint16_t* out_bf16, int64_t n, float lr,
                         float b1, float b2, float eps, float wd, float bias1, float bias2, float gscale,
                         int32_t threads) {
  if (!w || !m || !v || !g || n < 0 || bias1 <= 0.0f || bias2 <= 0.0f) return -1;
  if (n == 0) return 0;
  AdamArgs a{lr, b1, b2, eps, wd, 1.0f / bias1, 1.0f / bias2, gscale};
  int32_t hw = static_cast<int32_t>(std::thread::hardware_concurrency());
  if (threads <= 0) threads = hw > 0 ? hw : 1;
  const int64_t min_chunk = 1 << 16;
  threads = static_cast<int32_t>(std::max<int64_t>(1, std::min<int64_t>(threads, (n + min_chunk - 1) / min_chunk)));
  if (threads == 1) {
    adamw_range(w, m, v, g, out_bf16, 0, n, a);
    return 0;
  }
  const int64_t chunk = ((n + threads - 1) / threads + 15) & ~int64_t(15);
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int32_t t = 0; t < threads; ++t) {
    const int64_t lo = std::min<int64_t>(n, t * chunk), hi = std::min<int64_t>(n, lo + chunk);
    if (lo < hi) pool.emplace_back(adamw_range, w, m, v, g, out_bf16, lo, hi, a);
  }
  for (auto& th : pool) th.join();
  return 0;
}

// Sum of squares in double precision (for the gradient norm of a host-resident shard).
double apb_rt_cpu_sumsq(const float* g, int64_t n) {
  double acc = 0.0;
  for (int64_t i = 0; i < n; ++i) acc += static_cast<double>(g[i]) * g[i];
  return acc;
}

}  // extern "C"
