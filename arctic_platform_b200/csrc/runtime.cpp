// Host runtime of the package (no CUDA dependency): the pieces that sit on the
// critical path between kernels and would otherwise be Python loops.
//
//  * KV page allocator with reference counts (prefix sharing between the
//    rollouts of one prompt) for the sampler's paged cache.
//  * First-fit-decreasing token-budget micro-batching (same contract as
//    arctic_platform/rl/processors/microbatch.py:_ffd_allocate in the reference).
//  * ZoRRo layout tables: prompt grouping by hash + verification, and the
//    packed index tables (cu_seqlens for unique prompts / responses, per-response
//    prompt offsets, gather indices for predictor rows and labels) that the
//    attention and lm-head kernels consume.  The reference builds these with
//    per-segment Python loops and .item() calls (rl/zorro_train/zorro_train.py:564-722).
//  * Greedy cost-balanced partition of prompt groups across data-parallel ranks
//    (rl/zorro_train/seqlen_balancing.py:603-738).
//
// Everything is exported with C linkage and plain int32/int64 buffers so that
// Python reaches it through ctypes without copies.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <numeric>
#include <unordered_map>
#include <vector>

namespace {

struct PageAllocator {
  int32_t num_pages;
  std::vector<int32_t> free_list;
  std::vector<int32_t> refcnt;
  std::mutex mu;
};

inline uint64_t mix64(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  return h;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------ page allocator
void* apb_rt_pages_create(int32_t num_pages) {
  auto* a = new PageAllocator();
  a->num_pages = num_pages;
  a->refcnt.assign(num_pages, 0);
  a->free_list.resize(num_pages);
  for (int32_t i = 0; i < num_pages; ++i) a->free_list[i] = num_pages - 1 - i;  // pop yields 0,1,2,...
  return a;
}
void apb_rt_pages_destroy(void* h) { delete static_cast<PageAllocator*>(h); }
int32_t apb_rt_pages_free_count(void* h) {
  auto* a = static_cast<PageAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  return static_cast<int32_t>(a->free_list.size());
}
// Allocates n pages (refcount 1) into out[]; returns 0 or -1 when not enough pages (nothing allocated).
int32_t apb_rt_pages_alloc(void* h, int32_t n, int32_t* out) {
  auto* a = static_cast<PageAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  if (static_cast<int32_t>(a->free_list.size()) < n) return -1;
  for (int32_t i = 0; i < n; ++i) {
    const int32_t p = a->free_list.back();
    a->free_list.pop_back();
    a->refcnt[p] = 1;
    out[i] = p;
  }
  return 0;
}
// Adds one reference to each page (a new sequence sharing a prefix).
int32_t apb_rt_pages_retain(void* h, int32_t n, const int32_t* pages) {
  auto* a = static_cast<PageAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  for (int32_t i = 0; i < n; ++i) {
    if (pages[i] < 0 || pages[i] >= a->num_pages || a->refcnt[pages[i]] <= 0) return -1;
    a->refcnt[pages[i]]++;
  }
  return 0;
}
// Drops one reference; pages reaching zero return to the free list.  Returns number freed or -1.
int32_t apb_rt_pages_release(void* h, int32_t n, const int32_t* pages) {
  auto* a = static_cast<PageAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  int32_t freed = 0;
  for (int32_t i = 0; i < n; ++i) {
    const int32_t p = pages[i];
    if (p < 0 || p >= a->num_pages || a->refcnt[p] <= 0) return -1;
    if (--a->refcnt[p] == 0) {
      a->free_list.push_back(p);
      ++freed;
    }
  }
  return freed;
}
int32_t apb_rt_pages_refcount(void* h, int32_t page) {
  auto* a = static_cast<PageAllocator*>(h);
  std::lock_guard<std::mutex> g(a->mu);
  return (page < 0 || page >= a->num_pages) ? -1 : a->refcnt[page];
}

// ------------------------------------------------------------ FFD packing
// Items with sizes[n]; bins of capacity `cap`; at least `min_groups` bins and
// the bin count rounded up to a multiple of `divisor`.  group_of[n] receives
// the bin of each item.  Returns the number of bins, or -1 when an item is
// larger than the capacity.
int32_t apb_rt_ffd_pack(const int64_t* sizes, int32_t n, int64_t cap, int32_t min_groups, int32_t divisor,
                        int32_t* group_of) {
  std::vector<int32_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return sizes[a] > sizes[b]; });
  std::vector<int64_t> load;
  if (min_groups > 0) load.assign(min_groups, 0);
  for (int32_t idx : order) {
    if (sizes[idx] > cap) return -1;
    int32_t chosen = -1;
    if (min_groups > 0) {
      // while the mandatory bins exist, prefer the emptiest one that fits (keeps them balanced)
      int64_t best = INT64_MAX;
      for (size_t b = 0; b < load.size(); ++b)
        if (load[b] + sizes[idx] <= cap && load[b] < best) {
          best = load[b];
          chosen = static_cast<int32_t>(b);
        }
    } else {
      for (size_t b = 0; b < load.size(); ++b)
        if (load[b] + sizes[idx] <= cap) {
          chosen = static_cast<int32_t>(b);
          break;
        }
    }
    if (chosen < 0) {
      load.push_back(0);
      chosen = static_cast<int32_t>(load.size()) - 1;
    }
    load[chosen] += sizes[idx];
    group_of[idx] = chosen;
  }
  int32_t bins = static_cast<int32_t>(load.size());
  if (divisor > 1 && bins % divisor) bins += divisor - bins % divisor;
  return bins;
}

// ------------------------------------------------------------ ZoRRo grouping
// Rows of `prompts` ([B, P] int64, row stride `stride`) that are identical get
// the same group id (ids numbered by first appearance).  Hash first, then
// verify with memcmp so collisions cannot merge different prompts.
// Returns the number of groups.
int32_t apb_rt_group_prompts(const int64_t* prompts, int32_t B, int32_t P, int64_t stride, int32_t* group_of) {
  std::unordered_map<uint64_t, std::vector<int32_t>> buckets;  // hash -> representative rows
  std::vector<int32_t> rep_group;                               // group id of a representative row
  rep_group.assign(B, -1);
  int32_t groups = 0;
  for (int32_t b = 0; b < B; ++b) {
    const int64_t* row = prompts + static_cast<int64_t>(b) * stride;
    uint64_t h = 0x1234567ull;
    for (int32_t i = 0; i < P; ++i) h = mix64(h, static_cast<uint64_t>(row[i]));
    auto& reps = buckets[h];
    int32_t found = -1;
    for (int32_t r : reps) {
      if (std::memcmp(prompts + static_cast<int64_t>(r) * stride, row, sizeof(int64_t) * P) == 0) {
        found = rep_group[r];
        break;
      }
    }
    if (found < 0) {
      found = groups++;
      reps.push_back(b);
      rep_group[b] = found;
    }
    group_of[b] = found;
  }
  return groups;
}

// Greedy min-cost assignment of groups to `ranks` bins with an equal number of
// samples per rank when `equal_samples` is set (groups are split when needed
// by the caller; here a group is atomic).  cost[g], samples[g] -> rank_of[g].
// Returns 0, or -1 if equal sample counts cannot be met with atomic groups.
int32_t apb_rt_balance_groups(const double* cost, const int32_t* samples, int32_t G, int32_t ranks,
                              int32_t equal_samples, int32_t* rank_of) {
  std::vector<int32_t> order(G);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return cost[a] > cost[b]; });
  std::vector<double> load(ranks, 0.0);
  std::vector<int64_t> count(ranks, 0);
  int64_t total = 0;
  for (int32_t g = 0; g < G; ++g) total += samples[g];
  const int64_t per_rank = equal_samples ? total / ranks : INT64_MAX;
  if (equal_samples && total % ranks) return -1;
  for (int32_t g : order) {
    int32_t best = -1;
    for (int32_t r = 0; r < ranks; ++r) {
      if (count[r] + samples[g] > per_rank) continue;
      if (best < 0 || load[r] < load[best]) best = r;
    }
    if (best < 0) return -1;
    load[best] += cost[g];
    count[best] += samples[g];
    rank_of[g] = best;
  }
  return 0;
}

int32_t apb_rt_version() { return 1; }
}
