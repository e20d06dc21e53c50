// Work-table builders for the segment attention kernels (host side, no CUDA).
//
// A "segment" is a run of query rows of the packed token axis with two key
// ranges: a fully visible prefix range (the group's shared prompt under ZoRRo)
// and its own range under a bottom-right aligned causal mask:
//     seg = {q_start, q_len, pre_start, pre_len, own_start, own_len}
// Plain packed causal attention is the special case pre_len = 0, own = q.
//
// Forward table: one entry per (query tile of 128 rows, KV head, pair of query
// heads), longest first.  Backward table: one entry per (key block of 128 rows,
// KV head) with the list of 64-row query tiles that can see the block, so that
// dK/dV of a shared prompt block are accumulated by ONE CTA over all rollouts of
// the group and written once, without atomics and without replicated K/V.
#include <algorithm>
#include <cstdint>
#include <map>
#include <numeric>
#include <vector>

namespace {
constexpr int kQTileFwd = 128;
constexpr int kKvBlock = 128;
constexpr int kQTileBwd = 64;
constexpr int kBig = 1 << 28;

struct Seg {
  int32_t q_start, q_len, pre_start, pre_len, own_start, own_len;
};
}  // namespace

extern "C" {

// Returns the number of forward entries; writes at most `cap` entries of 8 int32 to `out`
// (call with cap = 0 to size the buffer).
int64_t apb_rt_attn_fwd_work(const int32_t* segs, int32_t S, int32_t Hq, int32_t Hkv, int32_t* out, int64_t cap) {
  const Seg* sg = reinterpret_cast<const Seg*>(segs);
  const int ratio = Hq / Hkv;
  const int pairs = (ratio + 1) / 2;
  struct Item {
    int32_t v[8];
    int64_t cost;
  };
  std::vector<Item> items;
  for (int s = 0; s < S; ++s) {
    const Seg& g = sg[s];
    const int delta = g.own_len - g.q_len;
    for (int t0 = 0; t0 < g.q_len; t0 += kQTileFwd) {
      const int q_valid = std::min(kQTileFwd, g.q_len - t0);
      int own_vis = std::min<int>(g.own_len, t0 + q_valid + delta);
      if (own_vis < 0) own_vis = 0;
      const int64_t cost = (g.pre_len + kKvBlock - 1) / kKvBlock + (own_vis + kKvBlock - 1) / kKvBlock;
      if (cost == 0) continue;
      for (int kvh = 0; kvh < Hkv; ++kvh) {
        for (int pi = 0; pi < pairs; ++pi) {
          const int head0 = kvh * ratio + 2 * pi;
          const int pair = (2 * pi + 1 < ratio) ? 1 : 0;
          Item it;
          it.v[0] = g.q_start + t0;
          it.v[1] = q_valid;
          it.v[2] = g.pre_start;
          it.v[3] = g.pre_len;
          it.v[4] = g.own_start;
          it.v[5] = own_vis;
          it.v[6] = t0 + delta;
          it.v[7] = head0 | (pair << 16);
          it.cost = cost;
          items.push_back(it);
        }
      }
    }
  }
  std::stable_sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.cost > b.cost; });
  const int64_t n = static_cast<int64_t>(items.size());
  for (int64_t i = 0; i < n && i < cap; ++i) std::copy(items[i].v, items[i].v + 8, out + i * 8);
  return n;
}

// Backward tables.  cta_out: [n_cta][8] = {kv_row0, kv_valid, kvh, list_off, list_cnt, 0, 0, 0};
// list_out: [n_list][4] = {q_row0, q_valid, diag_rel, 0} where key row r of the block is visible to
// query column c of the tile iff r <= c + diag_rel.  counts[0] = n_cta, counts[1] = n_list.
// Returns 0, or -1 when two key ranges overlap without sharing their start (unsupported layout).
int32_t apb_rt_attn_bwd_work(const int32_t* segs, int32_t S, int32_t Hkv, int32_t* cta_out, int64_t cta_cap,
                             int32_t* list_out, int64_t list_cap, int64_t* counts) {
  const Seg* sg = reinterpret_cast<const Seg*>(segs);
  struct Tile {
    int32_t q_row0, q_valid, diag;
  };
  struct Range {
    int32_t len = 0;
    std::vector<std::pair<int32_t, bool>> users;  // (segment, uses it as prefix)
  };
  std::map<int32_t, Range> ranges;  // by start row
  for (int s = 0; s < S; ++s) {
    if (sg[s].pre_len > 0) {
      Range& r = ranges[sg[s].pre_start];
      r.len = std::max(r.len, sg[s].pre_len);
      r.users.push_back({s, true});
    }
    if (sg[s].own_len > 0) {
      Range& r = ranges[sg[s].own_start];
      r.len = std::max(r.len, sg[s].own_len);
      r.users.push_back({s, false});
    }
  }
  int32_t prev_end = INT32_MIN;
  for (auto& kv : ranges) {
    if (kv.first < prev_end) return -1;
    prev_end = kv.first + kv.second.len;
  }
  struct Block {
    int32_t kv_row0, kv_valid;
    std::vector<Tile> tiles;
  };
  std::vector<Block> blocks;
  for (auto& kv : ranges) {
    const int32_t start = kv.first;
    const Range& r = kv.second;
    const int nb = (r.len + kKvBlock - 1) / kKvBlock;
    const size_t base = blocks.size();
    for (int b = 0; b < nb; ++b) blocks.push_back({start + b * kKvBlock, std::min(kKvBlock, r.len - b * kKvBlock), {}});
    for (auto& u : r.users) {
      const Seg& g = sg[u.first];
      const int range_len = u.second ? g.pre_len : g.own_len;
      const int nbu = (range_len + kKvBlock - 1) / kKvBlock;
      const int delta = g.own_len - g.q_len;
      for (int t0 = 0; t0 < g.q_len; t0 += kQTileBwd) {
        const int q_valid = std::min(kQTileBwd, g.q_len - t0);
        for (int b = 0; b < nbu; ++b) {
          int diag;
          if (u.second) {
            diag = kBig;
          } else {
            diag = t0 + delta - b * kKvBlock;
            if (diag + q_valid - 1 < 0) continue;  // whole tile is above the diagonal for this block
          }
          // a user with a shorter range than the merged one only sees its own rows; the kernel masks by
          // kv_valid of the merged block, so differing lengths on one start are rejected here
          if (range_len != r.len) return -1;
          blocks[base + b].tiles.push_back({g.q_start + t0, q_valid, diag});
        }
      }
    }
  }
  std::vector<size_t> order(blocks.size());
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(),
                   [&](size_t a, size_t b) { return blocks[a].tiles.size() > blocks[b].tiles.size(); });
  int64_t n_cta = 0, n_list = 0;
  for (size_t oi : order) {
    const Block& bl = blocks[oi];
    const int64_t off = n_list;
    for (const Tile& t : bl.tiles) {
      if (n_list < list_cap) {
        int32_t* d = list_out + n_list * 4;
        d[0] = t.q_row0;
        d[1] = t.q_valid;
        d[2] = t.diag;
        d[3] = 0;
      }
      ++n_list;
    }
    for (int kvh = 0; kvh < Hkv; ++kvh) {
      if (n_cta < cta_cap) {
        int32_t* d = cta_out + n_cta * 8;
        d[0] = bl.kv_row0;
        d[1] = bl.kv_valid;
        d[2] = kvh;
        d[3] = static_cast<int32_t>(off);
        d[4] = static_cast<int32_t>(bl.tiles.size());
        d[5] = d[6] = d[7] = 0;
      }
      ++n_cta;
    }
  }
  counts[0] = n_cta;
  counts[1] = n_list;
  return 0;
}
}
