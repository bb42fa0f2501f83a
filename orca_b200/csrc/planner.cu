// Offline cache planning (MRD / LRU / 2Q).  The neighbour tables of every batch come from one
// large launch of the sampling kernel; this file holds the sequential part, which walks the batches
// in order on the host: the split of each batch's neighbour table into in-batch and out-of-batch
// occurrences, the per-node occurrence lists, and the three replacement policies.
//
// Two pieces of numba behaviour are part of the observable result of the reference planners and are
// reproduced here: the order in which its nopython np.argsort leaves equal keys (an unstable
// median-of-three quicksort that finishes ranges shorter than 16 by insertion), and the stream of its
// private MT19937 behind np.random.choice(..., replace=False) (a Fisher-Yates shuffle, first k kept).
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"

namespace orca {
namespace plan {

// ------------------------------------------------------------------------------ random stream
class Twister {
 public:
  explicit Twister(uint32_t seed) {
    s_[0] = seed;
    for (uint32_t i = 1; i < N; ++i) s_[i] = 1812433253u * (s_[i - 1] ^ (s_[i - 1] >> 30)) + i;
    pos_ = N;
  }
  uint32_t next() {
    if (pos_ >= N) refill();
    uint32_t y = s_[pos_++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    return y ^ (y >> 18);
  }
  // uniform integer in [0, n): draw the low bits needed for n-1, redraw while >= n
  int64_t below(int64_t n) {
    if (n <= 1) return 0;
    int bits = 64 - __builtin_clzll((unsigned long long)(n - 1));
    while (true) {
      uint64_t r;
      if (bits <= 32) {
        r = next() & (0xffffffffu >> (32 - bits));
      } else {
        uint64_t hi = next() & (0xffffffffu >> (64 - bits));
        r = (hi << 32) | next();
      }
      if ((int64_t)r < n) return (int64_t)r;
    }
  }
  template <class T>
  void shuffle(std::vector<T> &x) {
    for (int64_t i = (int64_t)x.size() - 1; i > 0; --i) std::swap(x[i], x[below(i + 1)]);
  }

 private:
  static constexpr uint32_t N = 624, M = 397;
  void refill() {
    for (uint32_t i = 0; i < N; ++i) {
      uint32_t y = (s_[i] & 0x80000000u) | (s_[(i + 1) % N] & 0x7fffffffu);
      s_[i] = s_[(i + M) % N] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    pos_ = 0;
  }
  uint32_t s_[N];
  uint32_t pos_;
};

// ------------------------------------------------------------------------------ argsort order
// Index permutation that orders `key` exactly as numba's quicksort-based argsort does.
template <class T>
class TieOrderSort {
 public:
  void run(const T *key, int64_t n, std::vector<int64_t> &idx) {
    key_ = key;
    idx.resize(n);
    for (int64_t i = 0; i < n; ++i) idx[i] = i;
    if (n < 2) return;
    r_ = idx.data();
    std::vector<std::pair<int64_t, int64_t>> todo;
    todo.emplace_back(0, n - 1);
    while (!todo.empty()) {
      auto [lo, hi] = todo.back();
      todo.pop_back();
      while (hi - lo >= 15) {
        const int64_t p = split(lo, hi);
        if (hi - p > p - lo) {  // keep working on the smaller side, park the larger
          if (hi > p) todo.emplace_back(p + 1, hi);
          hi = p - 1;
        } else {
          if (p > lo) todo.emplace_back(lo, p - 1);
          lo = p + 1;
        }
      }
      insertion(lo, hi);
    }
  }

 private:
  const T &k(int64_t pos) const { return key_[r_[pos]]; }
  void insertion(int64_t lo, int64_t hi) {
    for (int64_t i = lo + 1; i <= hi; ++i) {
      const int64_t moving = r_[i];
      const T v = key_[moving];
      int64_t j = i;
      for (; j > lo && v < k(j - 1); --j) r_[j] = r_[j - 1];
      r_[j] = moving;
    }
  }
  int64_t split(int64_t lo, int64_t hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (k(mid) < k(lo)) std::swap(r_[lo], r_[mid]);
    if (k(hi) < k(mid)) std::swap(r_[hi], r_[mid]);
    if (k(mid) < k(lo)) std::swap(r_[lo], r_[mid]);
    const T pivot = k(mid);
    std::swap(r_[hi], r_[mid]);  // pivot parked at the right end
    int64_t i = lo, j = hi - 1;
    while (true) {
      while (i < hi && k(i) < pivot) ++i;
      while (j >= lo && pivot < k(j)) --j;
      if (i >= j) break;
      std::swap(r_[i], r_[j]);
      ++i;
      --j;
    }
    std::swap(r_[i], r_[hi]);
    return i;
  }
  const T *key_ = nullptr;
  int64_t *r_ = nullptr;
};

// ------------------------------------------------------------------------------ batch lists
// What utils/cache.py:19-89 (read_batches) extracts from the sampled tables.
struct BatchLists {
  int64_t n_batches = 0;
  std::vector<int64_t> tgt_off, ngh_off;  // per batch
  std::vector<int32_t> tgt;               // ascending unique query nodes of the batch
  std::vector<int32_t> ngh;               // out-of-batch neighbour occurrences, table order
  // per node: (batch, kind) records, kind 0 = target, 1 = out-of-batch neighbour; ascending batch
  std::vector<int64_t> occ_off;
  std::vector<int32_t> occ_batch;
  std::vector<uint8_t> occ_kind;
};

static void build_lists(const int64_t *src, const int64_t *dst, int64_t n_edges, int bs, int k,
                        const int32_t *nbr, int64_t n_nodes, bool want_occ, BatchLists &L) {
  const int64_t nb = (n_edges + bs - 1) / bs;
  L.n_batches = nb;
  L.tgt_off.assign(nb + 1, 0);
  L.ngh_off.assign(nb + 1, 0);
  L.tgt.clear();
  L.ngh.clear();
  std::vector<int32_t> stamp(n_nodes, -1);      // last batch in which the node was a target
  std::vector<int32_t> seen_out(n_nodes, -1);   // last batch in which it was an out-of-batch neighbour
  std::vector<int32_t> occ_count(want_occ ? n_nodes : 0, 0);
  std::vector<int32_t> uniq_out;                // per batch, insertion order (sorted later per node anyway)
  std::vector<int64_t> out_off(nb + 1, 0);
  std::vector<int32_t> out_all;
  for (int64_t b = 0; b < nb; ++b) {
    const int64_t s = b * bs, e = std::min(n_edges, s + bs), m = e - s;
    const size_t t0 = L.tgt.size();
    for (int64_t i = 0; i < 2 * m; ++i) {
      const int32_t v = (int32_t)(i < m ? src[s + i] : dst[s + i - m]);
      if (stamp[v] != b) {
        stamp[v] = (int32_t)b;
        L.tgt.push_back(v);
      }
    }
    std::sort(L.tgt.begin() + t0, L.tgt.end());
    L.tgt_off[b + 1] = (int64_t)L.tgt.size();
    const int32_t *tab = nbr + (size_t)2 * s * k;
    for (int64_t i = 0; i < 2 * m * k; ++i) {
      const int32_t v = tab[i];
      if (v == 0 || stamp[v] == b) continue;
      L.ngh.push_back(v);
      if (want_occ && seen_out[v] != b) {
        seen_out[v] = (int32_t)b;
        out_all.push_back(v);
      }
    }
    L.ngh_off[b + 1] = (int64_t)L.ngh.size();
    out_off[b + 1] = (int64_t)out_all.size();
  }
  if (!want_occ) return;
  // occurrence lists: counting pass, then a fill pass in batch order (so each list ascends)
  for (int64_t b = 0; b < nb; ++b) {
    for (int64_t i = L.tgt_off[b]; i < L.tgt_off[b + 1]; ++i) occ_count[L.tgt[i]]++;
    for (int64_t i = out_off[b]; i < out_off[b + 1]; ++i) occ_count[out_all[i]]++;
  }
  L.occ_off.assign(n_nodes + 1, 0);
  for (int64_t v = 0; v < n_nodes; ++v) L.occ_off[v + 1] = L.occ_off[v] + occ_count[v] + 1;  // + terminator
  L.occ_batch.resize(L.occ_off[n_nodes]);
  L.occ_kind.resize(L.occ_off[n_nodes]);
  std::vector<int64_t> cur(L.occ_off.begin(), L.occ_off.end() - 1);
  for (int64_t b = 0; b < nb; ++b) {
    for (int64_t i = L.tgt_off[b]; i < L.tgt_off[b + 1]; ++i) {
      const int64_t p = cur[L.tgt[i]]++;
      L.occ_batch[p] = (int32_t)b;
      L.occ_kind[p] = 0;
    }
    for (int64_t i = out_off[b]; i < out_off[b + 1]; ++i) {
      const int64_t p = cur[out_all[i]]++;
      L.occ_batch[p] = (int32_t)b;
      L.occ_kind[p] = 1;
    }
  }
  for (int64_t v = 0; v < n_nodes; ++v) {  // "never again" terminator
    L.occ_batch[cur[v]] = (int32_t)nb;
    L.occ_kind[cur[v]] = 2;
  }
}

}  // namespace plan
}  // namespace orca

namespace orca {
namespace plan {

struct PlanOut {
  int32_t *flat;
  int64_t *off;
  int64_t cap;
  int64_t used = 0;
  bool overflow = false;
  int32_t *begin_batch(int64_t b) {
    off[b] = used;
    return flat + used;
  }
  bool room(int64_t n) {
    if (used + n > cap) overflow = true;
    return !overflow;
  }
};

struct Stats {
  double reuse = 0, recompute = 0, dist = 0;
};

// utils/cache.py:92-166.  Candidates of a batch = uncached out-of-batch neighbours + cached nodes +
// targets (ascending, unique); key = batches until the next use as a NEIGHBOUR, or 1e8+1 if the
// node is next needed as a target or never; the first `budget` of the tie-order argsort stay cached.
static void solve_mrd(const BatchLists &L, int64_t n_nodes, int64_t budget, PlanOut &out, Stats &st) {
  const int64_t FAR = 100000001;
  std::vector<uint8_t> cached(n_nodes, 0), fresh(n_nodes, 0), listed(n_nodes, 0);
  std::vector<double> since(n_nodes, 0.0);
  std::vector<int64_t> cursor(L.occ_off.begin(), L.occ_off.end() - 1);
  std::vector<int32_t> held;  // ids currently cached
  std::vector<int32_t> cand, fresh_ids;
  std::vector<int64_t> key, order;
  TieOrderSort<int64_t> sorter;
  for (int64_t b = 0; b < L.n_batches; ++b) {
    cand.clear();
    fresh_ids.clear();
    auto add = [&](int32_t v) {
      if (!listed[v]) { listed[v] = 1; cand.push_back(v); }
    };
    for (int64_t i = L.ngh_off[b]; i < L.ngh_off[b + 1]; ++i) {
      const int32_t v = L.ngh[i];
      if (cached[v]) { st.reuse += 1; st.dist += (double)b - since[v]; }
      else { st.recompute += 1; add(v); if (!fresh[v]) { fresh[v] = 1; fresh_ids.push_back(v); } }
    }
    for (int32_t v : held) add(v);
    for (int64_t i = L.tgt_off[b]; i < L.tgt_off[b + 1]; ++i) {
      const int32_t v = L.tgt[i];
      add(v);
      if (!fresh[v]) { fresh[v] = 1; fresh_ids.push_back(v); }
    }
    std::sort(cand.begin(), cand.end());
    key.resize(cand.size());
    for (size_t i = 0; i < cand.size(); ++i) {
      const int32_t v = cand[i];
      int64_t c = cursor[v];
      while (L.occ_batch[c] <= b) ++c;
      cursor[v] = c;
      key[i] = L.occ_kind[c] == 1 ? (int64_t)L.occ_batch[c] - b : FAR;
      listed[v] = 0;
    }
    sorter.run(key.data(), (int64_t)key.size(), order);
    for (int32_t v : held) cached[v] = 0;
    held.clear();
    const int64_t keep = std::min<int64_t>(budget, (int64_t)cand.size());
    int32_t *dst = out.begin_batch(b);
    if (!out.room(keep)) return;
    for (int64_t i = 0; i < keep; ++i) {
      const int32_t v = cand[order[i]];
      dst[i] = v;
      cached[v] = 1;
      held.push_back(v);
      if (fresh[v]) since[v] = (double)b;
    }
    out.used += keep;
    for (int32_t v : fresh_ids) fresh[v] = 0;
  }
  out.off[L.n_batches] = out.used;
}

// ids with flag set, ascending
static void ascending_set(const std::vector<uint8_t> &flag, std::vector<int64_t> &ids) {
  ids.clear();
  for (size_t v = 0; v < flag.size(); ++v)
    if (flag[v]) ids.push_back((int64_t)v);
}

// utils/cache.py:338-403
static void solve_lru(const BatchLists &L, int64_t n_nodes, int64_t budget, uint32_t seed, PlanOut &out,
                      Stats &st) {
  Twister rng(seed);
  std::vector<uint8_t> cached(n_nodes, 0), listed(n_nodes, 0);
  std::vector<double> used_at(n_nodes, 0.0), arrived(n_nodes, 0.0), last;
  std::vector<int64_t> cand, held, order;
  TieOrderSort<double> sorter;
  for (int64_t b = 0; b < L.n_batches; ++b) {
    cand.clear();
    for (int64_t i = L.ngh_off[b]; i < L.ngh_off[b + 1]; ++i) {
      const int32_t v = L.ngh[i];
      if (cached[v]) { st.reuse += 1; st.dist += (double)b - arrived[v]; }
      else { st.recompute += 1; if (!listed[v]) { listed[v] = 1; cand.push_back(v); } }
    }
    for (int64_t i = L.ngh_off[b]; i < L.ngh_off[b + 1]; ++i)
      if (cached[L.ngh[i]]) used_at[L.ngh[i]] = (double)b;
    std::sort(cand.begin(), cand.end());
    for (int64_t v : cand) listed[v] = 0;
    ascending_set(cached, held);
    const int64_t n_held = (int64_t)held.size(), n_cand = (int64_t)cand.size();
    const int64_t room = budget - n_held;
    const int64_t evict = room >= n_cand ? 0 : std::min(n_cand - room, n_held);
    const int64_t take = (evict + room >= n_cand) ? n_cand : budget;
    if (evict != 0) {
      last.resize(n_held);
      for (int64_t i = 0; i < n_held; ++i) last[i] = used_at[held[i]];
      sorter.run(last.data(), n_held, order);
      for (int64_t i = 0; i < evict; ++i) cached[held[order[i]]] = 0;
    }
    rng.shuffle(cand);
    for (int64_t i = 0; i < take; ++i) {
      const int64_t v = cand[i];
      cached[v] = 1;
      used_at[v] = arrived[v] = (double)b;
    }
    ascending_set(cached, held);
    int32_t *dst = out.begin_batch(b);
    if (!out.room((int64_t)held.size())) return;
    for (size_t i = 0; i < held.size(); ++i) dst[i] = (int32_t)held[i];
    out.used += (int64_t)held.size();
  }
  out.off[L.n_batches] = out.used;
}

// utils/cache.py:175-333: a FIFO half and an LRU half of budget/2 entries each
static void solve_2q(const BatchLists &L, int64_t n_nodes, int64_t budget, uint32_t seed, PlanOut &out,
                     Stats &st) {
  Twister rng(seed);
  const int64_t half = budget / 2;
  std::vector<uint8_t> in_fifo(n_nodes, 0), in_lru(n_nodes, 0), mark(n_nodes, 0);
  std::vector<double> lru_used(n_nodes, 0.0), lru_arr(n_nodes, 0.0), fifo_arr(n_nodes, 0.0), last;
  std::vector<int64_t> promote, fresh, touched, ids, order;
  TieOrderSort<double> sorter;
  int64_t n_fifo = 0, n_lru = 0;
  auto uniq_sorted = [&](std::vector<int64_t> &x) {
    std::sort(x.begin(), x.end());
    x.erase(std::unique(x.begin(), x.end()), x.end());
  };
  for (int64_t b = 0; b < L.n_batches; ++b) {
    const double now = (double)b;
    promote.clear(); fresh.clear(); touched.clear();
    for (int64_t i = L.ngh_off[b]; i < L.ngh_off[b + 1]; ++i) {
      const int32_t v = L.ngh[i];
      if (in_fifo[v]) { st.reuse += 1; st.dist += now - fifo_arr[v]; promote.push_back(v); }
      else if (in_lru[v]) { st.reuse += 1; st.dist += now - lru_arr[v]; touched.push_back(v); }
      else { st.recompute += 1; fresh.push_back(v); }
    }
    uniq_sorted(promote); uniq_sorted(fresh); uniq_sorted(touched);
    const int64_t n_promote = (int64_t)promote.size(), n_fresh = (int64_t)fresh.size();
    // FIFO half
    const int64_t fifo_kept = n_fifo - n_promote, fifo_room = half - fifo_kept;
    for (int64_t v : promote) in_fifo[v] = 0;
    if (n_fresh <= fifo_room) {
      for (int64_t v : fresh) { in_fifo[v] = 1; fifo_arr[v] = now; }
      n_fifo = fifo_kept + n_fresh;
    } else if (n_fresh >= half) {
      ids = fresh;
      rng.shuffle(ids);
      std::fill(in_fifo.begin(), in_fifo.end(), 0);
      std::fill(fifo_arr.begin(), fifo_arr.end(), 0.0);
      for (int64_t i = 0; i < half; ++i) { in_fifo[ids[i]] = 1; fifo_arr[ids[i]] = now; }
      n_fifo = half;
    } else {
      ascending_set(in_fifo, ids);
      rng.shuffle(ids);
      for (int64_t i = 0; i < n_fresh - fifo_room; ++i) in_fifo[ids[i]] = 0;
      for (int64_t v : fresh) { in_fifo[v] = 1; fifo_arr[v] = now; }
      n_fifo = half;
    }
    // LRU half
    for (int64_t v : touched) lru_used[v] = now;
    const int64_t lru_room = half - n_lru, lru_evictable = n_lru - (int64_t)touched.size();
    auto admit = [&](int64_t v) { in_lru[v] = 1; lru_used[v] = now; lru_arr[v] = fifo_arr[v]; };
    if (n_promote <= lru_room) {
      for (int64_t v : promote) admit(v);
      n_lru += n_promote;
    } else if (n_promote <= lru_room + lru_evictable) {
      ascending_set(in_lru, ids);
      last.resize(ids.size());
      for (size_t i = 0; i < ids.size(); ++i) last[i] = lru_used[ids[i]];
      sorter.run(last.data(), (int64_t)ids.size(), order);
      for (int64_t i = 0; i < n_promote - lru_room; ++i) in_lru[ids[order[i]]] = 0;
      for (int64_t v : promote) admit(v);
      n_lru = half;
    } else {
      ascending_set(in_lru, ids);
      for (int64_t v : ids) if (lru_used[v] < now) in_lru[v] = 0;
      ids = promote;
      rng.shuffle(ids);
      for (int64_t i = 0; i < half - (int64_t)touched.size(); ++i) admit(ids[i]);
      n_lru = half;
    }
    // plan = FIFO ids ascending, then LRU ids ascending
    int32_t *dst = out.begin_batch(b);
    ascending_set(in_fifo, ids);
    n_fifo = (int64_t)ids.size();
    if (!out.room(n_fifo)) return;
    for (size_t i = 0; i < ids.size(); ++i) dst[i] = (int32_t)ids[i];
    out.used += n_fifo;
    ascending_set(in_lru, ids);
    n_lru = (int64_t)ids.size();
    if (!out.room(n_lru)) return;
    for (size_t i = 0; i < ids.size(); ++i) dst[n_fifo + i] = (int32_t)ids[i];
    out.used += n_lru;
  }
  out.off[L.n_batches] = out.used;
  (void)mark;
}

}  // namespace plan
}  // namespace orca

using namespace orca;

extern "C" int orca_plan_host(int32_t strategy, const int64_t *h_src, const int64_t *h_dst, int64_t n_edges,
                              int32_t bs, int32_t k, const int32_t *h_nbr, int64_t n_nodes, int32_t budget,
                              uint32_t seed, int32_t *h_plan_flat, int64_t plan_cap, int64_t *h_plan_off,
                              double *h_stats) {
  ORCA_CHECK_ARG(h_src && h_dst && h_nbr && h_plan_flat && h_plan_off && h_stats);
  ORCA_CHECK_ARG(n_edges >= 0 && bs > 0 && k >= 1 && k <= ORCA_MAX_K && n_nodes > 0 && budget > 0);
  ORCA_CHECK_ARG(strategy >= 0 && strategy <= 2);
  for (int64_t i = 0; i < n_edges; ++i)
    if (h_src[i] < 0 || h_src[i] >= n_nodes || h_dst[i] < 0 || h_dst[i] >= n_nodes)
      return set_error(ORCA_E_BOUNDS, "orca_plan_host: edge %lld has an endpoint outside [0,%lld)", (long long)i,
                       (long long)n_nodes);
  plan::BatchLists L;
  plan::build_lists(h_src, h_dst, n_edges, bs, k, h_nbr, n_nodes, strategy == 0, L);
  plan::PlanOut out{h_plan_flat, h_plan_off, plan_cap};
  plan::Stats st;
  if (strategy == 0) plan::solve_mrd(L, n_nodes, budget, out, st);
  else if (strategy == 1) plan::solve_lru(L, n_nodes, budget, seed, out, st);
  else plan::solve_2q(L, n_nodes, budget, seed, out, st);
  if (out.overflow) return set_error(ORCA_E_CAPACITY, "orca_plan_host: plan buffer of %lld entries is too small",
                                     (long long)plan_cap);
  h_stats[0] = st.reuse;
  h_stats[1] = st.recompute;
  h_stats[2] = st.dist;
  return ORCA_OK;
}
