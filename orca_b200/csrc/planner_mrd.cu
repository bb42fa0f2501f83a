// MRD cache planning on the device (utils/cache.py:19-89 read_batches + :92-166 MRD_numba).
//
// Input: the query list of all batches (batch b = its sources, then its destinations) and the neighbour
// table the sampling kernel produced for it.  Two persistent kernels walk the batches (each exists for one
// CTA and for one thread-block cluster; the cluster form is the one normally launched):
//
//   next_use_kernel   backwards.  Keeps, per node, the code of its nearest LATER use
//                     (2 * batch + 1 if that use is as an out-of-batch neighbour, 2 * batch if as a
//                     target, 2 * n_batches if none) and stores, beside every entry of the query list
//                     and of the neighbour table, the code its node has at that batch.  This replaces
//                     the reference's per-node occurrence lists and their cursors: the key of a
//                     candidate at batch b is (code & 1) ? (code >> 1) - b : 1e8 + 1.
//   mrd_kernel        forwards.  Per batch: targets and uncached out-of-batch neighbours are marked in
//                     a bitmap of fresh nodes (and counted for the reuse statistics), the candidates
//                     cached | fresh are listed in ascending order from the bitmaps, their keys are read
//                     from the codes, and the first `budget` positions of numba's argsort become the
//                     new cache.
//
// The first `budget` places of numba's argsort, with its order among equal keys, come from the steps described
// in tie_order.cuh: block-wide in the one-CTA kernel, spread over the cluster in the cluster kernel.
#include "common.cuh"
#include "tie_order.cuh"

namespace orca {
namespace mrd {

constexpr int T = 1024;
constexpr int NW = T / 32;
constexpr int32_t FAR_KEY = 100000001;  // MAX_DISTANCE + 1 of utils/cache.py:95,147-149

struct Work {
  int32_t *nx_query;  // [2E]     code of the next use, per query-list entry
  int32_t *nx_table;  // [2E*k]   the same per neighbour-table entry (out-of-batch entries only)
  int32_t *code;      // [n_nodes] backward pass: nearest later use; forward pass: next use
  int32_t *stamp;     // [n_nodes] last batch in which the node was a target
  int32_t *since;     // [n_nodes] batch in which the cached embedding was computed (time_flag)
  uint32_t *cached;   // [words]
  uint32_t *fresh;    // [words]  uncached out-of-batch neighbours and targets of the batch (new_computed)
  int32_t *cand;      // [cap] candidate ids, ascending
  uint64_t *e;        // [cap] key << 32 | index into cand, in sort order
  int2 *seg;          // [cap] range (lo, hi) a position belongs to
  int2 *pre;          // [cap] prefix counts (left list, right list) before the position
  int32_t *lpos, *rpos;        // [cap] positions of a range's left / right list, stored from its lo
  int32_t *pivot;     // [cap] per range, at index lo
  int32_t *swaps;     // [2][cap] per range, at index lo: pair swaps of its step; the halves alternate by
                      // depth, because a step's count is still read while the next pivots are parked
};

__host__ __device__ inline int64_t words_of(int64_t n_nodes) { return (n_nodes + 31) / 32; }
__host__ __device__ inline int64_t cand_cap(int32_t bs, int32_t k, int32_t budget) {
  return (int64_t)budget + 2ll * bs * (k + 1);
}

using tie::key_of;
using tie::live;

// ------------------------------------------------------------------------------ backward pass
__global__ void __launch_bounds__(T) next_use_kernel(const int32_t *nodes, const int32_t *nbr, int64_t n_edges,
                                                     int32_t bs, int32_t k, int64_t n_nodes, Work w) {
  const int tid = threadIdx.x;
  const int64_t nb = (n_edges + bs - 1) / bs;
  for (int64_t v = tid; v < n_nodes; v += T) {
    w.code[v] = (int32_t)(2 * nb);
    w.stamp[v] = -1;
  }
  __syncthreads();
  for (int64_t b = nb - 1; b >= 0; --b) {
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s;
    const int32_t *tab = nbr + 2 * s * k;
    int32_t *nq = w.nx_query + 2 * s;
    int32_t *nt = w.nx_table + 2 * s * k;
    for (int i = tid; i < m2; i += T) {
      const int32_t v = q[i];
      nq[i] = w.code[v];
      w.stamp[v] = (int32_t)b;
    }
    __syncthreads();
    for (int i = tid; i < m2 * k; i += T) {
      const int32_t v = tab[i];
      if (v != 0 && w.stamp[v] != (int32_t)b) nt[i] = w.code[v];
    }
    __syncthreads();
    for (int i = tid; i < m2; i += T) w.code[q[i]] = (int32_t)(2 * b);
    for (int i = tid; i < m2 * k; i += T) {
      const int32_t v = tab[i];
      if (v != 0 && w.stamp[v] != (int32_t)b) w.code[v] = (int32_t)(2 * b + 1);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------ forward pass
__global__ void __launch_bounds__(T) mrd_kernel(const int32_t *nodes, const int32_t *nbr, int64_t n_edges, int32_t bs,
                                                int32_t k, int64_t n_nodes, int32_t budget, Work w,
                                                int32_t *plan, int64_t plan_cap, int64_t *plan_off,
                                                int64_t *stats, int32_t *status) {
  __shared__ int s_l[NW], s_r[NW];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int64_t nb = (n_edges + bs - 1) / bs;
  const int64_t words = words_of(n_nodes);
  for (int64_t v = tid; v < n_nodes; v += T) {
    w.stamp[v] = -1;
    w.since[v] = 0;
  }
  for (int64_t i = tid; i < words; i += T) {
    w.cached[i] = 0;
    w.fresh[i] = 0;
  }
  __syncthreads();
  long long reuse = 0, recompute = 0, dist = 0;
  int64_t used = 0;
  const int wchunk = (int)(((words + NW - 1) / NW + 31) & ~31ll);  // bitmap words per warp
  const int64_t cap = cand_cap(bs, k, budget);
  for (int64_t b = 0; b < nb; ++b) {
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s;
    const int32_t *tab = nbr + 2 * s * k;
    const int32_t *nq = w.nx_query + 2 * s;
    const int32_t *nt = w.nx_table + 2 * s * k;
    // targets
    for (int i = tid; i < m2; i += T) {
      const int32_t v = q[i];
      w.stamp[v] = (int32_t)b;
      w.code[v] = nq[i];
      atomicOr(&w.fresh[v >> 5], 1u << (v & 31));
    }
    __syncthreads();
    // out-of-batch neighbour occurrences: reuse statistics, uncached ones become fresh
    for (int i = tid; i < m2 * k; i += T) {
      const int32_t v = tab[i];
      if (v == 0 || w.stamp[v] == (int32_t)b) continue;
      w.code[v] = nt[i];
      if ((__ldcg(&w.cached[v >> 5]) >> (v & 31)) & 1u) {
        ++reuse;
        dist += b - w.since[v];
      } else {
        ++recompute;
        atomicOr(&w.fresh[v >> 5], 1u << (v & 31));
      }
    }
    __syncthreads();
    // candidates = cached | fresh in ascending order, with their keys
    {
      int cnt = 0;
      for (int j = lane; j < wchunk; j += 32) {
        const int64_t wi = (int64_t)warp * wchunk + j;
        if (wi < words) cnt += __popc(__ldcg(&w.cached[wi]) | __ldcg(&w.fresh[wi]));
      }
      for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
      if (lane == 0) s_l[warp] = cnt;
    }
    __syncthreads();
    int n = 0, base = 0;
    for (int i = 0; i < NW; ++i) {
      const int c = s_l[i];
      if (i < warp) base += c;
      n += c;
    }
    for (int j = 0; j < wchunk; j += 32) {
      const int64_t wi = (int64_t)warp * wchunk + j + lane;
      uint32_t bits = 0;
      if (wi < words) {
        bits = __ldcg(&w.cached[wi]) | __ldcg(&w.fresh[wi]);
        w.cached[wi] = 0;
      }
      const int c = __popc(bits);
      int incl = c;
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      int pos = base + incl - c;
      base += __shfl_sync(0xffffffffu, incl, 31);
      while (bits) {
        const int bit = __ffs(bits) - 1;
        bits &= bits - 1;
        const int32_t v = (int32_t)(wi * 32 + bit);
        const int32_t code = w.code[v];
        const int32_t key = (code & 1) ? (code >> 1) - (int32_t)b : FAR_KEY;
        w.cand[pos] = v;
        w.e[pos] = ((uint64_t)(uint32_t)key << 32) | (uint32_t)pos;
        ++pos;
      }
    }
    const int keep = min(n, budget);
    if (used + keep > plan_cap) {  // uniform over the block
      if (tid == 0) report(status, ORCA_E_CAPACITY, (int)b);
      break;
    }
    // ---- the first `keep` positions of numba's argsort
    const tie::Buf sb{w.e, w.seg, w.pre, w.lpos, w.rpos, w.pivot, w.swaps, cap};
    if (!tie::sort_first(sb, n, keep, s_l, s_r)) {   // uniform over the block
      if (tid == 0) report(status, ORCA_E_TIMEOUT, (int)b);
      break;
    }
    // ranges shorter than 16: stable order by key; the first `keep` places are the new cache
    if (tid == 0) plan_off[b] = used;
    for (int pos = tid; pos < n; pos += T) {
      const int place = tie::place_of(sb, pos, keep);
      if (place < 0) continue;
      const int32_t v = w.cand[(uint32_t)w.e[pos]];
      plan[used + place] = v;
      atomicOr(&w.cached[v >> 5], 1u << (v & 31));
      if ((__ldcg(&w.fresh[v >> 5]) >> (v & 31)) & 1u) w.since[v] = (int32_t)b;
    }
    used += keep;
    __syncthreads();
    for (int64_t i = tid; i < words; i += T) w.fresh[i] = 0;
    __syncthreads();
  }
  // totals
  for (int o = 16; o > 0; o >>= 1) {
    reuse += __shfl_xor_sync(0xffffffffu, reuse, o);
    recompute += __shfl_xor_sync(0xffffffffu, recompute, o);
    dist += __shfl_xor_sync(0xffffffffu, dist, o);
  }
  if (lane == 0) {
    atomicAdd((unsigned long long *)&stats[0], (unsigned long long)reuse);
    atomicAdd((unsigned long long *)&stats[1], (unsigned long long)recompute);
    atomicAdd((unsigned long long *)&stats[2], (unsigned long long)dist);
  }
  if (tid == 0) plan_off[nb] = used;
}

// ------------------------------------------------------------------------------ cluster form
// The same two sweeps on a thread-block cluster: C CTAs of 1024 threads share every phase, positions and
// table entries are dealt out over all of them, and a phase boundary is a cluster barrier (release /
// acquire).  Data another CTA wrote in an earlier phase is read from L2 (ld.global.cg); the range a
// position belongs to lives in the registers of the thread that owns the position.  For candidate lists of
// at most MAX_ITEMS * 1024 * C entries.
constexpr int MAX_ITEMS = 8;

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint64_t ldcg64(const uint64_t *p) { return __ldcg((const unsigned long long *)p); }

struct ClusterWork {
  Work w;
  int2 *tot;        // [warps of the cluster] totals of a counting pass
  int32_t *place;   // [cap] per range, at index lo: where its pivot ends up
  int32_t *live;    // [1] id of the last partition depth that left a live range
  uint32_t *fresh2; // [2][words] fresh bitmaps of even / odd batches
};

__global__ void __launch_bounds__(T, 1) next_use_cluster_kernel(const int32_t *nodes, const int32_t *nbr,
                                                                int64_t n_edges, int32_t bs, int32_t k,
                                                                int64_t n_nodes, Work w) {
  const int GT = T * (int)cluster_size();
  const int gt = (int)cluster_rank() * T + threadIdx.x;
  const int64_t nb = (n_edges + bs - 1) / bs;
  for (int64_t v = gt; v < n_nodes; v += GT) {
    w.code[v] = (int32_t)(2 * nb);
    w.stamp[v] = -1;
  }
  cluster_sync();
  for (int64_t b = nb - 1; b >= 0; --b) {
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s;
    const int32_t *tab = nbr + 2 * s * k;
    int32_t *nq = w.nx_query + 2 * s;
    int32_t *nt = w.nx_table + 2 * s * k;
    for (int i = gt; i < m2; i += GT) {
      const int32_t v = q[i];
      nq[i] = __ldcg(&w.code[v]);
      w.stamp[v] = (int32_t)b;
    }
    cluster_sync();
    for (int i = gt; i < m2 * k; i += GT) {
      const int32_t v = tab[i];
      if (v != 0 && __ldcg(&w.stamp[v]) != (int32_t)b) nt[i] = __ldcg(&w.code[v]);
    }
    cluster_sync();
    for (int i = gt; i < m2; i += GT) w.code[q[i]] = (int32_t)(2 * b);
    for (int i = gt; i < m2 * k; i += GT) {
      const int32_t v = tab[i];
      if (v != 0 && __ldcg(&w.stamp[v]) != (int32_t)b) w.code[v] = (int32_t)(2 * b + 1);
    }
    cluster_sync();
  }
}

// median of three with the pivot parked at hi, for data other CTAs may have written
__device__ __forceinline__ void park_pivot_cg(const Work &w, int lo, int hi) {
  const int mid = (lo + hi) >> 1;
  uint64_t a = ldcg64(&w.e[lo]), c = ldcg64(&w.e[mid]), d = ldcg64(&w.e[hi]);
  uint64_t t;
  if (key_of(c) < key_of(a)) { t = a; a = c; c = t; }
  if (key_of(d) < key_of(c)) { t = d; d = c; c = t; }
  if (key_of(c) < key_of(a)) { t = a; a = c; c = t; }
  w.e[lo] = a;
  w.e[mid] = d;
  w.e[hi] = c;
  w.pivot[lo] = key_of(c);
}

__global__ void __launch_bounds__(T, 1) mrd_cluster_kernel(const int32_t *nodes, const int32_t *nbr, int64_t n_edges,
                                                           int32_t bs, int32_t k, int64_t n_nodes, int32_t budget,
                                                           ClusterWork cw, int32_t *plan, int64_t plan_cap,
                                                           int64_t *plan_off, int64_t *stats, int32_t *status) {
  const Work &w = cw.w;
  const int GT = T * (int)cluster_size();
  const int gt = (int)cluster_rank() * T + threadIdx.x;
  const int lane = threadIdx.x & 31, gwarp = gt >> 5, n_warps = GT >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  const int64_t nb = (n_edges + bs - 1) / bs;
  const int64_t words = words_of(n_nodes);
  for (int64_t v = gt; v < n_nodes; v += GT) {
    w.stamp[v] = -1;
    w.since[v] = 0;
  }
  for (int64_t i = gt; i < words; i += GT) {
    w.cached[i] = 0;
    cw.fresh2[i] = 0;
    cw.fresh2[words + i] = 0;
  }
  if (gt == 0) *cw.live = 0;
  cluster_sync();
  long long reuse = 0, recompute = 0, dist = 0;
  int64_t used = 0;
  int epoch = 0;
  const int wchunk = (int)(((words + n_warps - 1) / n_warps + 31) & ~31ll);  // bitmap words per warp
  // sums of the per-warp totals of a counting pass: before this warp, and over all warps
  auto warp_prefix = [&](int &before_x, int &before_y, int &all_x) {
    int bx = 0, by = 0, ax = 0;
    for (int j = lane; j < n_warps; j += 32) {
      const int2 c = __ldcg(&cw.tot[j]);
      ax += c.x;
      if (j < gwarp) {
        bx += c.x;
        by += c.y;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      bx += __shfl_xor_sync(0xffffffffu, bx, o);
      by += __shfl_xor_sync(0xffffffffu, by, o);
      ax += __shfl_xor_sync(0xffffffffu, ax, o);
    }
    before_x = bx;
    before_y = by;
    all_x = ax;
  };
  for (int64_t b = 0; b < nb; ++b) {
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s;
    const int32_t *tab = nbr + 2 * s * k;
    const int32_t *nq = w.nx_query + 2 * s;
    const int32_t *nt = w.nx_table + 2 * s * k;
    uint32_t *fresh = cw.fresh2 + (b & 1) * words;
    uint32_t *stale = cw.fresh2 + ((b + 1) & 1) * words;   // the previous batch's: cleared on the way
    for (int i = gt; i < m2; i += GT) {
      const int32_t v = q[i];
      w.stamp[v] = (int32_t)b;
      w.code[v] = nq[i];
      atomicOr(&fresh[v >> 5], 1u << (v & 31));
    }
    cluster_sync();
    // (four entries at a time: the loads of one step are issued together, not entry after entry)
    for (int i0 = gt; i0 < m2 * k; i0 += 4 * GT) {
      int32_t v[4], st[4], sn[4], cd[4];
      uint32_t cw_[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * GT;
        v[u] = i < m2 * k ? tab[i] : 0;
        cd[u] = i < m2 * k ? nt[i] : 0;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        st[u] = v[u] != 0 ? __ldcg(&w.stamp[v[u]]) : (int32_t)b;
        cw_[u] = v[u] != 0 ? __ldcg(&w.cached[v[u] >> 5]) : 0u;
        sn[u] = v[u] != 0 ? __ldcg(&w.since[v[u]]) : 0;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v[u] == 0 || st[u] == (int32_t)b) continue;
        w.code[v[u]] = cd[u];
        if ((cw_[u] >> (v[u] & 31)) & 1u) {
          ++reuse;
          dist += b - sn[u];
        } else {
          ++recompute;
          atomicOr(&fresh[v[u] >> 5], 1u << (v[u] & 31));
        }
      }
    }
    cluster_sync();
    {
      int cnt = 0;
      for (int j = lane; j < wchunk; j += 32) {
        const int64_t wi = (int64_t)gwarp * wchunk + j;
        if (wi < words) cnt += __popc(__ldcg(&w.cached[wi]) | __ldcg(&fresh[wi]));
      }
      for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
      if (lane == 0) cw.tot[gwarp] = make_int2(cnt, 0);
    }
    cluster_sync();
    int n, base, unused;
    warp_prefix(base, unused, n);
    for (int j = 0; j < wchunk; j += 32) {
      const int64_t wi = (int64_t)gwarp * wchunk + j + lane;
      uint32_t bits = 0;
      if (wi < words) {
        bits = __ldcg(&w.cached[wi]) | __ldcg(&fresh[wi]);
        w.cached[wi] = 0;
        stale[wi] = 0;
      }
      const int c = __popc(bits);
      int incl = c;
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      int pos = base + incl - c;
      base += __shfl_sync(0xffffffffu, incl, 31);
      while (bits) {
        const int bit = __ffs(bits) - 1;
        bits &= bits - 1;
        w.cand[pos++] = (int32_t)(wi * 32 + bit);   // (keys follow below, one thread per position)
      }
    }
    const int keep = min(n, budget);
    if (used + keep > plan_cap) {  // uniform over the cluster
      if (gt == 0) report(status, ORCA_E_CAPACITY, (int)b);
      break;
    }
    // ---- the first `keep` positions of numba's argsort.  Thread owns positions gwarp*32*items + i*32 + lane.
    const int items = (n + GT - 1) / GT;
    const int first_pos = gwarp * 32 * items + lane;
    int lo[MAX_ITEMS], hi[MAX_ITEMS];
#pragma unroll
    for (int i = 0; i < MAX_ITEMS; ++i) {
      lo[i] = 0;
      hi[i] = (i < items && first_pos + 32 * i < n) ? n - 1 : -1;   // hi < 0: no such position
    }
    bool any = live(0, n - 1, keep);
    cluster_sync();
    // keys: a word of the bitmaps can hold 32 candidates, so its thread does not chase their codes one after
    // the other; the owner of each position reads its candidate's code
#pragma unroll
    for (int i = 0; i < MAX_ITEMS; ++i) {
      if (i < items && hi[i] >= 0) {
        const int pos = first_pos + 32 * i;
        const int32_t code = __ldcg(&w.code[__ldcg(&w.cand[pos])]);
        const int32_t key = (code & 1) ? (code >> 1) - (int32_t)b : FAR_KEY;
        w.e[pos] = ((uint64_t)(uint32_t)key << 32) | (uint32_t)pos;
      }
    }
    cluster_sync();
    if (any && gt == 0) park_pivot_cg(w, 0, n - 1);
    cluster_sync();
    int depth = 0;
    while (any) {
      ++epoch;
      if (++depth > n) break;   // every step shortens the longest live range: more steps than entries is a fault
      uint32_t fl = 0, fr = 0;
      int cl = 0, cr = 0;
#pragma unroll
      for (int i = 0; i < MAX_ITEMS; ++i) {
        if (i < items) {
          const int pos = first_pos + 32 * i;
          bool is_l = false, is_r = false;
          if (hi[i] >= 0 && live(lo[i], hi[i], keep) && pos < hi[i]) {
            const int32_t kv = key_of(ldcg64(&w.e[pos])), pv = __ldcg(&w.pivot[lo[i]]);
            is_l = kv >= pv;
            is_r = kv <= pv;
          }
          cl += __popc(__ballot_sync(0xffffffffu, is_l));
          cr += __popc(__ballot_sync(0xffffffffu, is_r));
          fl |= (is_l ? 1u : 0u) << i;
          fr |= (is_r ? 1u : 0u) << i;
        }
      }
      if (lane == 0) cw.tot[gwarp] = make_int2(cl, cr);
      cluster_sync();
      int bl, br;
      warp_prefix(bl, br, unused);
#pragma unroll
      for (int i = 0; i < MAX_ITEMS; ++i) {
        if (i < items) {
          const int pos = first_pos + 32 * i;
          const uint32_t ml = __ballot_sync(0xffffffffu, (fl >> i) & 1u), mr = __ballot_sync(0xffffffffu, (fr >> i) & 1u);
          if (hi[i] >= 0 && live(lo[i], hi[i], keep))
            w.pre[pos] = make_int2(bl + __popc(ml & lt_mask), br + __popc(mr & lt_mask));
          bl += __popc(ml);
          br += __popc(mr);
        }
      }
      cluster_sync();
#pragma unroll
      for (int i = 0; i < MAX_ITEMS; ++i) {
        if (i < items && (((fl | fr) >> i) & 1u)) {
          const int pos = first_pos + 32 * i;
          const int2 me = __ldcg(&w.pre[pos]), a = __ldcg(&w.pre[lo[i]]), z = __ldcg(&w.pre[hi[i]]);
          if ((fl >> i) & 1u) w.lpos[lo[i] + me.x - a.x] = pos;
          if ((fr >> i) & 1u) w.rpos[lo[i] + z.y - me.y - 1] = pos;
        }
      }
      cluster_sync();
#pragma unroll
      for (int i = 0; i < MAX_ITEMS; ++i) {
        if (i < items && hi[i] >= 0 && live(lo[i], hi[i], keep)) {
          const int pos = first_pos + 32 * i;
          if (pos >= hi[i]) continue;
          const int2 a = __ldcg(&w.pre[lo[i]]), z = __ldcg(&w.pre[hi[i]]);
          const int n_left = z.x - a.x, pairs = min(n_left, z.y - a.y);
          const int m = pos - lo[i];
          if (m < pairs) {
            const int pl = __ldcg(&w.lpos[pos]), pr = __ldcg(&w.rpos[pos]);
            const bool ok = pl < pr;
            const int next_l = m + 1 < n_left ? __ldcg(&w.lpos[pos + 1]) : hi[i];
            const bool next_ok = m + 1 < pairs && next_l < __ldcg(&w.rpos[pos + 1]);
            if (ok) {
              const uint64_t x = ldcg64(&w.e[pl]), y = ldcg64(&w.e[pr]);
              w.e[pl] = y;
              w.e[pr] = x;
              if (!next_ok) cw.place[lo[i]] = min(next_l, pr);
            } else if (m == 0) {
              cw.place[lo[i]] = pl;
            }
          } else if (m == 0) {
            cw.place[lo[i]] = n_left > 0 ? __ldcg(&w.lpos[pos]) : hi[i];
          }
        }
      }
      cluster_sync();
      bool more = false;
#pragma unroll
      for (int i = 0; i < MAX_ITEMS; ++i) {
        if (i < items && hi[i] >= 0 && live(lo[i], hi[i], keep)) {
          const int pos = first_pos + 32 * i;
          const int p = __ldcg(&cw.place[lo[i]]);
          if (pos == p + 1) {
            const uint64_t x = ldcg64(&w.e[p]), y = ldcg64(&w.e[hi[i]]);
            w.e[p] = y;
            w.e[hi[i]] = x;
          }
          if (pos < p) hi[i] = p - 1;
          else if (pos > p) lo[i] = p + 1;
          else lo[i] = hi[i] = p;
          if (live(lo[i], hi[i], keep)) {
            more = true;
            if (pos == lo[i]) park_pivot_cg(w, lo[i], hi[i]);
          }
        }
      }
      if (more) *cw.live = epoch;
      cluster_sync();
      any = __ldcg(cw.live) == epoch;
    }
    if (depth > n) {   // uniform over the cluster
      if (gt == 0) report(status, ORCA_E_TIMEOUT, (int)b);
      break;
    }
    // ranges shorter than 16: stable order by key; the first `keep` places are the new cache
    if (gt == 0) plan_off[b] = used;
#pragma unroll
    for (int i = 0; i < MAX_ITEMS; ++i) {
      if (i < items && hi[i] >= 0 && lo[i] < keep) {
        const int pos = first_pos + 32 * i;
        const uint64_t me = ldcg64(&w.e[pos]);
        const int32_t kv = key_of(me);
        int place = lo[i];
        for (int qpos = lo[i]; qpos <= hi[i]; ++qpos) {
          const int32_t ko = key_of(ldcg64(&w.e[qpos]));
          place += (ko < kv || (ko == kv && qpos < pos)) ? 1 : 0;
        }
        if (place < keep) {
          const int32_t v = __ldcg(&w.cand[(uint32_t)me]);
          plan[used + place] = v;
          atomicOr(&w.cached[v >> 5], 1u << (v & 31));
          if ((__ldcg(&fresh[v >> 5]) >> (v & 31)) & 1u) w.since[v] = (int32_t)b;
        }
      }
    }
    used += keep;
    // (no barrier here: the next batch's first phase writes stamps, codes and the other fresh bitmap only)
  }
  for (int o = 16; o > 0; o >>= 1) {
    reuse += __shfl_xor_sync(0xffffffffu, reuse, o);
    recompute += __shfl_xor_sync(0xffffffffu, recompute, o);
    dist += __shfl_xor_sync(0xffffffffu, dist, o);
  }
  if (lane == 0) {
    atomicAdd((unsigned long long *)&stats[0], (unsigned long long)reuse);
    atomicAdd((unsigned long long *)&stats[1], (unsigned long long)recompute);
    atomicAdd((unsigned long long *)&stats[2], (unsigned long long)dist);
  }
  if (gt == 0) plan_off[nb] = used;
}

struct Layout {
  int64_t off[20];
  int64_t total;
};

static Layout layout(int64_t n_edges, int32_t bs, int32_t k, int64_t n_nodes, int32_t budget) {
  Layout L;
  const int64_t cap = cand_cap(bs, k, budget), words = words_of(n_nodes);
  const int64_t sizes[20] = {2 * n_edges * 4,   2 * n_edges * k * 4, n_nodes * 4, n_nodes * 4, n_nodes * 4, words * 4,
                             2 * words * 4,     cap * 4,             cap * 8,     cap * 8,     cap * 8,     cap * 4,
                             cap * 4,           cap * 4,             2 * cap * 4, 1024 * 8,    cap * 4,     256,
                             0,                 0};
  int64_t at = 0;
  for (int i = 0; i < 20; ++i) {
    L.off[i] = at;
    at += (sizes[i] + 255) & ~255ll;
  }
  L.total = at;
  return L;
}

}  // namespace mrd
}  // namespace orca

using namespace orca;

extern "C" int64_t orca_plan_mrd_workspace_bytes(int64_t n_edges, int32_t bs, int32_t k, int64_t n_nodes,
                                                 int32_t budget) {
  if (n_edges < 0 || bs <= 0 || k < 1 || n_nodes <= 0 || budget <= 0) return -1;
  return mrd::layout(n_edges, bs, k, n_nodes, budget).total;
}

extern "C" int orca_plan_mrd(const int32_t *d_nodes, int64_t n_edges, int32_t bs, int32_t k, const int32_t *d_nbr,
                             int64_t n_nodes, int32_t budget, int32_t *d_plan_flat, int64_t plan_cap,
                             int64_t *d_plan_off, int64_t *d_stats, int32_t *d_status, void *d_workspace,
                             int64_t workspace_bytes, void *stream) {
  ORCA_CHECK_ARG(d_nodes && d_nbr && d_plan_flat && d_plan_off && d_stats && d_status && d_workspace);
  ORCA_CHECK_ARG(n_edges >= 0 && bs > 0 && k >= 1 && k <= ORCA_MAX_K && n_nodes > 0 && budget > 0);
  ORCA_CHECK_ARG(n_nodes < (1ll << 31) && (n_edges + bs - 1) / bs < (1ll << 29));
  ORCA_CHECK_ARG(mrd::cand_cap(bs, k, budget) < (1ll << 31));
  const mrd::Layout L = mrd::layout(n_edges, bs, k, n_nodes, budget);
  if (workspace_bytes < L.total)
    return set_error(ORCA_E_CAPACITY, "orca_plan_mrd: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                     (long long)L.total);
  ORCA_CHECK_ARG(((uintptr_t)d_workspace & 255) == 0);
  char *base = (char *)d_workspace;
  mrd::Work w;
  w.nx_query = (int32_t *)(base + L.off[0]);
  w.nx_table = (int32_t *)(base + L.off[1]);
  w.code = (int32_t *)(base + L.off[2]);
  w.stamp = (int32_t *)(base + L.off[3]);
  w.since = (int32_t *)(base + L.off[4]);
  w.cached = (uint32_t *)(base + L.off[5]);
  w.fresh = (uint32_t *)(base + L.off[6]);
  w.cand = (int32_t *)(base + L.off[7]);
  w.e = (uint64_t *)(base + L.off[8]);
  w.seg = (int2 *)(base + L.off[9]);
  w.pre = (int2 *)(base + L.off[10]);
  w.lpos = (int32_t *)(base + L.off[11]);
  w.rpos = (int32_t *)(base + L.off[12]);
  w.pivot = (int32_t *)(base + L.off[13]);
  w.swaps = (int32_t *)(base + L.off[14]);
  cudaStream_t s = (cudaStream_t)stream;
  ORCA_CUDA(cudaMemsetAsync(d_stats, 0, 3 * sizeof(int64_t), s));
  if (n_edges == 0) {
    ORCA_CUDA(cudaMemsetAsync(d_plan_off, 0, sizeof(int64_t), s));
    return ORCA_OK;
  }
  // A cluster of 16 (else 8) CTAs shares every phase when the device can place such a cluster and the
  // candidate list fits its threads' registers (measured at c5: 0.81 s with 16 CTAs, 0.91 s with 8, 2.3 s
  // with one CTA; a phase costs a cluster barrier of ~600 cycles, an L2 round trip of ~300 per dependent
  // load and the release of its stores); one CTA does the same work otherwise.
  const int64_t cap = mrd::cand_cap(bs, k, budget);
  int cluster = 0;
  for (int c : {16, 8}) {
    if (cluster != 0 || cap > (int64_t)mrd::MAX_ITEMS * mrd::T * c) continue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c);
    cfg.blockDim = dim3(mrd::T);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (c > 8) {
      if (cudaFuncSetAttribute(mrd::mrd_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess ||
          cudaFuncSetAttribute(mrd::next_use_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        (void)cudaGetLastError();
        continue;
      }
    }
    int fits = 0;
    if (cudaOccupancyMaxActiveClusters(&fits, mrd::mrd_cluster_kernel, &cfg) != cudaSuccess || fits < 1) {
      (void)cudaGetLastError();
      continue;
    }
    cluster = c;
  }
  if (cluster != 0) {
    mrd::ClusterWork cw;
    cw.w = w;
    cw.fresh2 = w.fresh;
    cw.tot = (int2 *)(base + L.off[15]);
    cw.place = (int32_t *)(base + L.off[16]);
    cw.live = (int32_t *)(base + L.off[17]);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster);
    cfg.blockDim = dim3(mrd::T);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ORCA_CUDA(cudaLaunchKernelEx(&cfg, mrd::next_use_cluster_kernel, d_nodes, d_nbr, n_edges, bs, k, n_nodes, w));
    ORCA_COUNT_LAUNCH();
    ORCA_CUDA(cudaLaunchKernelEx(&cfg, mrd::mrd_cluster_kernel, d_nodes, d_nbr, n_edges, bs, k, n_nodes, budget, cw,
                                 d_plan_flat, plan_cap, d_plan_off, d_stats, d_status));
    ORCA_COUNT_LAUNCH();
    return ORCA_OK;
  }
  mrd::next_use_kernel<<<1, mrd::T, 0, s>>>(d_nodes, d_nbr, n_edges, bs, k, n_nodes, w);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  mrd::mrd_kernel<<<1, mrd::T, 0, s>>>(d_nodes, d_nbr, n_edges, bs, k, n_nodes, budget, w, d_plan_flat, plan_cap,
                                       d_plan_off, d_stats, d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}
