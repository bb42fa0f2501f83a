// LRU and 2Q cache planning on the device (utils/cache.py:338-403 and 175-333, with read_batches :19-89).
//
// Both policies walk the batches in order and evict at random: numba's np.random.choice(..., replace=False)
// is a Fisher-Yates shuffle driven by its private Mersenne Twister, first entries kept.  One draw decides
// the next swap and how many draws a swap consumes depends on the draws themselves (rejection sampling), so
// the shuffle is one serial chain per batch: thread 0 of the block walks it, generator state in shared
// memory.  Everything around it is data parallel over the block: the split of the batch's neighbour table
// into targets / out-of-batch neighbours (stamps), the reuse statistics, sets as bitmaps that list their
// members in ascending order by a popcount scan (np.unique / np.where of the reference), and the LRU
// evictions, which are the first entries of numba's argsort of the last-use times (tie_order.cuh).
// One CTA of 1024 threads per plan.
#include <algorithm>

#include "common.cuh"
#include "tie_order.cuh"

namespace orca {
namespace rnd {

constexpr int T = tie::T;
constexpr int NW = tie::NW;

// numba's generator (MT19937) and its bounded draw: the low bits that cover n - 1, redrawn while >= n
struct Twister {
  static constexpr int N = 624, M = 397;
  uint32_t s[N];
  int pos;
  __device__ void seed(uint32_t x) {
    s[0] = x;
    for (int i = 1; i < N; ++i) s[i] = 1812433253u * (s[i - 1] ^ (s[i - 1] >> 30)) + (uint32_t)i;
    pos = N;
  }
  __device__ void refill() {
    for (int i = 0; i < N; ++i) {
      const uint32_t y = (s[i] & 0x80000000u) | (s[(i + 1) % N] & 0x7fffffffu);
      s[i] = s[(i + M) % N] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
    }
    pos = 0;
  }
  __device__ uint32_t next() {
    if (pos >= N) refill();
    uint32_t y = s[pos++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    return y ^ (y >> 18);
  }
  __device__ int below(int n) {   // n <= 2^31 here
    if (n <= 1) return 0;
    const uint32_t mask = 0xffffffffu >> __clz((unsigned)(n - 1));
    while (true) {
      const uint32_t r = next() & mask;
      if (r < (uint32_t)n) return (int)r;
    }
  }
  // Fisher-Yates from the back, as numba shuffles; the caller keeps the first entries
  __device__ void shuffle(int32_t *x, int n) {
    for (int i = n - 1; i > 0; --i) {
      const int j = below(i + 1);
      const int32_t a = x[i];
      x[i] = x[j];
      x[j] = a;
    }
  }
};

struct Work {
  int32_t *stamp;                 // [n_nodes] last batch in which the node was a target
  int32_t *t0, *t1, *t2;          // [n_nodes] LRU: last use, arrival; 2Q: LRU last use, LRU arrival, FIFO arrival
  uint32_t *bm[5];                // [words] LRU: cached, candidates; 2Q: fifo, lru, promote, fresh, touched
  int32_t *list[4];               // [cap] member lists
  tie::Buf sort;
  int64_t cap;
};

// (bitmap words are changed by atomics, which act in L2: they are read from there, not through L1)
__device__ __forceinline__ bool bit(const uint32_t *bm, int32_t v) { return (__ldcg(&bm[v >> 5]) >> (v & 31)) & 1u; }
__device__ __forceinline__ void set_bit(uint32_t *bm, int32_t v) { atomicOr(&bm[v >> 5], 1u << (v & 31)); }
__device__ __forceinline__ void clear_bit(uint32_t *bm, int32_t v) { atomicAnd(&bm[v >> 5], ~(1u << (v & 31))); }

// Members of a bitmap in ascending order -> out; returns their number (the same in every thread).  All T
// threads call it; `clear` empties the bitmap on the way.  s_cnt: NW ints of shared memory.
__device__ int list_members(uint32_t *bm, int64_t words, int32_t *out, bool clear, int *s_cnt) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wchunk = (int)(((words + NW - 1) / NW + 31) & ~31ll);
  __syncthreads();   // (earlier writes to the bitmap; earlier readers of s_cnt)
  int cnt = 0;
  for (int j = lane; j < wchunk; j += 32) {
    const int64_t wi = (int64_t)warp * wchunk + j;
    if (wi < words) cnt += __popc(__ldcg(&bm[wi]));
  }
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) s_cnt[warp] = cnt;
  __syncthreads();
  int n = 0, base = 0;
  for (int i = 0; i < NW; ++i) {
    const int c = s_cnt[i];
    if (i < warp) base += c;
    n += c;
  }
  for (int j = 0; j < wchunk; j += 32) {
    const int64_t wi = (int64_t)warp * wchunk + j + lane;
    uint32_t bits = 0;
    if (wi < words) {
      bits = __ldcg(&bm[wi]);
      if (clear && bits) bm[wi] = 0;
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
      out[pos++] = (int32_t)(wi * 32 + (__ffs(bits) - 1));
      bits &= bits - 1;
    }
  }
  __syncthreads();
  return n;
}

// the first `count` entries of numba's argsort of key[ids[i]] (i < n): calls f(id) for each of them
template <class F>
__device__ bool for_first_by_key(const Work &w, const int32_t *ids, int n, int count, const int32_t *key, int *s_a,
                                 int *s_b, F f) {
  for (int i = threadIdx.x; i < n; i += T) w.sort.e[i] = ((uint64_t)(uint32_t)key[ids[i]] << 32) | (uint32_t)i;
  __syncthreads();
  if (!tie::sort_first(w.sort, n, count, s_a, s_b)) return false;
  for (int pos = threadIdx.x; pos < n; pos += T)
    if (tie::place_of(w.sort, pos, count) >= 0) f(ids[(uint32_t)w.sort.e[pos]]);
  __syncthreads();
  return true;
}

struct Totals {
  long long reuse = 0, recompute = 0, dist = 0;
};
__device__ void write_totals(const Totals &t, int64_t *stats) {
  long long a = t.reuse, b = t.recompute, c = t.dist;
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
    c += __shfl_xor_sync(0xffffffffu, c, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd((unsigned long long *)&stats[0], (unsigned long long)a);
    atomicAdd((unsigned long long *)&stats[1], (unsigned long long)b);
    atomicAdd((unsigned long long *)&stats[2], (unsigned long long)c);
  }
}

// ------------------------------------------------------------------------------ LRU (utils/cache.py:338-403)
__global__ void __launch_bounds__(T) lru_kernel(const int32_t *nodes, const int32_t *nbr, int64_t n_edges, int32_t bs,
                                                int32_t k, int64_t n_nodes, int32_t budget, uint32_t seed, Work w,
                                                int32_t *plan, int64_t plan_cap, int64_t *plan_off, int64_t *stats,
                                                int32_t *status) {
  __shared__ Twister rng;
  __shared__ int s_a[NW], s_b[NW];
  const int tid = threadIdx.x;
  const int64_t nb = (n_edges + bs - 1) / bs, words = (n_nodes + 31) / 32;
  uint32_t *cached = w.bm[0], *candbm = w.bm[1];
  int32_t *used_at = w.t0, *arrived = w.t1;
  int32_t *cand = w.list[0], *held = w.list[1];
  for (int64_t v = tid; v < n_nodes; v += T) {
    w.stamp[v] = -1;
    used_at[v] = 0;
    arrived[v] = 0;
  }
  for (int64_t i = tid; i < words; i += T) cached[i] = candbm[i] = 0;
  if (tid == 0) rng.seed(seed);
  __syncthreads();
  Totals tot;
  int64_t used = 0;
  for (int64_t b = 0; b < nb; ++b) {
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s, *tab = nbr + 2 * s * k;
    for (int i = tid; i < m2; i += T) w.stamp[q[i]] = (int32_t)b;
    __syncthreads();
    for (int i = tid; i < m2 * k; i += T) {
      const int32_t v = tab[i];
      if (v == 0 || w.stamp[v] == (int32_t)b) continue;
      if (bit(cached, v)) {
        ++tot.reuse;
        tot.dist += b - arrived[v];
        used_at[v] = (int32_t)b;
      } else {
        ++tot.recompute;
        set_bit(candbm, v);
      }
    }
    const int n_cand = list_members(candbm, words, cand, true, s_a);
    const int n_held = list_members(cached, words, held, false, s_a);
    const int room = budget - n_held;
    const int evict = room >= n_cand ? 0 : min(n_cand - room, n_held);
    const int take = (evict + room >= n_cand) ? n_cand : budget;
    if (evict != 0) {
      if (!for_first_by_key(w, held, n_held, evict, used_at, s_a, s_b, [&](int32_t v) { clear_bit(cached, v); })) {
        if (tid == 0) report(status, ORCA_E_TIMEOUT, (int)b);
        break;
      }
    }
    if (tid == 0) rng.shuffle(cand, n_cand);
    __syncthreads();
    for (int i = tid; i < take; i += T) {
      const int32_t v = cand[i];
      set_bit(cached, v);
      used_at[v] = arrived[v] = (int32_t)b;
    }
    const int n_plan = list_members(cached, words, held, false, s_a);
    if (used + n_plan > plan_cap) {
      if (tid == 0) report(status, ORCA_E_CAPACITY, (int)b);
      break;
    }
    for (int i = tid; i < n_plan; i += T) plan[used + i] = held[i];
    if (tid == 0) plan_off[b] = used;
    used += n_plan;
    __syncthreads();
  }
  write_totals(tot, stats);
  if (tid == 0) plan_off[nb] = used;
}

// ------------------------------------------------------------------------------ 2Q (utils/cache.py:175-333)
// a FIFO half and an LRU half of budget / 2 entries each
__global__ void __launch_bounds__(T) twoq_kernel(const int32_t *nodes, const int32_t *nbr, int64_t n_edges, int32_t bs,
                                                 int32_t k, int64_t n_nodes, int32_t budget, uint32_t seed, Work w,
                                                 int32_t *plan, int64_t plan_cap, int64_t *plan_off, int64_t *stats,
                                                 int32_t *status) {
  __shared__ Twister rng;
  __shared__ int s_a[NW], s_b[NW];
  const int tid = threadIdx.x;
  const int64_t nb = (n_edges + bs - 1) / bs, words = (n_nodes + 31) / 32;
  const int half = budget / 2;
  uint32_t *fifo = w.bm[0], *lru = w.bm[1], *promote_bm = w.bm[2], *fresh_bm = w.bm[3], *touched_bm = w.bm[4];
  int32_t *lru_used = w.t0, *lru_arr = w.t1, *fifo_arr = w.t2;
  int32_t *promote = w.list[0], *fresh = w.list[1], *touched = w.list[2], *ids = w.list[3];
  for (int64_t v = tid; v < n_nodes; v += T) {
    w.stamp[v] = -1;
    lru_used[v] = lru_arr[v] = fifo_arr[v] = 0;
  }
  for (int64_t i = tid; i < words; i += T) fifo[i] = lru[i] = promote_bm[i] = fresh_bm[i] = touched_bm[i] = 0;
  if (tid == 0) rng.seed(seed);
  __syncthreads();
  Totals tot;
  int64_t used = 0;
  int n_fifo = 0, n_lru = 0;
  bool failed = false;
  for (int64_t b = 0; b < nb && !failed; ++b) {
    const int32_t now = (int32_t)b;
    const int64_t s = b * bs;
    const int m2 = 2 * (int)(min(n_edges, s + bs) - s);
    const int32_t *q = nodes + 2 * s, *tab = nbr + 2 * s * k;
    for (int i = tid; i < m2; i += T) w.stamp[q[i]] = now;
    __syncthreads();
    for (int i = tid; i < m2 * k; i += T) {
      const int32_t v = tab[i];
      if (v == 0 || w.stamp[v] == now) continue;
      if (bit(fifo, v)) {
        ++tot.reuse;
        tot.dist += now - fifo_arr[v];
        set_bit(promote_bm, v);
      } else if (bit(lru, v)) {
        ++tot.reuse;
        tot.dist += now - lru_arr[v];
        set_bit(touched_bm, v);
      } else {
        ++tot.recompute;
        set_bit(fresh_bm, v);
      }
    }
    const int n_promote = list_members(promote_bm, words, promote, true, s_a);
    const int n_fresh = list_members(fresh_bm, words, fresh, true, s_a);
    const int n_touched = list_members(touched_bm, words, touched, true, s_a);
    // ---- FIFO half
    const int fifo_kept = n_fifo - n_promote, fifo_room = half - fifo_kept;
    for (int i = tid; i < n_promote; i += T) clear_bit(fifo, promote[i]);
    __syncthreads();
    if (n_fresh <= fifo_room) {
      for (int i = tid; i < n_fresh; i += T) {
        set_bit(fifo, fresh[i]);
        fifo_arr[fresh[i]] = now;
      }
      n_fifo = fifo_kept + n_fresh;
    } else if (n_fresh >= half) {
      for (int i = tid; i < n_fresh; i += T) ids[i] = fresh[i];
      for (int64_t i = tid; i < words; i += T) fifo[i] = 0;
      for (int64_t v = tid; v < n_nodes; v += T) fifo_arr[v] = 0;
      __syncthreads();
      if (tid == 0) rng.shuffle(ids, n_fresh);
      __syncthreads();
      for (int i = tid; i < half; i += T) {
        set_bit(fifo, ids[i]);
        fifo_arr[ids[i]] = now;
      }
      n_fifo = half;
    } else {
      const int n_ids = list_members(fifo, words, ids, false, s_a);
      if (tid == 0) rng.shuffle(ids, n_ids);
      __syncthreads();
      for (int i = tid; i < n_fresh - fifo_room; i += T) clear_bit(fifo, ids[i]);
      __syncthreads();
      for (int i = tid; i < n_fresh; i += T) {
        set_bit(fifo, fresh[i]);
        fifo_arr[fresh[i]] = now;
      }
      n_fifo = half;
    }
    __syncthreads();
    // ---- LRU half
    for (int i = tid; i < n_touched; i += T) lru_used[touched[i]] = now;
    __syncthreads();
    const int lru_room = half - n_lru, lru_evictable = n_lru - n_touched;
    auto admit = [&](int32_t v) {
      set_bit(lru, v);
      lru_used[v] = now;
      lru_arr[v] = fifo_arr[v];
    };
    if (n_promote <= lru_room) {
      for (int i = tid; i < n_promote; i += T) admit(promote[i]);
      n_lru += n_promote;
    } else if (n_promote <= lru_room + lru_evictable) {
      const int n_ids = list_members(lru, words, ids, false, s_a);
      if (!for_first_by_key(w, ids, n_ids, n_promote - lru_room, lru_used, s_a, s_b,
                            [&](int32_t v) { clear_bit(lru, v); })) {
        if (tid == 0) report(status, ORCA_E_TIMEOUT, (int)b);
        failed = true;
        continue;
      }
      for (int i = tid; i < n_promote; i += T) admit(promote[i]);
      n_lru = half;
    } else {
      const int n_ids = list_members(lru, words, ids, false, s_a);
      for (int i = tid; i < n_ids; i += T)
        if (lru_used[ids[i]] < now) clear_bit(lru, ids[i]);
      __syncthreads();
      for (int i = tid; i < n_promote; i += T) ids[i] = promote[i];
      __syncthreads();
      if (tid == 0) rng.shuffle(ids, n_promote);
      __syncthreads();
      for (int i = tid; i < half - n_touched; i += T) admit(ids[i]);
      n_lru = half;
    }
    // ---- plan = FIFO ids ascending, then LRU ids ascending
    n_fifo = list_members(fifo, words, ids, false, s_a);
    if (used + n_fifo > plan_cap) {
      if (tid == 0) report(status, ORCA_E_CAPACITY, (int)b);
      break;
    }
    for (int i = tid; i < n_fifo; i += T) plan[used + i] = ids[i];
    n_lru = list_members(lru, words, ids, false, s_a);
    if (used + n_fifo + n_lru > plan_cap) {
      if (tid == 0) report(status, ORCA_E_CAPACITY, (int)b);
      break;
    }
    for (int i = tid; i < n_lru; i += T) plan[used + n_fifo + i] = ids[i];
    if (tid == 0) plan_off[b] = used;
    used += n_fifo + n_lru;
    __syncthreads();
  }
  write_totals(tot, stats);
  if (tid == 0) plan_off[nb] = used;
}

struct Layout {
  int64_t stamp, t[3], bm[5], list[4], sort, total, cap;
};
static Layout layout(int32_t bs, int32_t k, int64_t n_nodes, int32_t budget) {
  Layout L;
  const int64_t words = (n_nodes + 31) / 32;
  L.cap = std::max<int64_t>(2ll * bs * k, budget) + 64;
  int64_t at = 0;
  auto take = [&](int64_t bytes) {
    const int64_t o = at;
    at += (bytes + 255) & ~255ll;
    return o;
  };
  L.stamp = take(n_nodes * 4);
  for (int i = 0; i < 3; ++i) L.t[i] = take(n_nodes * 4);
  for (int i = 0; i < 5; ++i) L.bm[i] = take(words * 4);
  for (int i = 0; i < 4; ++i) L.list[i] = take(L.cap * 4);
  L.sort = take(tie::buf_bytes(L.cap) + 7 * 256);
  L.total = at;
  return L;
}

}  // namespace rnd
}  // namespace orca

using namespace orca;

extern "C" int64_t orca_plan_mrd_workspace_bytes(int64_t n_edges, int32_t bs, int32_t k, int64_t n_nodes, int32_t budget);
extern "C" int orca_plan_mrd(const int32_t *d_nodes, int64_t n_edges, int32_t bs, int32_t k, const int32_t *d_nbr,
                             int64_t n_nodes, int32_t budget, int32_t *d_plan_flat, int64_t plan_cap,
                             int64_t *d_plan_off, int64_t *d_stats, int32_t *d_status, void *d_workspace,
                             int64_t workspace_bytes, void *stream);

extern "C" int64_t orca_plan_device_workspace_bytes(int32_t strategy, int64_t n_edges, int32_t bs, int32_t k,
                                                    int64_t n_nodes, int32_t budget) {
  if (strategy == 0) return orca_plan_mrd_workspace_bytes(n_edges, bs, k, n_nodes, budget);
  if (strategy < 0 || strategy > 2 || n_edges < 0 || bs <= 0 || k < 1 || n_nodes <= 0 || budget <= 0) return -1;
  return rnd::layout(bs, k, n_nodes, budget).total;
}

extern "C" int orca_plan_device(int32_t strategy, const int32_t *d_nodes, int64_t n_edges, int32_t bs, int32_t k,
                                const int32_t *d_nbr, int64_t n_nodes, int32_t budget, uint32_t seed,
                                int32_t *d_plan_flat, int64_t plan_cap, int64_t *d_plan_off, int64_t *d_stats,
                                int32_t *d_status, void *d_workspace, int64_t workspace_bytes, void *stream) {
  if (strategy == 0)
    return orca_plan_mrd(d_nodes, n_edges, bs, k, d_nbr, n_nodes, budget, d_plan_flat, plan_cap, d_plan_off, d_stats,
                         d_status, d_workspace, workspace_bytes, stream);
  ORCA_CHECK_ARG(strategy == 1 || strategy == 2);
  ORCA_CHECK_ARG(d_nodes && d_nbr && d_plan_flat && d_plan_off && d_stats && d_status && d_workspace);
  ORCA_CHECK_ARG(n_edges >= 0 && bs > 0 && k >= 1 && k <= ORCA_MAX_K && n_nodes > 0 && budget > 0);
  ORCA_CHECK_ARG(n_nodes < (1ll << 31) && (n_edges + bs - 1) / bs < (1ll << 30) && 2ll * bs * k < (1ll << 30));
  ORCA_CHECK_ARG(((uintptr_t)d_workspace & 255) == 0);
  const rnd::Layout L = rnd::layout(bs, k, n_nodes, budget);
  if (workspace_bytes < L.total)
    return set_error(ORCA_E_CAPACITY, "orca_plan_device: workspace of %lld bytes, %lld needed",
                     (long long)workspace_bytes, (long long)L.total);
  char *base = (char *)d_workspace;
  rnd::Work w;
  w.stamp = (int32_t *)(base + L.stamp);
  w.t0 = (int32_t *)(base + L.t[0]);
  w.t1 = (int32_t *)(base + L.t[1]);
  w.t2 = (int32_t *)(base + L.t[2]);
  for (int i = 0; i < 5; ++i) w.bm[i] = (uint32_t *)(base + L.bm[i]);
  for (int i = 0; i < 4; ++i) w.list[i] = (int32_t *)(base + L.list[i]);
  w.cap = L.cap;
  {
    char *p = base + L.sort;
    auto take = [&](int64_t bytes) {
      char *o = p;
      p += (bytes + 255) & ~255ll;
      return o;
    };
    w.sort.e = (uint64_t *)take(L.cap * 8);
    w.sort.seg = (int2 *)take(L.cap * 8);
    w.sort.pre = (int2 *)take(L.cap * 8);
    w.sort.lpos = (int32_t *)take(L.cap * 4);
    w.sort.rpos = (int32_t *)take(L.cap * 4);
    w.sort.pivot = (int32_t *)take(L.cap * 4);
    w.sort.swaps = (int32_t *)take(2 * L.cap * 4);
    w.sort.cap = L.cap;
  }
  cudaStream_t s = (cudaStream_t)stream;
  ORCA_CUDA(cudaMemsetAsync(d_stats, 0, 3 * sizeof(int64_t), s));
  if (n_edges == 0) {
    ORCA_CUDA(cudaMemsetAsync(d_plan_off, 0, sizeof(int64_t), s));
    return ORCA_OK;
  }
  if (strategy == 1)
    rnd::lru_kernel<<<1, rnd::T, 0, s>>>(d_nodes, d_nbr, n_edges, bs, k, n_nodes, budget, seed, w, d_plan_flat,
                                        plan_cap, d_plan_off, d_stats, d_status);
  else
    rnd::twoq_kernel<<<1, rnd::T, 0, s>>>(d_nodes, d_nbr, n_edges, bs, k, n_nodes, budget, seed, w, d_plan_flat,
                                         plan_cap, d_plan_off, d_stats, d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}
