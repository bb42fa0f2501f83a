// The order numba's nopython np.argsort leaves among equal keys, reproduced by one thread block.
//
// numba sorts with an unstable quicksort: median of three, pivot parked at the right end, Hoare scans that
// stop on equal keys, ranges of fewer than 16 finished by insertion.  Which of several equal keys end up
// in the first `keep` places therefore depends on every swap it makes.  One partition step moves elements
// only by swapping the m-th position from the left whose key is >= pivot with the m-th position from the
// right whose key is <= pivot, for as long as the former lies left of the latter; both position lists
// follow from prefix counts, so a step is a block-wide scan plus independent swaps, and all ranges of one
// recursion depth are partitioned in the same step.  Ranges that start at or after `keep` are left alone.
// The final insertion sort is stable, so a position's place in its range is its rank by (key, position).
#pragma once

#include "common.cuh"

namespace orca {
namespace tie {

constexpr int T = 1024;     // threads of the block that sorts
constexpr int NW = T / 32;

struct Buf {
  uint64_t *e;       // [cap] key << 32 | payload, in sort order (keys are non-negative int32)
  int2 *seg;         // [cap] range (lo, hi) a position belongs to
  int2 *pre;         // [cap] prefix counts (left list, right list) before the position
  int32_t *lpos, *rpos;   // [cap] positions of a range's left / right list, stored from its lo
  int32_t *pivot;    // [cap] per range, at index lo
  int32_t *swaps;    // [2][cap] per range, at index lo: pair swaps of its step; the halves alternate by
                     // depth, because a step's count is still read while the next pivots are parked
  int64_t cap;
};
__host__ __device__ inline int64_t buf_bytes(int64_t cap) { return cap * (8 + 8 + 8 + 4 + 4 + 4 + 8); }

__device__ __forceinline__ int32_t key_of(uint64_t x) { return (int32_t)(x >> 32); }
__device__ __forceinline__ bool live(int lo, int hi, int keep) { return hi - lo >= 15 && lo < keep; }

// median of three on (lo, mid, hi), pivot parked at hi (the head of numba's partition step)
__device__ __forceinline__ void park_pivot(const Buf &w, int lo, int hi, int32_t *swaps) {
  const int mid = (lo + hi) >> 1;
  uint64_t a = w.e[lo], c = w.e[mid], d = w.e[hi];
  uint64_t t;
  if (key_of(c) < key_of(a)) { t = a; a = c; c = t; }
  if (key_of(d) < key_of(c)) { t = d; d = c; c = t; }
  if (key_of(c) < key_of(a)) { t = a; a = c; c = t; }
  w.e[lo] = a;
  w.e[mid] = d;
  w.e[hi] = c;
  w.pivot[lo] = key_of(c);
  swaps[lo] = 0;
}

// where the pivot of range (lo, hi) ends up once its pair swaps are done
__device__ __forceinline__ int pivot_place(const Buf &w, int lo, int hi, const int32_t *swaps) {
  const int2 a = w.pre[lo], z = w.pre[hi];
  const int n_left = z.x - a.x;
  const int m = swaps[lo];
  const int from_left = m < n_left ? w.lpos[lo + m] : hi;
  const int from_right = m > 0 ? w.rpos[lo + m - 1] : hi;
  return min(from_left, from_right);
}

// All T threads of the block call this with e[0 .. n) filled.  Afterwards every position below `keep` lies
// in a range shorter than 16 (seg) and place_of() gives its final place.  s_l, s_r: NW ints of shared
// memory each.  Returns false if the steps did not end (more steps than entries: a fault, not a state a
// correct run reaches).
__device__ inline bool sort_first(const Buf &w, int n, int keep, int *s_l, int *s_r) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int pos = tid; pos < n; pos += T) w.seg[pos] = make_int2(0, n - 1);
  bool any = n > 0 && live(0, n - 1, keep);
  int32_t *swaps = w.swaps, *swaps_next = w.swaps + w.cap;
  __syncthreads();
  if (any && tid == 0) park_pivot(w, 0, n - 1, swaps);
  __syncthreads();
  const int chunk = ((n + NW - 1) / NW + 31) & ~31;  // positions per warp in the scan
  int depth = 0;
  while (any) {
    if (++depth > n) return false;   // (uniform: every step shortens the longest live range)
    // prefix counts of the left list (key >= pivot) and the right list (key <= pivot) over [lo, hi)
    int cl = 0, cr = 0;
    for (int j = 0; j < chunk; j += 32) {
      const int pos = warp * chunk + j + lane;
      bool is_l = false, is_r = false;
      if (pos < n) {
        const int2 sg = w.seg[pos];
        if (live(sg.x, sg.y, keep) && pos < sg.y) {
          const int32_t kv = key_of(w.e[pos]), pv = w.pivot[sg.x];
          is_l = kv >= pv;
          is_r = kv <= pv;
        }
      }
      cl += __popc(__ballot_sync(0xffffffffu, is_l));
      cr += __popc(__ballot_sync(0xffffffffu, is_r));
    }
    if (lane == 0) {
      s_l[warp] = cl;
      s_r[warp] = cr;
    }
    __syncthreads();
    int bl = 0, br = 0;
    for (int i = 0; i < warp; ++i) {
      bl += s_l[i];
      br += s_r[i];
    }
    for (int j = 0; j < chunk; j += 32) {
      const int pos = warp * chunk + j + lane;
      bool is_l = false, is_r = false;
      if (pos < n) {
        const int2 sg = w.seg[pos];
        if (live(sg.x, sg.y, keep) && pos < sg.y) {
          const int32_t kv = key_of(w.e[pos]), pv = w.pivot[sg.x];
          is_l = kv >= pv;
          is_r = kv <= pv;
        }
      }
      const uint32_t ml = __ballot_sync(0xffffffffu, is_l), mr = __ballot_sync(0xffffffffu, is_r);
      if (pos < n) w.pre[pos] = make_int2(bl + __popc(ml & lt_mask), br + __popc(mr & lt_mask));
      bl += __popc(ml);
      br += __popc(mr);
    }
    __syncthreads();
    // the two position lists of every range
    for (int pos = tid; pos < n; pos += T) {
      const int2 sg = w.seg[pos];
      if (!live(sg.x, sg.y, keep) || pos >= sg.y) continue;
      const int32_t kv = key_of(w.e[pos]), pv = w.pivot[sg.x];
      const int2 me = w.pre[pos];
      if (kv >= pv) w.lpos[sg.x + me.x - w.pre[sg.x].x] = pos;
      if (kv <= pv) w.rpos[sg.x + w.pre[sg.y].y - me.y - 1] = pos;
    }
    __syncthreads();
    // pair m swaps while its left position is left of its right position
    for (int pos = tid; pos < n; pos += T) {
      const int2 sg = w.seg[pos];
      if (!live(sg.x, sg.y, keep) || pos >= sg.y) continue;
      const int2 a = w.pre[sg.x], z = w.pre[sg.y];
      const int pairs = min(z.x - a.x, z.y - a.y);
      const int m = pos - sg.x;
      if (m >= pairs) continue;
      const int pl = w.lpos[pos], pr = w.rpos[pos];
      if (pl >= pr) continue;
      const uint64_t x = w.e[pl], y = w.e[pr];
      w.e[pl] = y;
      w.e[pr] = x;
      if (m + 1 >= pairs || w.lpos[pos + 1] >= w.rpos[pos + 1]) swaps[sg.x] = m + 1;
    }
    __syncthreads();
    // pivot into place, ranges split, next pivots parked
    bool more = false;
    for (int pos = tid; pos < n; pos += T) {
      int2 sg = w.seg[pos];
      if (!live(sg.x, sg.y, keep)) continue;
      const int p = pivot_place(w, sg.x, sg.y, swaps);
      if (pos == p + 1) {
        // the first position right of the pivot's place moves the pivot there (nobody else reads
        // either slot in this phase: hi belongs to the right part, p to no part)
        const uint64_t x = w.e[p], y = w.e[sg.y];
        w.e[p] = y;
        w.e[sg.y] = x;
      }
      if (pos < p) sg.y = p - 1;
      else if (pos > p) sg.x = p + 1;
      else sg.x = sg.y = p;
      w.seg[pos] = sg;
      if (live(sg.x, sg.y, keep)) {
        more = true;
        if (pos == sg.x) park_pivot(w, sg.x, sg.y, swaps_next);
      }
    }
    any = __syncthreads_or(more);
    int32_t *t = swaps;
    swaps = swaps_next;
    swaps_next = t;
  }
  return true;
}

// final place of the entry at position pos (its range is shorter than 16 after sort_first), or -1 when it
// does not lie among the first `keep`
__device__ __forceinline__ int place_of(const Buf &w, int pos, int keep) {
  const int2 sg = w.seg[pos];
  if (sg.x >= keep) return -1;
  const int32_t kv = key_of(w.e[pos]);
  int place = sg.x;
  for (int q = sg.x; q <= sg.y; ++q) {
    const int32_t ko = key_of(w.e[q]);
    place += (ko < kv || (ko == kv && q < pos)) ? 1 : 0;
  }
  return place < keep ? place : -1;
}

}  // namespace tie
}  // namespace orca
