/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's offline cache planners.
 *
 * Nothing that ships may link or call this file: it exists so that the parity tests (and the CPU
 * leg of the benchmark) have an independent statement of what the reference computes.
 *
 * What is restated, with the reference lines each function follows:
 *   mrd_plan   utils/cache.py:92-166   (MRD_numba)
 *   lru_plan   utils/cache.py:338-403  (LRU_numba)
 *   twoq_plan  utils/cache.py:175-333  (TwoQ_numba)
 *
 * Two pieces of the arithmetic live outside the reference, in numba (the reference pins 0.54.1 in
 * README.md:24; parity is anchored on 0.65.0, the version that produced the golden fixtures):
 *   - np.argsort inside nopython code is numba's own unstable quicksort: median of three pivot,
 *     Hoare-style partition with the pivot parked at the right end, explicit stack that always
 *     continues with the smaller side, insertion sort for ranges shorter than 16.  The order of
 *     equal keys is part of the observable result (MRD keeps the first `budget` entries of it), so
 *     nb_argsort_* below performs the same sequence of comparisons and swaps.
 *   - np.random.choice(a, k, replace=False) inside nopython code is a Fisher-Yates shuffle of a
 *     copy of `a` driven by numba's private MT19937, seeded with np.random.seed(s) from jitted
 *     code (Knuth's linear-congruential initialisation), drawing masked 32-bit words with
 *     rejection, and returns the first k entries.
 *
 * Parity status: pinned by the golden fixtures under tests/golden (plans produced by the
 * reference itself under numba 0.65.0 with the generator seeded to 0).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ MT19937 (numba's private RNG) */
typedef struct { uint32_t mt[624]; int idx; } mt_t;

static void mt_seed(mt_t *s, uint32_t seed) {
  s->mt[0] = seed;
  for (int i = 1; i < 624; i++)
    s->mt[i] = 1812433253u * (s->mt[i - 1] ^ (s->mt[i - 1] >> 30)) + (uint32_t)i;
  s->idx = 624;
}

static void mt_twist(mt_t *s) {
  uint32_t *m = s->mt;
  for (int i = 0; i < 624; i++) {
    uint32_t y = (m[i] & 0x80000000u) | (m[(i + 1) % 624] & 0x7fffffffu);
    uint32_t v = m[(i + 397) % 624] ^ (y >> 1);
    if (y & 1u) v ^= 0x9908b0dfu;
    m[i] = v;
  }
}

static uint32_t mt_next(mt_t *s) {
  if (s->idx >= 624) { mt_twist(s); s->idx = 0; }
  uint32_t y = s->mt[s->idx++];
  y ^= y >> 11;
  y ^= (y << 7) & 0x9d2c5680u;
  y ^= (y << 15) & 0xefc60000u;
  y ^= y >> 18;
  return y;
}

/* np.random.randint(0, n) as numba lowers it: bits of (n-1), masked draw, reject >= n */
static int64_t mt_below(mt_t *s, int64_t n) {
  if (n == 1) return 0;
  uint64_t m = (uint64_t)(n - 1);
  int nbits = 0;
  while (m) { nbits++; m >>= 1; }
  for (;;) {
    uint64_t r;
    if (nbits <= 32) {
      r = mt_next(s) & (0xffffffffu >> (32 - nbits));
    } else {
      uint64_t hi = mt_next(s) & (0xffffffffu >> (64 - nbits));
      uint64_t lo = mt_next(s);
      r = (hi << 32) | lo;
    }
    if ((int64_t)r < n) return (int64_t)r;
  }
}

/* in-place shuffle: i from n-1 down to 1, swap with j = randint(i+1) */
static void mt_shuffle(mt_t *s, int64_t *x, int64_t n) {
  for (int64_t i = n - 1; i > 0; i--) {
    int64_t j = mt_below(s, i + 1);
    int64_t t = x[i]; x[i] = x[j]; x[j] = t;
  }
}

/* ------------------------------------------------------------------ numba's argsort (quicksort) */
#define NB_SMALL 15
#define DEFINE_ARGSORT(NAME, T)                                                          \
  static void NAME##_ins(const T *a, int64_t *r, int64_t lo, int64_t hi) {              \
    for (int64_t i = lo + 1; i <= hi; i++) {                                            \
      int64_t k = r[i]; T v = a[k]; int64_t j = i;                                      \
      while (j > lo && v < a[r[j - 1]]) { r[j] = r[j - 1]; j--; }                       \
      r[j] = k;                                                                         \
    }                                                                                   \
  }                                                                                     \
  static int64_t NAME##_part(const T *a, int64_t *r, int64_t lo, int64_t hi) {          \
    int64_t mid = (lo + hi) >> 1, t;                                                    \
    if (a[r[mid]] < a[r[lo]]) { t = r[lo]; r[lo] = r[mid]; r[mid] = t; }                \
    if (a[r[hi]] < a[r[mid]]) { t = r[hi]; r[hi] = r[mid]; r[mid] = t; }                \
    if (a[r[mid]] < a[r[lo]]) { t = r[lo]; r[lo] = r[mid]; r[mid] = t; }                \
    T pv = a[r[mid]];                                                                   \
    t = r[hi]; r[hi] = r[mid]; r[mid] = t;                                              \
    int64_t i = lo, j = hi - 1;                                                         \
    for (;;) {                                                                          \
      while (i < hi && a[r[i]] < pv) i++;                                               \
      while (j >= lo && pv < a[r[j]]) j--;                                              \
      if (i >= j) break;                                                                \
      t = r[i]; r[i] = r[j]; r[j] = t; i++; j--;                                        \
    }                                                                                   \
    t = r[i]; r[i] = r[hi]; r[hi] = t;                                                  \
    return i;                                                                           \
  }                                                                                     \
  void NAME(const T *a, int64_t n, int64_t *r) {                                        \
    for (int64_t i = 0; i < n; i++) r[i] = i;                                           \
    if (n < 2) return;                                                                  \
    int64_t slo[128], shi[128]; int sp = 0;                                             \
    slo[0] = 0; shi[0] = n - 1; sp = 1;                                                 \
    while (sp > 0) {                                                                    \
      sp--; int64_t lo = slo[sp], hi = shi[sp];                                         \
      while (hi - lo >= NB_SMALL) {                                                     \
        int64_t i = NAME##_part(a, r, lo, hi);                                          \
        if (hi - i > i - lo) {                                                          \
          if (hi > i) { slo[sp] = i + 1; shi[sp] = hi; sp++; }                          \
          hi = i - 1;                                                                   \
        } else {                                                                        \
          if (i > lo) { slo[sp] = lo; shi[sp] = i - 1; sp++; }                          \
          lo = i + 1;                                                                   \
        }                                                                               \
      }                                                                                 \
      NAME##_ins(a, r, lo, hi);                                                         \
    }                                                                                   \
  }

DEFINE_ARGSORT(nb_argsort_i64, int64_t)
DEFINE_ARGSORT(nb_argsort_f64, double)

/* ------------------------------------------------------------------ helpers */
static int cmp_i64(const void *a, const void *b) {
  int64_t x = *(const int64_t *)a, y = *(const int64_t *)b;
  return (x > y) - (x < y);
}

/* sorted unique in place, returns new length */
static int64_t sort_unique(int64_t *x, int64_t n) {
  if (n == 0) return 0;
  qsort(x, (size_t)n, sizeof(int64_t), cmp_i64);
  int64_t m = 1;
  for (int64_t i = 1; i < n; i++) if (x[i] != x[m - 1]) x[m++] = x[i];
  return m;
}

/* ids with flag==1, ascending (np.where(flag==1)[0]) */
static int64_t where_set(const uint8_t *flag, int64_t n, int64_t *out) {
  int64_t m = 0;
  for (int64_t i = 0; i < n; i++) if (flag[i]) out[m++] = i;
  return m;
}

/* ------------------------------------------------------------------ MRD
 * Lists arrive flattened: batch b's unique sorted targets are tgt[tgt_off[b]..tgt_off[b+1]), its
 * out-of-batch neighbour occurrences (not unique, table order) ngh[ngh_off[b]..), and node v's
 * occurrence records (batch, kind) occ_batch/occ_kind[occ_off[v]..occ_off[v+1]) with record 0 the
 * dummy (0,0) and the last record (num_batch, 2).
 * plan_flat needs room for num_batch*budget entries.  stats = {n_reuse, n_recompute, sum of reuse
 * distances}.  Returns 0.
 */
int mrd_plan(int64_t n_nodes, int64_t num_batch, int64_t budget,
             const int64_t *tgt_off, const int64_t *tgt,
             const int64_t *ngh_off, const int32_t *ngh,
             const int64_t *occ_off, const int32_t *occ_batch, const uint8_t *occ_kind,
             int64_t *plan_flat, int64_t *plan_off, double *stats) {
  const int64_t MAXD = 100000000;
  uint8_t *flag = (uint8_t *)calloc((size_t)n_nodes, 1);
  uint8_t *is_new = (uint8_t *)calloc((size_t)n_nodes, 1);
  double *time_flag = (double *)calloc((size_t)n_nodes, sizeof(double));
  int32_t *cursor = (int32_t *)malloc((size_t)n_nodes * sizeof(int32_t));
  for (int64_t i = 0; i < n_nodes; i++) cursor[i] = 1;
  int64_t max_ngh = 0, max_tgt = 0;
  for (int64_t b = 0; b < num_batch; b++) {
    if (ngh_off[b + 1] - ngh_off[b] > max_ngh) max_ngh = ngh_off[b + 1] - ngh_off[b];
    if (tgt_off[b + 1] - tgt_off[b] > max_tgt) max_tgt = tgt_off[b + 1] - tgt_off[b];
  }
  int64_t cap = max_ngh + max_tgt + budget + 8;
  int64_t *cand = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  int64_t *dist = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  int64_t *perm = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  int64_t *newc = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  int64_t *cached = (int64_t *)malloc((size_t)(budget + 8) * sizeof(int64_t));
  int64_t n_cached = 0;
  double n_reuse = 0, n_recompute = 0, total_dist = 0;
  plan_off[0] = 0;
  for (int64_t b = 0; b < num_batch; b++) {
    const int32_t *g = ngh + ngh_off[b];
    int64_t ng = ngh_off[b + 1] - ngh_off[b];
    const int64_t *t = tgt + tgt_off[b];
    int64_t nt = tgt_off[b + 1] - tgt_off[b];
    int64_t nc = 0, nn = 0;
    for (int64_t i = 0; i < ng; i++) {
      int64_t v = g[i];
      if (flag[v]) { n_reuse += 1; total_dist += (double)b - time_flag[v]; }
      else { n_recompute += 1; cand[nc++] = v; newc[nn++] = v; }
    }
    for (int64_t i = 0; i < n_cached; i++) cand[nc++] = cached[i];
    for (int64_t i = 0; i < nt; i++) { cand[nc++] = t[i]; newc[nn++] = t[i]; }
    nc = sort_unique(cand, nc);
    for (int64_t i = 0; i < nn; i++) is_new[newc[i]] = 1;
    for (int64_t i = 0; i < nc; i++) {
      int64_t v = cand[i];
      int64_t o = occ_off[v] + cursor[v];
      while (occ_batch[o] <= b) o++;
      cursor[v] = (int32_t)(o - occ_off[v]);
      dist[i] = (occ_kind[o] == 1) ? (int64_t)occ_batch[o] - b : MAXD + 1;
    }
    nb_argsort_i64(dist, nc, perm);
    for (int64_t i = 0; i < n_cached; i++) flag[cached[i]] = 0;
    int64_t keep = nc < budget ? nc : budget;
    int64_t *out = plan_flat + plan_off[b];
    for (int64_t i = 0; i < keep; i++) {
      int64_t v = cand[perm[i]];
      out[i] = v; flag[v] = 1;
      if (is_new[v]) time_flag[v] = (double)b;
    }
    plan_off[b + 1] = plan_off[b] + keep;
    /* cached set for the next batch: ascending ids */
    memcpy(cached, out, (size_t)keep * sizeof(int64_t));
    qsort(cached, (size_t)keep, sizeof(int64_t), cmp_i64);
    n_cached = keep;
    for (int64_t i = 0; i < nn; i++) is_new[newc[i]] = 0;
  }
  stats[0] = n_reuse; stats[1] = n_recompute; stats[2] = total_dist;
  free(flag); free(is_new); free(time_flag); free(cursor); free(cand); free(dist); free(perm);
  free(newc); free(cached);
  return 0;
}

/* ------------------------------------------------------------------ LRU
 * plan_flat needs room for num_batch*budget entries. */
int lru_plan(int64_t n_nodes, int64_t num_batch, int64_t budget,
             const int64_t *ngh_off, const int32_t *ngh, uint32_t seed,
             int64_t *plan_flat, int64_t *plan_off, double *stats) {
  mt_t rng; mt_seed(&rng, seed);
  uint8_t *flag = (uint8_t *)calloc((size_t)n_nodes, 1);
  double *time_flag = (double *)calloc((size_t)n_nodes, sizeof(double));
  double *arrive = (double *)calloc((size_t)n_nodes, sizeof(double));
  int64_t max_ngh = 0;
  for (int64_t b = 0; b < num_batch; b++)
    if (ngh_off[b + 1] - ngh_off[b] > max_ngh) max_ngh = ngh_off[b + 1] - ngh_off[b];
  int64_t *cand = (int64_t *)malloc((size_t)(max_ngh + 8) * sizeof(int64_t));
  int64_t *cached = (int64_t *)malloc((size_t)(n_nodes + 8) * sizeof(int64_t));
  int64_t *perm = (int64_t *)malloc((size_t)(n_nodes + 8) * sizeof(int64_t));
  double *last = (double *)malloc((size_t)(n_nodes + 8) * sizeof(double));
  double n_reuse = 0, n_recompute = 0, total_dist = 0;
  plan_off[0] = 0;
  for (int64_t b = 0; b < num_batch; b++) {
    const int32_t *g = ngh + ngh_off[b];
    int64_t ng = ngh_off[b + 1] - ngh_off[b];
    int64_t nc = 0;
    for (int64_t i = 0; i < ng; i++) {
      int64_t v = g[i];
      if (flag[v]) { n_reuse += 1; total_dist += (double)b - arrive[v]; }
      else { n_recompute += 1; cand[nc++] = v; }
    }
    for (int64_t i = 0; i < ng; i++) if (flag[g[i]]) time_flag[g[i]] = (double)b;
    int64_t n_cached = where_set(flag, n_nodes, cached);
    nc = sort_unique(cand, nc);
    int64_t avail = budget - n_cached;
    int64_t evict = 0;
    if (avail < nc) { evict = nc - avail; if (evict > n_cached) evict = n_cached; }
    int64_t to_cache = (evict + avail >= nc) ? nc : budget;
    if (evict != 0) {
      for (int64_t i = 0; i < n_cached; i++) last[i] = time_flag[cached[i]];
      nb_argsort_f64(last, n_cached, perm);
      for (int64_t i = 0; i < evict; i++) flag[cached[perm[i]]] = 0;
    }
    mt_shuffle(&rng, cand, nc);
    for (int64_t i = 0; i < to_cache; i++) {
      int64_t v = cand[i];
      flag[v] = 1; time_flag[v] = (double)b; arrive[v] = (double)b;
    }
    int64_t m = where_set(flag, n_nodes, plan_flat + plan_off[b]);
    plan_off[b + 1] = plan_off[b] + m;
  }
  stats[0] = n_reuse; stats[1] = n_recompute; stats[2] = total_dist;
  free(flag); free(time_flag); free(arrive); free(cand); free(cached); free(perm); free(last);
  return 0;
}

/* ------------------------------------------------------------------ 2Q
 * A FIFO half and an LRU half of budget/2 entries each.  plan = ids in the FIFO half (ascending)
 * followed by ids in the LRU half (ascending).  plan_flat needs num_batch*(budget+2) entries. */
int twoq_plan(int64_t n_nodes, int64_t num_batch, int64_t budget,
              const int64_t *ngh_off, const int32_t *ngh, uint32_t seed,
              int64_t *plan_flat, int64_t *plan_off, double *stats) {
  mt_t rng; mt_seed(&rng, seed);
  int64_t half = budget / 2;
  uint8_t *lru_f = (uint8_t *)calloc((size_t)n_nodes, 1);
  uint8_t *fif_f = (uint8_t *)calloc((size_t)n_nodes, 1);
  double *lru_time = (double *)calloc((size_t)n_nodes, sizeof(double));
  double *lru_arr = (double *)calloc((size_t)n_nodes, sizeof(double));
  double *fif_arr = (double *)calloc((size_t)n_nodes, sizeof(double));
  int64_t max_ngh = 0;
  for (int64_t b = 0; b < num_batch; b++)
    if (ngh_off[b + 1] - ngh_off[b] > max_ngh) max_ngh = ngh_off[b + 1] - ngh_off[b];
  int64_t *f2l = (int64_t *)malloc((size_t)(max_ngh + 8) * sizeof(int64_t));   /* FIFO hits   */
  int64_t *newf = (int64_t *)malloc((size_t)(max_ngh + 8) * sizeof(int64_t));  /* misses      */
  int64_t *l2l = (int64_t *)malloc((size_t)(max_ngh + 8) * sizeof(int64_t));   /* LRU hits    */
  int64_t *tmp = (int64_t *)malloc((size_t)(n_nodes + 8) * sizeof(int64_t));
  int64_t *perm = (int64_t *)malloc((size_t)(n_nodes + 8) * sizeof(int64_t));
  double *last = (double *)malloc((size_t)(n_nodes + 8) * sizeof(double));
  int64_t n_fif = 0, n_lru = 0;
  double n_reuse = 0, n_recompute = 0, total_dist = 0;
  plan_off[0] = 0;
  for (int64_t b = 0; b < num_batch; b++) {
    const int32_t *g = ngh + ngh_off[b];
    int64_t ng = ngh_off[b + 1] - ngh_off[b];
    int64_t n_f2l = 0, n_new = 0, n_l2l = 0;
    for (int64_t i = 0; i < ng; i++) {
      int64_t v = g[i];
      if (fif_f[v]) { n_reuse += 1; total_dist += (double)b - fif_arr[v]; f2l[n_f2l++] = v; }
      else if (lru_f[v]) { n_reuse += 1; total_dist += (double)b - lru_arr[v]; l2l[n_l2l++] = v; }
      else { n_recompute += 1; newf[n_new++] = v; }
    }
    n_f2l = sort_unique(f2l, n_f2l);
    n_new = sort_unique(newf, n_new);
    n_l2l = sort_unique(l2l, n_l2l);

    /* FIFO half */
    int64_t fif_used = n_fif - n_f2l;
    int64_t fif_avail = half - fif_used;
    for (int64_t i = 0; i < n_f2l; i++) fif_f[f2l[i]] = 0;
    if (n_new <= fif_avail) {
      for (int64_t i = 0; i < n_new; i++) { fif_f[newf[i]] = 1; fif_arr[newf[i]] = (double)b; }
      n_fif = fif_used + n_new;
    } else if (n_new >= half) {
      memcpy(tmp, newf, (size_t)n_new * sizeof(int64_t));
      mt_shuffle(&rng, tmp, n_new);
      memset(fif_f, 0, (size_t)n_nodes);
      memset(fif_arr, 0, (size_t)n_nodes * sizeof(double));
      for (int64_t i = 0; i < half; i++) { fif_f[tmp[i]] = 1; fif_arr[tmp[i]] = (double)b; }
      n_fif = half;
    } else {
      int64_t n_evict = n_new - fif_avail;
      int64_t m = where_set(fif_f, n_nodes, tmp);
      mt_shuffle(&rng, tmp, m);
      for (int64_t i = 0; i < n_evict; i++) fif_f[tmp[i]] = 0;
      for (int64_t i = 0; i < n_new; i++) { fif_f[newf[i]] = 1; fif_arr[newf[i]] = (double)b; }
      n_fif = half;
    }

    /* LRU half */
    for (int64_t i = 0; i < n_l2l; i++) lru_time[l2l[i]] = (double)b;
    int64_t lru_avail = half - n_lru;
    int64_t lru_may_evict = n_lru - n_l2l;
    if (n_f2l <= lru_avail) {
      for (int64_t i = 0; i < n_f2l; i++) {
        int64_t v = f2l[i]; lru_f[v] = 1; lru_time[v] = (double)b; lru_arr[v] = fif_arr[v];
      }
      n_lru += n_f2l;
    } else if (n_f2l <= lru_avail + lru_may_evict) {
      int64_t n_evict = n_f2l - lru_avail;
      int64_t m = where_set(lru_f, n_nodes, tmp);
      for (int64_t i = 0; i < m; i++) last[i] = lru_time[tmp[i]];
      nb_argsort_f64(last, m, perm);
      for (int64_t i = 0; i < n_evict; i++) lru_f[tmp[perm[i]]] = 0;
      for (int64_t i = 0; i < n_f2l; i++) {
        int64_t v = f2l[i]; lru_f[v] = 1; lru_time[v] = (double)b; lru_arr[v] = fif_arr[v];
      }
      n_lru = half;
    } else {
      int64_t m = where_set(lru_f, n_nodes, tmp);
      for (int64_t i = 0; i < m; i++) if (lru_time[tmp[i]] < (double)b) lru_f[tmp[i]] = 0;
      int64_t n_sel = half - n_l2l;
      memcpy(tmp, f2l, (size_t)n_f2l * sizeof(int64_t));
      mt_shuffle(&rng, tmp, n_f2l);
      for (int64_t i = 0; i < n_sel; i++) {
        int64_t v = tmp[i]; lru_f[v] = 1; lru_time[v] = (double)b; lru_arr[v] = fif_arr[v];
      }
      n_lru = half;
    }

    int64_t *out = plan_flat + plan_off[b];
    n_fif = where_set(fif_f, n_nodes, out);
    n_lru = where_set(lru_f, n_nodes, out + n_fif);
    plan_off[b + 1] = plan_off[b] + n_fif + n_lru;
  }
  stats[0] = n_reuse; stats[1] = n_recompute; stats[2] = total_dist;
  free(lru_f); free(fif_f); free(lru_time); free(lru_arr); free(fif_arr);
  free(f2l); free(newf); free(l2l); free(tmp); free(perm); free(last);
  return 0;
}
