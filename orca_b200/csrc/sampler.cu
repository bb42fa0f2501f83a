// Index-side kernels: adjacency build, temporal neighbour sampling, uncached-neighbour discovery
// and last-occurrence selection.  All results are integers (or exact conversions) and must equal
// the reference's bit for bit.
#include <algorithm>
#include <numeric>
#include <stdarg.h>
#include <vector>

#include "common.cuh"
#include "context.cuh"

namespace orca {

static thread_local char g_err[512] = "";
int set_error(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int &launch_counter() {
  static thread_local int c = 0;
  return c;
}

// ---------------------------------------------------------------------------------------------
// Sampling.  A group of G lanes (16 when k <= 16, else 32) serves one query.  The lower bound of
// the query time inside the node's time-sorted segment is found by a G-ary search: every round the
// lanes probe G evenly spaced timestamps, a ballot counts how many are smaller than the query time
// and the segment shrinks by a factor G+1, so a hub with millions of interactions needs five or six
// dependent loads instead of twenty-two.  The lanes then copy the k entries in front of the bound.
// ---------------------------------------------------------------------------------------------
template <int G>
__device__ __forceinline__ long long lower_bound_group(const double *__restrict__ ts, long long lo,
                                                       long long hi, double t, int lane,
                                                       unsigned gmask, int gshift) {
  // invariant: every index < lo has ts < t, every index >= hi has ts >= t
  while (hi - lo > G) {
    long long len = hi - lo;
    long long p = lo + (len * (lane + 1)) / (G + 1);
    bool less = ts[p] < t;
    unsigned b = (__ballot_sync(gmask, less) >> gshift) & ((G == 32) ? 0xffffffffu : ((1u << G) - 1u));
    int cnt = __popc(b);  // probes are increasing, so `less` holds for a prefix of the lanes
    long long nlo = cnt > 0 ? lo + (len * cnt) / (G + 1) + 1 : lo;
    long long nhi = cnt < G ? lo + (len * (cnt + 1)) / (G + 1) : hi;
    lo = nlo;
    hi = nhi;
  }
  long long p = lo + lane;
  bool less = (p < hi) && (ts[p] < t);
  unsigned b = (__ballot_sync(gmask, less) >> gshift) & ((G == 32) ? 0xffffffffu : ((1u << G) - 1u));
  return lo + __popc(b);
}

// One query: lower bound, copy of the k entries in front of it (right-aligned, zero padded), and --
// optionally -- marking of the sampled neighbours as candidates of the uncached set: the neighbour
// (the padding node 0 for an empty slot) gets its bit in `cand_bitmap` when its cache flag is clear.
// Hub nodes are sampled thousands of times per batch, so the bit is tested first and only the first
// few writers pay for an atomic on the same word; the one writer that flips the bit also appends the id
// to `cand_list` (if given), which lets the finishing kernel skip the scan of the whole bitmap.
template <int G>
__device__ __forceinline__ void sample_query(const int64_t *__restrict__ indptr, const int32_t *__restrict__ adj_nbr,
                                             const int32_t *__restrict__ adj_eid, const double *__restrict__ adj_ts,
                                             int64_t n_nodes, int node, double t, int q, int k, int lane,
                                             unsigned gmask, int gshift, int32_t *__restrict__ o_nbr,
                                             int32_t *__restrict__ o_eid, float *__restrict__ o_et,
                                             float *__restrict__ o_dt, int32_t *status,
                                             const uint8_t *__restrict__ cache_flag, uint32_t *__restrict__ cand_bitmap,
                                             int32_t *__restrict__ cand_count, int32_t *__restrict__ cand_list,
                                             const unsigned long long *__restrict__ last_pos = nullptr,
                                             unsigned long long base = 0) {
  long long beg = 0, end = 0;
  if (node >= 0 && node < n_nodes) {
    beg = indptr[node];
    end = indptr[node + 1];
  } else {
    report(status, ORCA_E_BOUNDS, q);
  }
  const long long bound = lower_bound_group<G>(adj_ts, beg, end, t, lane, gmask, gshift);
  if (lane < k) {
    const long long src = bound - k + lane;
    int nb = 0, ei = 0;
    float et = 0.f;
    if (src >= beg) {
      nb = adj_nbr[src];
      ei = adj_eid[src];
      et = (float)adj_ts[src];
    }
    const size_t o = (size_t)q * k + lane;
    o_nbr[o] = nb;
    o_eid[o] = ei;
    if (o_et) o_et[o] = et;
    if (o_dt) o_dt[o] = (float)(t - (double)et);
    // (with `last_pos`: a neighbour whose record already carries this batch's epoch is a row of the
    // batch and can be skipped; rows recorded later than this test slip through and are removed by the
    // finishing kernel, which sees all records)
    if (cand_bitmap != nullptr && cache_flag[nb] == 0 && (last_pos == nullptr || __ldcg(&last_pos[nb]) < base)) {
      const uint32_t bit = 1u << (nb & 31);
      if ((__ldcg(&cand_bitmap[nb >> 5]) & bit) == 0) {
        const uint32_t old = atomicOr(&cand_bitmap[nb >> 5], bit);
        if (cand_list != nullptr && (old & bit) == 0) {
          const int pos = atomicAdd(cand_count, 1);
          if (pos < ORCA_CAND_CAP) cand_list[pos] = nb;
        }
      }
    }
  }
}

template <int G>
__global__ void __launch_bounds__(256)
sample_topk_kernel(const int64_t *__restrict__ indptr, const int32_t *__restrict__ adj_nbr,
                   const int32_t *__restrict__ adj_eid, const double *__restrict__ adj_ts,
                   int64_t n_nodes, const int32_t *__restrict__ nodes, const double *__restrict__ qts,
                   int n_cap, const int32_t *__restrict__ d_n, int k, int32_t *__restrict__ o_nbr,
                   int32_t *__restrict__ o_eid, float *__restrict__ o_et, float *__restrict__ o_dt,
                   int32_t *status, const uint8_t *__restrict__ cache_flag, uint32_t *__restrict__ cand_bitmap) {
  dep_trigger();
  dep_wait();
  const int n = rows_of(n_cap, d_n);
  const int groups_per_block = blockDim.x / G;
  const int lane = threadIdx.x % G;
  const int gshift = (threadIdx.x % 32) / G * G;
  const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << gshift);
  for (int q = blockIdx.x * groups_per_block + threadIdx.x / G; q < n; q += gridDim.x * groups_per_block)
    sample_query<G>(indptr, adj_nbr, adj_eid, adj_ts, n_nodes, nodes[q], qts[q], q, k, lane, gmask, gshift, o_nbr,
                    o_eid, o_et, o_dt, status, cache_flag, cand_bitmap, nullptr, nullptr);
}

// The head of an eval batch in one launch: row list [src | dst | neg] with its query times and the
// [dst | src] partner list, the top-level neighbour table of those rows (which is also the layer-1
// table of the same rows), candidate marking, and the last-occurrence record of every row's node
// (History.push keeps the last of duplicate ids: atomicMax of epoch + position).
template <int G>
__global__ void __launch_bounds__(256)
batch_head_kernel(const int64_t *__restrict__ indptr, const int32_t *__restrict__ adj_nbr,
                  const int32_t *__restrict__ adj_eid, const double *__restrict__ adj_ts, int64_t n_nodes,
                  const int32_t *__restrict__ batch, const double *__restrict__ bts, int b, int k,
                  int32_t *__restrict__ nodes1, double *__restrict__ ts1, int32_t *__restrict__ cat_dst,
                  int32_t *__restrict__ o_nbr, int32_t *__restrict__ o_eid, float *__restrict__ o_dt, int32_t *status,
                  const uint8_t *__restrict__ cache_flag, uint32_t *__restrict__ cand_bitmap,
                  int32_t *__restrict__ cand_count, int32_t *__restrict__ cand_list,
                  unsigned long long *__restrict__ last_pos, long long base) {
  dep_trigger();
  dep_wait();
  const int n = 3 * b;
  const int groups_per_block = blockDim.x / G;
  const int lane = threadIdx.x % G;
  const int gshift = (threadIdx.x % 32) / G * G;
  const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << gshift);
  for (int q = blockIdx.x * groups_per_block + threadIdx.x / G; q < n; q += gridDim.x * groups_per_block) {
    const int node = batch[q];
    const double t = bts[q % b];
    if (lane == 0) {
      nodes1[q] = node;
      ts1[q] = t;
      if (q < 2 * b) cat_dst[q] = q < b ? batch[b + q] : batch[q - b];
      if (node >= 0 && node < n_nodes) atomicMax(&last_pos[node], (unsigned long long)(base + q));
    }
    sample_query<G>(indptr, adj_nbr, adj_eid, adj_ts, n_nodes, node, t, q, k, lane, gmask, gshift, o_nbr, o_eid,
                    nullptr, o_dt, status, cache_flag, cand_bitmap, cand_count, cand_list, last_pos,
                    (unsigned long long)base);
  }
}

__global__ void find_before_kernel(const int64_t *__restrict__ indptr, const double *__restrict__ adj_ts,
                                   int64_t n_nodes, const int32_t *__restrict__ nodes,
                                   const double *__restrict__ qts, int n, int32_t *__restrict__ out) {
  const int lane = threadIdx.x % 32;
  for (int q = (blockIdx.x * blockDim.x + threadIdx.x) / 32; q < n; q += gridDim.x * blockDim.x / 32) {
    const int node = nodes[q];
    long long beg = 0, end = 0;
    if (node >= 0 && node < n_nodes) {
      beg = indptr[node];
      end = indptr[node + 1];
    }
    long long b = lower_bound_group<32>(adj_ts, beg, end, qts[q], lane, 0xffffffffu, 0);
    if (lane == 0) out[q] = (int32_t)(b - beg);
  }
}

// ---------------------------------------------------------------------------------------------
// Uncached out-of-batch neighbours: one CTA builds a bitmap over node ids (in shared memory when
// n_nodes bits fit, else in the scratch the caller passed), marks every neighbour id whose cache
// flag is 0 (id 0, the padding node, included: its flag is never set), clears the bits of the query
// nodes, and emits the set bits in ascending order -- which is the sorted unique array the
// reference builds with np.unique / np.isin -- skipping the first one.
// ---------------------------------------------------------------------------------------------
constexpr int FU_THREADS = 1024;
constexpr int FU_SMEM_WORDS = 48 * 1024;  // 192 KB of bitmap = 1.57 M node ids

__global__ void __launch_bounds__(FU_THREADS)
find_uncached_kernel(const int32_t *__restrict__ nbr, int n_query, int k, const uint8_t *__restrict__ flag,
                     int64_t n_nodes, int32_t *__restrict__ nodes_io, double *__restrict__ ts_io,
                     int u_cap, int32_t *__restrict__ d_n_total, uint32_t *__restrict__ gbitmap,
                     int32_t *status) {
  extern __shared__ uint32_t s_bitmap[];
  __shared__ int s_scan[FU_THREADS / 32];
  __shared__ double s_tmax[FU_THREADS / 32];
  __shared__ int s_total;
  const int n_words = (int)((n_nodes + 31) / 32);
  uint32_t *bm = (n_words <= FU_SMEM_WORDS) ? s_bitmap : gbitmap;
  const int tid = threadIdx.x;
  for (int w = tid; w < n_words; w += FU_THREADS) bm[w] = 0u;
  __syncthreads();
  const int n_slots = n_query * k;
  // eight ids and then their eight cache flags are loaded before any of them is used, so the
  // dependent (id -> flag) global loads of a thread overlap instead of queueing behind each other
  for (int i0 = tid; i0 < n_slots; i0 += 8 * FU_THREADS) {
    int v[8];
    uint8_t fl[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * FU_THREADS;
      v[u] = i < n_slots ? nbr[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) fl[u] = (v[u] >= 0 && v[u] < n_nodes) ? flag[v[u]] : (uint8_t)1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (fl[u] == 0 && (((volatile uint32_t *)bm)[v[u] >> 5] & (1u << (v[u] & 31))) == 0)
        atomicOr(&bm[v[u] >> 5], 1u << (v[u] & 31));
      if (i0 + u * FU_THREADS < n_slots && (v[u] < 0 || v[u] >= n_nodes)) report(status, ORCA_E_BOUNDS, i0);
    }
  }
  // max query time (modules/embedding_module.py:254), fused here: one pass over n_query doubles
  double tmax = -1.0e300;
  for (int i = tid; i < n_query; i += FU_THREADS) tmax = fmax(tmax, ts_io[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
  if ((tid & 31) == 0) s_tmax[tid >> 5] = tmax;
  __syncthreads();
  for (int i = tid; i < n_query; i += FU_THREADS) {
    const int v = nodes_io[i];
    if (v >= 0 && v < n_nodes && (((volatile uint32_t *)bm)[v >> 5] & (1u << (v & 31))) != 0)
      atomicAnd(&bm[v >> 5], ~(1u << (v & 31)));
  }
  __syncthreads();
  tmax = s_tmax[0];
  for (int i = 1; i < FU_THREADS / 32; ++i) tmax = fmax(tmax, s_tmax[i]);
  // ordered compaction: each thread owns a contiguous run of words
  const int per = (n_words + FU_THREADS - 1) / FU_THREADS;
  const int w0 = tid * per;
  const int w1 = min(n_words, w0 + per);
  int cnt = 0;
  for (int w = w0; w < w1; ++w) cnt += __popc(bm[w]);
  // block exclusive scan of cnt
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += y;
  }
  if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    int v = s_scan[tid];
    int inc2 = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, inc2, o);
      if (tid >= o) inc2 += y;
    }
    s_scan[tid] = inc2 - v;
    if (tid == 31) s_total = inc2;
  }
  __syncthreads();
  int rank = s_scan[tid >> 5] + incl - cnt;  // number of set bits before this thread's run
  for (int w = w0; w < w1; ++w) {
    uint32_t bits = bm[w];
    while (bits) {
      const int bit = __ffs(bits) - 1;
      bits &= bits - 1;
      // rank 0 is dropped ("filter out dummy node", modules/embedding_module.py:212)
      if (rank >= 1) {
        const int slot = rank - 1;
        if (slot < u_cap) {
          nodes_io[n_query + slot] = w * 32 + bit;
          ts_io[n_query + slot] = tmax;
        }
      }
      ++rank;
    }
  }
  if (tid == 0) {
    int u = s_total > 0 ? s_total - 1 : 0;
    if (u > u_cap) {
      report(status, ORCA_E_CAPACITY, u);
      u = u_cap;
    }
    *d_n_total = n_query + u;
  }
}

// The same set from a candidate bitmap that the sampling launch already filled
// (orca_sample_topk_mark): only the cheap part is left for the single block -- clear the bits of the
// query nodes, count, scan, emit -- and the words are zeroed on the way so that the bitmap is clean
// for the next batch.
__device__ __forceinline__ int finish_from_bitmap(uint32_t *__restrict__ gbm, uint32_t *s_bitmap, int n_query,
                                                  int64_t n_nodes, int32_t *__restrict__ nodes_io,
                                                  double *__restrict__ ts_io, int u_cap,
                                                  int32_t *__restrict__ d_n_total, int32_t *status) {
  __shared__ int s_scan[FU_THREADS / 32];
  __shared__ double s_tmax[FU_THREADS / 32];
  __shared__ int s_total;
  const int n_words = (int)((n_nodes + 31) / 32);
  const bool staged = n_words <= FU_SMEM_WORDS;
  uint32_t *bm = staged ? s_bitmap : gbm;
  const int tid = threadIdx.x;
  if (staged) {
    // coalesced, unrolled copy of the bitmap into shared memory; the global words are zeroed on the
    // way so that the bitmap is clean for the next batch
    for (int w0 = tid; w0 < n_words; w0 += 8 * FU_THREADS) {
      uint32_t x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) x[u] = (w0 + u * FU_THREADS < n_words) ? __ldcg(&gbm[w0 + u * FU_THREADS]) : 0u;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int w = w0 + u * FU_THREADS;
        if (w < n_words) {
          s_bitmap[w] = x[u];
          if (x[u]) gbm[w] = 0u;
        }
      }
    }
    __syncthreads();
  }
  double tmax = -1.0e300;
  for (int i = tid; i < n_query; i += FU_THREADS) {
    tmax = fmax(tmax, ts_io[i]);
    const int v = nodes_io[i];
    if (v >= 0 && v < n_nodes) {
      const uint32_t bit = 1u << (v & 31);
      if (((volatile uint32_t *)bm)[v >> 5] & bit) atomicAnd(&bm[v >> 5], ~bit);   // test first: repeated query nodes
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
  if ((tid & 31) == 0) s_tmax[tid >> 5] = tmax;
  __threadfence_block();
  __syncthreads();
  tmax = s_tmax[0];
  for (int i = 1; i < FU_THREADS / 32; ++i) tmax = fmax(tmax, s_tmax[i]);
  // each thread owns a contiguous run of words (ascending order of the output)
  const int per = (n_words + FU_THREADS - 1) / FU_THREADS;
  const int w0 = tid * per, w1 = min(n_words, w0 + per);
  int cnt = 0;
  for (int w = w0; w < w1; ++w) cnt += __popc(bm[w]);
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += y;
  }
  if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    int v = s_scan[tid], inc2 = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, inc2, o);
      if (tid >= o) inc2 += y;
    }
    s_scan[tid] = inc2 - v;
    if (tid == 31) s_total = inc2;
  }
  __syncthreads();
  int rank = s_scan[tid >> 5] + incl - cnt;
  if (cnt > 0) {
    for (int w = w0; w < w1; ++w) {
      uint32_t bits = bm[w];
      if (bits == 0) continue;
      if (!staged) bm[w] = 0u;
      while (bits) {
        const int bit = __ffs(bits) - 1;
        bits &= bits - 1;
        if (rank >= 1 && rank - 1 < u_cap) {   // rank 0 is dropped (modules/embedding_module.py:212)
          nodes_io[n_query + rank - 1] = w * 32 + bit;
          ts_io[n_query + rank - 1] = tmax;
        }
        ++rank;
      }
    }
  }
  int u = s_total > 0 ? s_total - 1 : 0;
  if (u > u_cap) {
    if (tid == 0) report(status, ORCA_E_CAPACITY, u);
    u = u_cap;
  }
  if (tid == 0) *d_n_total = n_query + u;
  return u;
}

__global__ void __launch_bounds__(FU_THREADS)
find_uncached_marked_kernel(uint32_t *__restrict__ gbm, int n_query, int64_t n_nodes,
                            int32_t *__restrict__ nodes_io, double *__restrict__ ts_io, int u_cap,
                            int32_t *__restrict__ d_n_total, int32_t *status) {
  extern __shared__ uint32_t s_bitmap[];
  finish_from_bitmap(gbm, s_bitmap, n_query, n_nodes, nodes_io, ts_io, u_cap, d_n_total, status);
}

// The finish when the sampling launch also listed the candidates (batch_head_kernel).  A short list
// -- the usual case: most sampled neighbours are cached or in the batch -- is ranked directly: clear
// the bits of the batch's own nodes, keep the candidates whose bit survived, order them by counting
// (rank = number of smaller kept ids), drop rank 0, and clear their bits again, which leaves the bitmap
// clean without touching the rest of it.  A list that overflowed falls back to the bitmap scan.
__global__ void __launch_bounds__(FU_THREADS)
uncached_finish_kernel(uint32_t *__restrict__ gbm, int32_t *__restrict__ cand_count,
                       const int32_t *__restrict__ cand_list, int n_query, int64_t n_nodes,
                       int32_t *__restrict__ nodes_io, double *__restrict__ ts_io, int u_cap,
                       int32_t *__restrict__ d_n_total, int32_t *__restrict__ d_n_unc, int32_t *status,
                       const unsigned long long *__restrict__ last_pos, unsigned long long base) {
  extern __shared__ uint32_t s_bitmap[];
  __shared__ double s_tmax2[FU_THREADS / 32];
  __shared__ int s_kept;
  const int tid = threadIdx.x;
  dep_trigger();
  dep_wait();
  const int nc = *cand_count;
  if (nc > ORCA_CAND_CAP) {
    const int u = finish_from_bitmap(gbm, s_bitmap, n_query, n_nodes, nodes_io, ts_io, u_cap, d_n_total, status);
    if (tid == 0) {
      *d_n_unc = u;
      *cand_count = 0;
      if (status != nullptr) status[1] = n_query + u;
    }
    return;
  }
  int *s_c = reinterpret_cast<int *>(s_bitmap);   // ORCA_CAND_CAP kept ids (INT_MAX = dropped)
  if (nc == 0) {   // nothing sampled outside the cache and the batch
    if (tid == 0) {
      *d_n_total = n_query;
      *d_n_unc = 0;
      if (status != nullptr) status[1] = n_query;
    }
    return;
  }
  if (tid == 0) s_kept = 0;
  double tmax = -1.0e300;
  for (int i = tid; i < n_query; i += FU_THREADS) tmax = fmax(tmax, ts_io[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
  if ((tid & 31) == 0) s_tmax2[tid >> 5] = tmax;
  __syncthreads();
  tmax = s_tmax2[0];
  for (int i = 1; i < FU_THREADS / 32; ++i) tmax = fmax(tmax, s_tmax2[i]);
  for (int i = tid; i < nc; i += FU_THREADS) {
    const int c = cand_list[i];
    // a row of this batch carries a record of this batch's epoch (all records are in by now)
    const bool keep = __ldcg(&last_pos[c]) < base;
    atomicAnd(&gbm[c >> 5], ~(1u << (c & 31)));
    if (keep) atomicAdd(&s_kept, 1);
    s_c[i] = keep ? c : 0x7fffffff;
  }
  __syncthreads();
  for (int i = tid; i < nc; i += FU_THREADS) {
    const int c = s_c[i];
    if (c == 0x7fffffff) continue;
    int rank = 0;
    for (int j = 0; j < nc; ++j) rank += s_c[j] < c ? 1 : 0;
    if (rank >= 1 && rank - 1 < u_cap) {   // rank 0 is dropped (modules/embedding_module.py:212)
      nodes_io[n_query + rank - 1] = c;
      ts_io[n_query + rank - 1] = tmax;
    }
  }
  if (tid == 0) {
    int u = s_kept > 0 ? s_kept - 1 : 0;
    if (u > u_cap) {
      report(status, ORCA_E_CAPACITY, u);
      u = u_cap;
    }
    *d_n_total = n_query + u;
    *d_n_unc = u;
    *cand_count = 0;
    if (status != nullptr) status[1] = n_query + u;   // rows at layer 1 (status word layout, common.cuh)
  }
}


// ---------------------------------------------------------------------------------------------
// Last occurrence: pass 1 records, per id, the largest (epoch_base + position); pass 2 flags the
// positions that hold the record and, optionally, compacts them in position order.
// ---------------------------------------------------------------------------------------------
__global__ void last_pos_mark_kernel(const int32_t *__restrict__ ids, int n_cap, const int32_t *d_n,
                                     int64_t n_nodes, unsigned long long *__restrict__ last_pos,
                                     long long base) {
  const int n = rows_of(n_cap, d_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int v = ids[i];
    if (v >= 0 && v < n_nodes) atomicMax(&last_pos[v], (unsigned long long)(base + i));
  }
}

__global__ void last_pos_flag_kernel(const int32_t *__restrict__ ids, int n_cap, const int32_t *d_n,
                                     int64_t n_nodes, const unsigned long long *__restrict__ last_pos,
                                     long long base, uint8_t *__restrict__ is_last) {
  const int n = rows_of(n_cap, d_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_cap; i += gridDim.x * blockDim.x) {
    uint8_t f = 0;
    if (i < n) {
      const int v = ids[i];
      f = (v >= 0 && v < n_nodes && last_pos[v] == (unsigned long long)(base + i)) ? 1 : 0;
    }
    is_last[i] = f;
  }
}

// single CTA ordered compaction of the flagged positions
__global__ void __launch_bounds__(1024)
compact_flags_kernel(const uint8_t *__restrict__ is_last, int n_cap, const int32_t *d_n,
                     int32_t *__restrict__ compact, int32_t *__restrict__ n_compact) {
  __shared__ int s_scan[32];
  __shared__ int s_base;
  const int n = rows_of(n_cap, d_n);
  const int tid = threadIdx.x;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int start = 0; start < n; start += 1024) {
    const int i = start + tid;
    const int f = (i < n) ? is_last[i] : 0;
    int incl = f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, incl, o);
      if ((tid & 31) >= o) incl += y;
    }
    if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
      int v = s_scan[tid], inc2 = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, inc2, o);
        if (tid >= o) inc2 += y;
      }
      s_scan[tid] = inc2 - v;
    }
    __syncthreads();
    const int pos = s_base + s_scan[tid >> 5] + incl - f;
    if (f) compact[pos] = i;
    __syncthreads();
    if (tid == 1023) s_base = pos + f;
    __syncthreads();
  }
  if (tid == 0) *n_compact = s_base;
}

// Last occurrence of every id of a short list and the ordered list of those positions, in one block:
// record (atomicMax of epoch + position), then flag + scan + emit.
__global__ void __launch_bounds__(1024)
last_occ_compact_kernel(const int32_t *__restrict__ ids, int n, int64_t n_nodes,
                        unsigned long long *__restrict__ last_pos, long long base,
                        int32_t *__restrict__ compact, int32_t *__restrict__ n_compact, int32_t *status) {
  __shared__ int s_scan[32];
  __shared__ int s_base;
  const int tid = threadIdx.x;
  dep_trigger();
  dep_wait();
  if (tid == 0) s_base = 0;
  // four positions per thread and sweep, loaded up front so that their round trips overlap
  constexpr int U = 4;
  for (int i0 = 0; i0 < n; i0 += U * 1024) {
    int v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = i0 + u * 1024 + tid;
      v[u] = i < n ? ids[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (v[u] >= 0 && v[u] < n_nodes) atomicMax(&last_pos[v[u]], (unsigned long long)(base + i0 + u * 1024 + tid));
  }
  __threadfence();
  __syncthreads();
  for (int i0 = 0; i0 < n; i0 += U * 1024) {
    int f[U];
    {
      int v[U];
      unsigned long long rec[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * 1024 + tid;
        v[u] = i < n ? ids[i] : -1;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) rec[u] = (v[u] >= 0 && v[u] < n_nodes) ? __ldcg(&last_pos[v[u]]) : 0ull;
#pragma unroll
      for (int u = 0; u < U; ++u)
        f[u] = (v[u] >= 0 && v[u] < n_nodes && rec[u] == (unsigned long long)(base + i0 + u * 1024 + tid)) ? 1 : 0;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i0 + u * 1024 >= n) break;
      int incl = f[u];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += y;
      }
      if ((tid & 31) == 31) s_scan[tid >> 5] = incl;
      __syncthreads();
      if (tid < 32) {
        int x = s_scan[tid], inc2 = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int y = __shfl_up_sync(0xffffffffu, inc2, o);
          if (tid >= o) inc2 += y;
        }
        s_scan[tid] = inc2 - x;
      }
      __syncthreads();
      const int pos = s_base + s_scan[tid >> 5] + incl - f[u];
      if (f[u]) compact[pos] = i0 + u * 1024 + tid;
      __syncthreads();
      if (tid == 1023) s_base = pos + f[u];
      __syncthreads();
    }
  }
  if (tid == 0) {
    *n_compact = s_base;
    if (status != nullptr) status[2] = s_base;   // unique positives (status word layout, common.cuh)
  }
}

// ---- launchers of the fused batch kernels (used by the batch pipeline)
static int sm_count() {
  Ctx *c = cur();
  return c != nullptr ? c->sm_count : 148;
}

int launch_batch_head(const orca_tgn_t *m, const int32_t *d_batch, const double *d_bts, int b, int32_t *nodes1,
                      double *ts1, int32_t *cat_dst, int32_t *o_nbr, int32_t *o_eid, float *o_dt, int32_t *status,
                      int64_t *d_last_pos, long long base, cudaStream_t s) {
  const int k = m->k, n = 3 * b, threads = 256;
  int32_t *cand_count = reinterpret_cast<int32_t *>(m->cand_bitmap + (m->n_nodes + 31) / 32);
  int32_t *cand_list = cand_count + 1;
  unsigned long long *lp = reinterpret_cast<unsigned long long *>(d_last_pos);
  if (k <= 16) {
    const int grid = std::min(ceil_div(n, threads / 16), sm_count() * 16);
    ORCA_CUDA(launch_dep(batch_head_kernel<16>, grid, threads, 0, s, m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts,
                         m->n_nodes, d_batch, d_bts, b, k, nodes1, ts1, cat_dst, o_nbr, o_eid, o_dt, status,
                         m->cache_flag, m->cand_bitmap, cand_count, cand_list, lp, base));
  } else {
    const int grid = std::min(ceil_div(n, threads / 32), sm_count() * 16);
    ORCA_CUDA(launch_dep(batch_head_kernel<32>, grid, threads, 0, s, m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts,
                         m->n_nodes, d_batch, d_bts, b, k, nodes1, ts1, cat_dst, o_nbr, o_eid, o_dt, status,
                         m->cache_flag, m->cand_bitmap, cand_count, cand_list, lp, base));
  }
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int launch_uncached_finish(const orca_tgn_t *m, int n_query, int32_t *nodes_io, double *ts_io, int u_cap,
                           int32_t *d_n_total, int32_t *d_n_unc, int32_t *status, const int64_t *d_last_pos,
                           long long base, cudaStream_t s) {
  const int64_t words = (m->n_nodes + 31) / 32;
  ORCA_CHECK_ARG(words < (1ll << 31));
  size_t smem = std::max<size_t>(words <= FU_SMEM_WORDS ? (size_t)words * 4 : 0, (size_t)ORCA_CAND_CAP * 4);
  static thread_local int configured_device = -1;
  int dev = 0;
  ORCA_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    ORCA_CUDA(cudaFuncSetAttribute(uncached_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   FU_SMEM_WORDS * 4));
    configured_device = dev;
  }
  int32_t *cand_count = reinterpret_cast<int32_t *>(m->cand_bitmap + words);
  ORCA_CUDA(launch_dep(uncached_finish_kernel, 1, FU_THREADS, smem, s, m->cand_bitmap, cand_count, cand_count + 1,
                       n_query, m->n_nodes, nodes_io, ts_io, u_cap, d_n_total, d_n_unc, status,
                       reinterpret_cast<const unsigned long long *>(d_last_pos), (unsigned long long)base));
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int launch_last_occ_compact(const int32_t *d_ids, int n, int64_t n_nodes, int64_t *d_last_pos, long long base,
                            int32_t *d_compact, int32_t *d_n_compact, int32_t *d_status, cudaStream_t s) {
  ORCA_CUDA(launch_dep(last_occ_compact_kernel, 1, 1024, 0, s, d_ids, n, n_nodes,
                       reinterpret_cast<unsigned long long *>(d_last_pos), base, d_compact, d_n_compact, d_status));
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace orca

using namespace orca;

extern "C" {

const char *orca_last_error(void) { return orca::g_err; }
int orca_version(void) { return 1; }

int orca_csr_build_host(const int64_t *h_src, const int64_t *h_dst, const int64_t *h_eidx,
                        const double *h_ts, int64_t n_edges, int64_t n_nodes, int64_t *h_indptr,
                        int32_t *h_nbr, int32_t *h_eid, double *h_adj_ts) {
  ORCA_CHECK_ARG(h_src && h_dst && h_eidx && h_ts && h_indptr && h_nbr && h_eid && h_adj_ts);
  ORCA_CHECK_ARG(n_edges >= 0 && n_nodes > 0);
  std::fill(h_indptr, h_indptr + n_nodes + 1, (int64_t)0);
  for (int64_t i = 0; i < n_edges; ++i) {
    if (h_src[i] < 0 || h_src[i] >= n_nodes || h_dst[i] < 0 || h_dst[i] >= n_nodes)
      return set_error(ORCA_E_BOUNDS, "orca_csr_build_host: edge %lld has an endpoint outside [0,%lld)",
                       (long long)i, (long long)n_nodes);
    h_indptr[h_src[i] + 1]++;
    h_indptr[h_dst[i] + 1]++;
  }
  for (int64_t v = 0; v < n_nodes; ++v) h_indptr[v + 1] += h_indptr[v];
  std::vector<int64_t> cur(h_indptr, h_indptr + n_nodes);
  // counting pass in stream order keeps insertion order inside each node's list
  for (int64_t i = 0; i < n_edges; ++i) {
    int64_t p = cur[h_src[i]]++;
    h_nbr[p] = (int32_t)h_dst[i]; h_eid[p] = (int32_t)h_eidx[i]; h_adj_ts[p] = h_ts[i];
    p = cur[h_dst[i]]++;
    h_nbr[p] = (int32_t)h_src[i]; h_eid[p] = (int32_t)h_eidx[i]; h_adj_ts[p] = h_ts[i];
  }
  // stable sort by time of the lists that are not already sorted (streams usually are)
  std::vector<int64_t> perm;
  std::vector<int32_t> tn, te;
  std::vector<double> tt;
  for (int64_t v = 0; v < n_nodes; ++v) {
    const int64_t b = h_indptr[v], e = h_indptr[v + 1];
    if (std::is_sorted(h_adj_ts + b, h_adj_ts + e)) continue;
    const int64_t m = e - b;
    perm.resize(m);
    std::iota(perm.begin(), perm.end(), (int64_t)0);
    std::stable_sort(perm.begin(), perm.end(),
                     [&](int64_t x, int64_t y) { return h_adj_ts[b + x] < h_adj_ts[b + y]; });
    tn.assign(h_nbr + b, h_nbr + e); te.assign(h_eid + b, h_eid + e); tt.assign(h_adj_ts + b, h_adj_ts + e);
    for (int64_t i = 0; i < m; ++i) {
      h_nbr[b + i] = tn[perm[i]]; h_eid[b + i] = te[perm[i]]; h_adj_ts[b + i] = tt[perm[i]];
    }
  }
  return ORCA_OK;
}

static int orca_sample_topk_impl(const int64_t *d_indptr, const int32_t *d_adj_nbr, const int32_t *d_adj_eid,
                            const double *d_adj_ts, int64_t n_nodes, const int32_t *d_nodes,
                            const double *d_ts, int32_t n_query_cap, const int32_t *d_n_query, int32_t k,
                            int32_t *d_nbr, int32_t *d_eid, float *d_edge_times, float *d_delta,
                            int32_t *d_status, const uint8_t *d_cache_flag, uint32_t *d_cand_bitmap, void *stream) {
  ORCA_CHECK_ARG(d_indptr && d_adj_nbr && d_adj_eid && d_adj_ts && d_nodes && d_ts && d_nbr && d_eid);
  ORCA_CHECK_ARG(n_query_cap >= 0 && n_nodes > 0);
  ORCA_CHECK_ARG(k >= 1 && k <= ORCA_MAX_K);
  if (n_query_cap == 0) return ORCA_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  if (k <= 16) {
    const int per = threads / 16;
    // (a launch whose row count lives on the device usually covers far fewer rows than its capacity)
    const int grid = std::min(ceil_div(n_query_cap, per), d_n_query ? sm_count() * 2 : sm_count() * 16);
    ORCA_CUDA(launch_dep(sample_topk_kernel<16>, grid, threads, 0, s, d_indptr, d_adj_nbr, d_adj_eid, d_adj_ts, n_nodes,
                         d_nodes, d_ts, n_query_cap, d_n_query, k, d_nbr, d_eid, d_edge_times, d_delta, d_status,
                         d_cache_flag, d_cand_bitmap));
  } else {
    const int per = threads / 32;
    const int grid = std::min(ceil_div(n_query_cap, per), sm_count() * 16);
    ORCA_CUDA(launch_dep(sample_topk_kernel<32>, grid, threads, 0, s, d_indptr, d_adj_nbr, d_adj_eid, d_adj_ts, n_nodes,
                         d_nodes, d_ts, n_query_cap, d_n_query, k, d_nbr, d_eid, d_edge_times, d_delta, d_status,
                         d_cache_flag, d_cand_bitmap));
  }
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_sample_topk(const int64_t *d_indptr, const int32_t *d_adj_nbr, const int32_t *d_adj_eid,
                     const double *d_adj_ts, int64_t n_nodes, const int32_t *d_nodes,
                     const double *d_ts, int32_t n_query_cap, const int32_t *d_n_query, int32_t k,
                     int32_t *d_nbr, int32_t *d_eid, float *d_edge_times, float *d_delta,
                     int32_t *d_status, void *stream) {
  return orca_sample_topk_impl(d_indptr, d_adj_nbr, d_adj_eid, d_adj_ts, n_nodes, d_nodes, d_ts, n_query_cap,
                          d_n_query, k, d_nbr, d_eid, d_edge_times, d_delta, d_status, nullptr, nullptr, stream);
}

int orca_sample_topk_mark(const int64_t *d_indptr, const int32_t *d_adj_nbr, const int32_t *d_adj_eid,
                          const double *d_adj_ts, int64_t n_nodes, const int32_t *d_nodes,
                          const double *d_ts, int32_t n_query_cap, const int32_t *d_n_query, int32_t k,
                          int32_t *d_nbr, int32_t *d_eid, float *d_edge_times, float *d_delta,
                          int32_t *d_status, const uint8_t *d_cache_flag, uint32_t *d_cand_bitmap,
                          void *stream) {
  ORCA_CHECK_ARG(d_cache_flag && d_cand_bitmap);
  return orca_sample_topk_impl(d_indptr, d_adj_nbr, d_adj_eid, d_adj_ts, n_nodes, d_nodes, d_ts, n_query_cap,
                          d_n_query, k, d_nbr, d_eid, d_edge_times, d_delta, d_status, d_cache_flag,
                          d_cand_bitmap, stream);
}

int orca_find_before(const int64_t *d_indptr, const double *d_adj_ts, int64_t n_nodes,
                     const int32_t *d_nodes, const double *d_ts, int32_t n_query,
                     int32_t *d_count, void *stream) {
  ORCA_CHECK_ARG(d_indptr && d_adj_ts && d_nodes && d_ts && d_count && n_query >= 0);
  if (n_query == 0) return ORCA_OK;
  const int grid = std::min(ceil_div(n_query, 8), sm_count() * 8);
  find_before_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(d_indptr, d_adj_ts, n_nodes, d_nodes, d_ts,
                                                            n_query, d_count);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int64_t orca_find_uncached_scratch_bytes(int64_t n_nodes) {
  const int64_t words = (n_nodes + 31) / 32;
  return words <= FU_SMEM_WORDS ? 16 : words * 4;
}

int orca_find_uncached(const int32_t *d_nbr, int32_t n_query, int32_t k, const uint8_t *d_cache_flag,
                       int64_t n_nodes, int32_t *d_nodes_io, double *d_ts_io, int32_t u_cap,
                       int32_t *d_n_total, void *d_bitmap, int32_t *d_status, void *stream) {
  ORCA_CHECK_ARG(d_nbr && d_cache_flag && d_nodes_io && d_ts_io && d_n_total);
  ORCA_CHECK_ARG(n_query >= 0 && k >= 1 && k <= ORCA_MAX_K && u_cap >= 0 && n_nodes > 0);
  const int64_t words = (n_nodes + 31) / 32;
  ORCA_CHECK_ARG(words < (1ll << 31));
  size_t smem = 0;
  if (words <= FU_SMEM_WORDS) {
    smem = (size_t)words * 4;
    static thread_local int configured_device = -1;
    int dev = 0;
    ORCA_CUDA(cudaGetDevice(&dev));
    if (configured_device != dev) {
      ORCA_CUDA(cudaFuncSetAttribute(find_uncached_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     FU_SMEM_WORDS * 4));
      configured_device = dev;
    }
  } else {
    ORCA_CHECK_ARG(d_bitmap != nullptr);
  }
  find_uncached_kernel<<<1, FU_THREADS, smem, (cudaStream_t)stream>>>(
      d_nbr, n_query, k, d_cache_flag, n_nodes, d_nodes_io, d_ts_io, u_cap, d_n_total,
      (uint32_t *)d_bitmap, d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_find_uncached_marked(uint32_t *d_cand_bitmap, int32_t n_query, int64_t n_nodes, int32_t *d_nodes_io,
                              double *d_ts_io, int32_t u_cap, int32_t *d_n_total, int32_t *d_status,
                              void *stream) {
  ORCA_CHECK_ARG(d_cand_bitmap && d_nodes_io && d_ts_io && d_n_total);
  ORCA_CHECK_ARG(n_query >= 0 && u_cap >= 0 && n_nodes > 0 && (n_nodes + 31) / 32 < (1ll << 31));
  const int64_t words = (n_nodes + 31) / 32;
  size_t smem = 0;
  if (words <= FU_SMEM_WORDS) {
    smem = (size_t)words * 4;
    static thread_local int configured_device = -1;
    int dev = 0;
    ORCA_CUDA(cudaGetDevice(&dev));
    if (configured_device != dev) {
      ORCA_CUDA(cudaFuncSetAttribute(find_uncached_marked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     FU_SMEM_WORDS * 4));
      configured_device = dev;
    }
  }
  find_uncached_marked_kernel<<<1, FU_THREADS, smem, (cudaStream_t)stream>>>(d_cand_bitmap, n_query, n_nodes,
                                                                         d_nodes_io, d_ts_io, u_cap, d_n_total,
                                                                         d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_last_occurrence(const int32_t *d_ids, int32_t n_cap, const int32_t *d_n, int64_t n_nodes,
                         int64_t *d_last_pos, int64_t epoch_base, uint8_t *d_is_last,
                         int32_t *d_compact, int32_t *d_n_compact, void *stream) {
  ORCA_CHECK_ARG(d_ids && d_last_pos && d_is_last && n_cap >= 0 && n_nodes > 0 && epoch_base > 0);
  ORCA_CHECK_ARG((d_compact == nullptr) == (d_n_compact == nullptr));
  cudaStream_t s = (cudaStream_t)stream;
  if (n_cap == 0) {
    if (d_n_compact) ORCA_CUDA(cudaMemsetAsync(d_n_compact, 0, sizeof(int32_t), s));
    return ORCA_OK;
  }
  const int grid = std::min(ceil_div(n_cap, 256), sm_count() * 8);
  last_pos_mark_kernel<<<grid, 256, 0, s>>>(d_ids, n_cap, d_n, n_nodes, (unsigned long long *)d_last_pos,
                                            (long long)epoch_base);
  ORCA_COUNT_LAUNCH();
  last_pos_flag_kernel<<<grid, 256, 0, s>>>(d_ids, n_cap, d_n, n_nodes,
                                            (const unsigned long long *)d_last_pos, (long long)epoch_base,
                                            d_is_last);
  ORCA_COUNT_LAUNCH();
  if (d_compact) {
    compact_flags_kernel<<<1, 1024, 0, s>>>(d_is_last, n_cap, d_n, d_compact, d_n_compact);
    ORCA_COUNT_LAUNCH();
  }
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // extern "C"
