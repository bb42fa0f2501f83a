// Time-sorted adjacency built on the device (utils/util.py:91-105, get_neighbor_finder).
//
// Every edge i contributes two records: 2i under its source (neighbour = destination) and 2i + 1 under
// its destination.  The reference appends them in this order and then sorts each node's list by
// timestamp with Python's stable sort, so the wanted order of all records is (node, timestamp, record
// number).  That is a stable least-significant-digit radix sort of the record numbers, first by the
// eight bytes of the timestamp (mapped to an unsigned key of the same order), then by the bytes of the
// node id.  One pass = a per-block digit histogram, an exclusive scan of the (digit, block) counts, and a
// stable scatter.  Inside a block every warp owns a contiguous run of the tile and walks it 32 records
// at a time; lanes with the same digit find one another with match.any, so a record's rank among its
// digit is the warp's running count plus the number of lower lanes in its group.
#include "common.cuh"
#include "context.cuh"

namespace orca {
namespace csr {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int RUN = 2048;            // records per warp
constexpr int TILE = WARPS * RUN;    // records per block
constexpr int BINS = 256;

struct Edges {
  const int64_t *src, *dst;
  const double *ts;
  int64_t n_records;
};

// unsigned key with the order of the doubles (-0.0 and +0.0 equal)
__device__ __forceinline__ uint64_t time_key(double t) {
  const uint64_t u = (uint64_t)__double_as_longlong(t + 0.0);
  return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}

__device__ __forceinline__ int digit_of(const Edges &e, uint32_t rec, int pass) {
  const int64_t edge = rec >> 1;
  if (pass < 8) return (int)((time_key(e.ts[edge]) >> (8 * pass)) & 0xff);
  const int64_t node = (rec & 1) ? e.dst[edge] : e.src[edge];
  return (int)(((uint64_t)node >> (8 * (pass - 8))) & 0xff);
}

// Walks the warp's run; calls emit(index in the array, record, rank base from `count`, lower lanes of
// the same digit) and advances the warp's counts.
template <bool SCATTER>
__device__ __forceinline__ void walk_run(const Edges &e, const uint32_t *perm_in, uint32_t *perm_out, int pass,
                                         int64_t first, int32_t *count /* [BINS] of this warp */) {
  const int lane = threadIdx.x & 31;
  const uint32_t lower = (1u << lane) - 1u;
  for (int r = 0; r < RUN; r += 32) {
    const int64_t i = first + r + lane;
    const bool valid = i < e.n_records;
    uint32_t rec = 0;
    int digit = BINS + lane;  // lanes past the end group with nobody
    if (valid) {
      rec = perm_in ? perm_in[i] : (uint32_t)i;
      digit = digit_of(e, rec, pass);
    }
    const uint32_t group = __match_any_sync(0xffffffffu, digit);
    if (valid) {
      const int before = __popc(group & lower);
      if (SCATTER) perm_out[count[digit] + before] = rec;
    }
    __syncwarp();
    if (valid && (group & lower) == 0) count[digit] += __popc(group);
    __syncwarp();
  }
}

// counts[digit * n_blocks + block] = records of the block's tile with that digit
__global__ void __launch_bounds__(THREADS) digit_count_kernel(Edges e, const uint32_t *perm_in, int pass,
                                                              int32_t *counts, int n_blocks) {
  __shared__ int32_t count[WARPS][BINS];
  for (int i = threadIdx.x; i < WARPS * BINS; i += THREADS) (&count[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  walk_run<false>(e, perm_in, nullptr, pass, (int64_t)blockIdx.x * TILE + (int64_t)warp * RUN, count[warp]);
  __syncthreads();
  int total = 0;
  for (int w = 0; w < WARPS; ++w) total += count[w][threadIdx.x];
  counts[(int64_t)threadIdx.x * n_blocks + blockIdx.x] = total;
}

// offsets = exclusive scan of counts (after scan_kernel); stable scatter of the block's tile
__global__ void __launch_bounds__(THREADS) digit_scatter_kernel(Edges e, const uint32_t *perm_in, uint32_t *perm_out,
                                                                int pass, const int32_t *offsets, int n_blocks) {
  __shared__ int32_t count[WARPS][BINS];
  for (int i = threadIdx.x; i < WARPS * BINS; i += THREADS) (&count[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  const int64_t first = (int64_t)blockIdx.x * TILE + (int64_t)warp * RUN;
  walk_run<false>(e, perm_in, nullptr, pass, first, count[warp]);
  __syncthreads();
  int32_t at = offsets[(int64_t)threadIdx.x * n_blocks + blockIdx.x];
  for (int w = 0; w < WARPS; ++w) {
    const int32_t c = count[w][threadIdx.x];
    count[w][threadIdx.x] = at;
    at += c;
  }
  __syncthreads();
  walk_run<true>(e, perm_in, perm_out, pass, first, count[warp]);
}

// In-place exclusive scan by one block (the arrays here have at most a few million entries); `total`
// (may be null) receives the sum.  OUT = int32_t in place, or int64_t into a second array of n + 1.
template <typename OUT>
__global__ void __launch_bounds__(1024) scan_kernel(const int32_t *in, OUT *out, int64_t n, bool write_total) {
  __shared__ int64_t warp_sum[32];
  __shared__ int64_t carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < n; base += 4096) {
    const int64_t i = base + 4 * (int64_t)tid;
    int32_t v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = i + j < n ? in[i + j] : 0;
    const int64_t mine = (int64_t)v[0] + v[1] + v[2] + v[3];
    int64_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int64_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    int64_t before = carry_s;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    int64_t run = before + incl - mine;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i + j < n) out[i + j] = (OUT)run;
      run += v[j];
    }
    __syncthreads();
    if (tid == 1023) carry_s = run;
    __syncthreads();
  }
  if (write_total && tid == 0) out[n] = (OUT)carry_s;
}

__global__ void degree_kernel(Edges e, int64_t n_nodes, int32_t *degree, int32_t *status) {
  const int64_t n_edges = e.n_records / 2;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_edges; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = e.src[i], d = e.dst[i];
    if (s < 0 || s >= n_nodes || d < 0 || d >= n_nodes) {
      report(status, ORCA_E_BOUNDS, (int)(i < 0x7fffffff ? i : 0x7fffffff));
      continue;
    }
    atomicAdd(&degree[s], 1);
    atomicAdd(&degree[d], 1);
  }
}

__global__ void emit_kernel(Edges e, const int64_t *eidx, const uint32_t *perm, int32_t *nbr, int32_t *eid,
                            double *adj_ts) {
  for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < e.n_records; p += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t rec = perm[p];
    const int64_t edge = rec >> 1;
    nbr[p] = (int32_t)((rec & 1) ? e.src[edge] : e.dst[edge]);
    eid[p] = (int32_t)eidx[edge];
    adj_ts[p] = e.ts[edge];
  }
}

static int sm_count() {
  Ctx *c = cur();
  return c != nullptr ? c->sm_count : 148;
}

static int node_passes(int64_t n_nodes) {
  int p = 1;
  while (p < 8 && ((n_nodes - 1) >> (8 * p)) != 0) ++p;
  return p;
}

struct Layout {
  int64_t perm_a, perm_b, counts, degree, total;
  int n_blocks;
};
static Layout layout(int64_t n_edges, int64_t n_nodes) {
  Layout L;
  const int64_t n = 2 * n_edges;
  L.n_blocks = (int)((n + TILE - 1) / TILE);
  auto up = [](int64_t b) { return (b + 255) & ~255ll; };
  L.perm_a = 0;
  L.perm_b = L.perm_a + up(n * 4);
  L.counts = L.perm_b + up(n * 4);
  L.degree = L.counts + up((int64_t)BINS * L.n_blocks * 4);
  L.total = L.degree + up(n_nodes * 4);
  return L;
}

}  // namespace csr
}  // namespace orca

using namespace orca;

extern "C" int64_t orca_csr_build_workspace_bytes(int64_t n_edges, int64_t n_nodes) {
  if (n_edges < 0 || n_nodes <= 0) return -1;
  return csr::layout(n_edges, n_nodes).total;
}

extern "C" int orca_csr_build(const int64_t *d_src, const int64_t *d_dst, const int64_t *d_eidx, const double *d_ts,
                              int64_t n_edges, int64_t n_nodes, int64_t *d_indptr, int32_t *d_nbr, int32_t *d_eid,
                              double *d_adj_ts, int32_t *d_status, void *d_workspace, int64_t workspace_bytes,
                              void *stream) {
  ORCA_CHECK_ARG(d_indptr && d_status && d_workspace);
  ORCA_CHECK_ARG(n_edges >= 0 && n_nodes > 0 && n_nodes < (1ll << 31) && n_edges < (1ll << 30));
  ORCA_CHECK_ARG(n_edges == 0 || (d_src && d_dst && d_eidx && d_ts && d_nbr && d_eid && d_adj_ts));
  ORCA_CHECK_ARG(((uintptr_t)d_workspace & 255) == 0);
  const csr::Layout L = csr::layout(n_edges, n_nodes);
  if (workspace_bytes < L.total)
    return set_error(ORCA_E_CAPACITY, "orca_csr_build: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                     (long long)L.total);
  cudaStream_t s = (cudaStream_t)stream;
  char *base = (char *)d_workspace;
  uint32_t *perm[2] = {(uint32_t *)(base + L.perm_a), (uint32_t *)(base + L.perm_b)};
  int32_t *counts = (int32_t *)(base + L.counts);
  int32_t *degree = (int32_t *)(base + L.degree);
  csr::Edges e{d_src, d_dst, d_ts, 2 * n_edges};
  ORCA_CUDA(cudaMemsetAsync(degree, 0, n_nodes * sizeof(int32_t), s));
  if (n_edges > 0) {
    const int grid = (int)std::min<int64_t>((n_edges + 255) / 256, csr::sm_count() * 16);
    csr::degree_kernel<<<grid, 256, 0, s>>>(e, n_nodes, degree, d_status);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
  }
  csr::scan_kernel<int64_t><<<1, 1024, 0, s>>>(degree, d_indptr, n_nodes, true);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  if (n_edges == 0) return ORCA_OK;
  const int passes = 8 + csr::node_passes(n_nodes);
  const uint32_t *in = nullptr;  // the first pass reads the records in their own order
  int out = 0;
  for (int pass = 0; pass < passes; ++pass) {
    csr::digit_count_kernel<<<L.n_blocks, csr::THREADS, 0, s>>>(e, in, pass, counts, L.n_blocks);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
    csr::scan_kernel<int32_t><<<1, 1024, 0, s>>>(counts, counts, (int64_t)csr::BINS * L.n_blocks, false);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
    csr::digit_scatter_kernel<<<L.n_blocks, csr::THREADS, 0, s>>>(e, in, perm[out], pass, counts, L.n_blocks);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
    in = perm[out];
    out ^= 1;
  }
  const int grid = (int)std::min<int64_t>((2 * n_edges + 255) / 256, csr::sm_count() * 16);
  csr::emit_kernel<<<grid, 256, 0, s>>>(e, d_eidx, in, d_nbr, d_eid, d_adj_ts);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}
