// One eval batch of the temporal-embedding path, enqueued without host synchronisation:
// sample -> find uncached -> sample -> attention layer 1 (memory rows) -> history push / flags ->
// attention layer 2 (history rows) -> link scores -> raw messages -> GRU memory update.
//
// The budgeted two-layer batch is spread over four streams ("lanes") so that only what truly depends
// on the previous batch waits for it:
//   index lane   everything that reads nothing but the graph, the batch and the offline plan: row
//                list, top-level sampling, uncached set, sampling of the appended rows, the winners of
//                the raw messages, and then the cache flags of this batch's plan (their next reader is
//                the next batch's index work, which follows in this lane).  Runs a batch ahead.
//   layer-1 lane query projection, gather and output of layer 1 over the memory table (and the history
//                push in its epilogue).  Starts when the previous batch's memory update has landed.
//   side lane    raw messages and the GRU projection read the same pre-update memory as layer 1 and
//                run beside it; only the final scatter into the memory table waits for layer 1.
//   caller's stream  layer 2 over the history table and the link scores; runs beside the next
//                batch's layer 1.
// Index-side buffers and the layer-1 output exist twice (batch parity); a parity is reused only when
// the batch that used it has completed.  All four lanes collapse onto the caller's stream while tracing
// or when look-ahead is switched off.
//
// Several GPUs of one node share a batch (orca_tgn_eval_batch_sharded, one process per GPU, replicated
// tables): either every rank takes its share of the rows of both layers, or -- orca_tgn_t.layer1_ranks --
// the first ranks run the layer-1 and side lanes and the others the caller's-stream part, a batch apart.
// In both, the rows a rank computes reach the other ranks by peer stores from the epilogue of the kernel
// that computes them, followed by a flag; every wait on a flag is bounded.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "context.cuh"
#include "index_ops.cuh"
#include "tc_gemm.cuh"

namespace orca {

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

// index-side buffers of one batch (one set per batch parity)
struct IdxBuf {
  int32_t *nodes1; double *ts1; int32_t *n1; int32_t *n_unc;
  int32_t *nbr1, *eid1; float *dt1;            // layer-1 neighbour table (rows of this GPU)
  int32_t *nbr2, *eid2; float *dt2;            // top-level table when it is a table of its own
  int32_t *cat_dst; int32_t *win_pos; int32_t *n_win; int32_t *win_nodes;
  int32_t *loc_nodes; double *loc_ts; int32_t *n1_loc;               // sharded layer 1
  int32_t *feat_idx; int32_t *nbr2_loc, *eid2_loc; float *dt2_loc;  // sharded layer 2 / no-reuse index
  int32_t *order1, *order2;                    // rows of the two gather launches, heaviest first
};
// projection / gather buffers of one attention layer in flight (one set per compute lane)
struct LaneBuf {
  float *qt, *ctx, *hidden; uint8_t *valid;
};
struct Workspace {
  IdxBuf idx[2];
  LaneBuf lane[2];
  float *emb1[2];
  float *emb2;
  uint8_t *win1;
  float *gru_h;
  void *bitmap;
  size_t bytes;
};

static Workspace carve(void *base, int b_cap, int u_cap, int k, int64_t n_nodes) {
  Workspace w{};
  size_t off = 0;
  char *p = (char *)base;
  const size_t N = 3 * (size_t)b_cap, R1 = N + (size_t)u_cap;
  auto take = [&](size_t bytes) { void *r = p ? p + off : nullptr; off += align_up(bytes); return r; };
  for (int q = 0; q < 2; ++q) {
    IdxBuf &x = w.idx[q];
    x.nodes1 = (int32_t *)take(R1 * 4);   // (parity 0: first array of the workspace)
    x.ts1 = (double *)take(R1 * 8);
    x.n1 = (int32_t *)take(4);
    x.n_unc = (int32_t *)take(4);
    x.nbr1 = (int32_t *)take(R1 * k * 4);
    x.eid1 = (int32_t *)take(R1 * k * 4);
    x.dt1 = (float *)take(R1 * k * 4);
    x.nbr2 = (int32_t *)take(N * k * 4);
    x.eid2 = (int32_t *)take(N * k * 4);
    x.dt2 = (float *)take(N * k * 4);
    x.cat_dst = (int32_t *)take(2 * (size_t)b_cap * 4);
    x.win_pos = (int32_t *)take(2 * (size_t)b_cap * 4);
    x.n_win = (int32_t *)take(4);
    x.win_nodes = (int32_t *)take(2 * (size_t)b_cap * 4);
    x.loc_nodes = (int32_t *)take(R1 * 4);
    x.loc_ts = (double *)take(R1 * 8);
    x.n1_loc = (int32_t *)take(4);
    x.feat_idx = (int32_t *)take(N * 4);
    x.nbr2_loc = (int32_t *)take(N * k * 4);
    x.eid2_loc = (int32_t *)take(N * k * 4);
    x.dt2_loc = (float *)take(N * k * 4);
    x.order1 = (int32_t *)take(R1 * 4);
    x.order2 = (int32_t *)take(N * 4);
  }
  for (int q = 0; q < 2; ++q) {
    const size_t rows = q == 0 ? R1 : N;   // lane 0: layer 1 (and the one-lane modes), lane 1: layer 2
    w.lane[q].qt = (float *)take(rows * QT_LD * 4);
    w.lane[q].ctx = (float *)take(rows * QT * 4);
    w.lane[q].hidden = (float *)take(rows * D * 4);
    w.lane[q].valid = (uint8_t *)take(rows);
  }
  for (int q = 0; q < 2; ++q) w.emb1[q] = (float *)take(R1 * D * 4);
  w.emb2 = (float *)take(N * D * 4);
  w.win1 = (uint8_t *)take(R1);
  w.gru_h = (float *)take(2 * (size_t)b_cap * D * 4);
  w.bitmap = take((size_t)orca_find_uncached_scratch_bytes(n_nodes));
  w.bytes = off;
  return w;
}

// nodes1[0..3b) = [src|dst|neg], ts1[r] = ts[r % b], cat_dst = [dst|src]
__global__ void batch_prep_kernel(const int32_t *__restrict__ batch, const double *__restrict__ ts, int b,
                                  int32_t *__restrict__ nodes1, double *__restrict__ ts1,
                                  int32_t *__restrict__ cat_dst, int32_t *__restrict__ n1) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < 3 * b) {
    nodes1[i] = batch[i];
    ts1[i] = ts[i % b];
  }
  if (i < 2 * b) cat_dst[i] = i < b ? batch[b + i] : batch[i - b];
  if (i == 0) *n1 = 3 * b;
}

__global__ void set_flags_counted_kernel(uint8_t *__restrict__ flag, int64_t n_nodes,
                                         const int32_t *__restrict__ ids, int cap, const int32_t *d_n) {
  const int n = rows_of(cap, d_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int v = ids[i];
    if (v >= 0 && v < n_nodes) flag[v] = 1;
  }
}

// History.update_flag with a plan (modules/history.py:25-30): clear the flags of the plan that set them,
// set the flags of this plan, keep a copy of it for the next call.  One block: the clearing must be
// complete before the setting starts (an id may be in both plans).
__global__ void __launch_bounds__(1024)
plan_flags_kernel(uint8_t *__restrict__ flag, int64_t n_nodes, int32_t *__restrict__ prev_plan, int n_prev,
                  const int32_t *__restrict__ plan, int n_plan) {
  const int tid = threadIdx.x;
  // eight independent loads per thread in flight: the loop is a chain of L2 round trips otherwise
  for (int i0 = tid; i0 < n_prev; i0 += 8 * 1024) {
    int v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = i0 + u * 1024 < n_prev ? prev_plan[i0 + u * 1024] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (v[u] >= 0 && v[u] < n_nodes) flag[v[u]] = 0;
  }
  __threadfence();
  __syncthreads();
  for (int i0 = tid; i0 < n_plan; i0 += 8 * 1024) {
    int v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = i0 + u * 1024 < n_plan ? plan[i0 + u * 1024] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (v[u] >= 0 && v[u] < n_nodes) flag[v[u]] = 1;
      if (i0 + u * 1024 < n_plan) prev_plan[i0 + u * 1024] = v[u];
    }
  }
}

// ---- row sharding over `world` ranks: layer-1 row i -> rank i % world, slot i / world
__global__ void shard_l1_kernel(const int32_t *__restrict__ nodes1, const double *__restrict__ ts1,
                                const int32_t *__restrict__ n1, int rank, int world, int rpr,
                                int32_t *__restrict__ loc_nodes, double *__restrict__ loc_ts,
                                int32_t *__restrict__ n1_loc) {
  const int n = *n1;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j == 0) *n1_loc = n > rank ? (n - rank + world - 1) / world : 0;
  if (j >= rpr) return;
  const int i = rank + j * world;
  loc_nodes[j] = i < n ? nodes1[i] : 0;
  loc_ts[j] = i < n ? ts1[i] : 0.0;
}

// History.push of ALL layer-1 rows from the all-gathered buffer: row i sits at slot
// (i % world) * rpr + i / world.  Nothing is pushed once the batch has reported an error (a wait on the
// peers that gave up leaves the buffer incomplete: the replica stays as it was instead of diverging).
__global__ void push_gathered_kernel(float *__restrict__ table, const float *__restrict__ emb_all,
                                     const int32_t *__restrict__ ids, const unsigned long long *__restrict__ last_pos,
                                     long long base, int all_from, const int32_t *__restrict__ n1, int world,
                                     int rpr, const int32_t *__restrict__ status) {
  if (status != nullptr && *status != 0) return;
  const int n = *n1;
  const int t = threadIdx.x % 64;
  if (t >= D / 4) return;
  for (int i = blockIdx.x * 4 + threadIdx.x / 64; i < n; i += gridDim.x * 4) {
    // the last occurrence of an id wins; the appended rows are distinct and always win
    if (i < all_from && last_pos[ids[i]] != (unsigned long long)(base + i)) continue;
    const size_t slot = (size_t)(i % world) * rpr + i / world;
    reinterpret_cast<float4 *>(table + (size_t)ids[i] * D)[t] =
        reinterpret_cast<const float4 *>(emb_all + slot * D)[t];
  }
}

// top-layer rows of the local edges e = rank + j * world: local row p * b_loc + j <- batch row p * b + e
// (rows_world: the number of ranks the layer-1 rows are dealt out over, which fixes where a row sits in the
// gathered buffer)
__global__ void shard_l2_kernel(const int32_t *__restrict__ nbr2, const int32_t *__restrict__ eid2,
                                const float *__restrict__ dt2, int b, int k, int rank, int world, int rows_world,
                                int rpr, int b_loc, int32_t *__restrict__ feat_idx, int32_t *__restrict__ nbr_loc,
                                int32_t *__restrict__ eid_loc, float *__restrict__ dt_loc) {
  const int lr = blockIdx.x * blockDim.x / 32 + threadIdx.x / 32;   // one warp per local row
  const int lane = threadIdx.x % 32;
  if (lr >= 3 * b_loc) return;
  const int p = lr / b_loc, j = lr - p * b_loc;
  const int row = p * b + rank + j * world;
  if (lane == 0) feat_idx[lr] = (row % rows_world) * rpr + row / rows_world;
  if (lane < k) {
    nbr_loc[(size_t)lr * k + lane] = nbr2[(size_t)row * k + lane];
    eid_loc[(size_t)lr * k + lane] = eid2[(size_t)row * k + lane];
    dt_loc[(size_t)lr * k + lane] = dt2[(size_t)row * k + lane];
  }
}

// recursion without reuse: every top-level neighbour slot becomes a layer-1 row of its own, queried at
// the time of the row that sampled it; the top layer then gathers those rows by position
__global__ void expand_rows_kernel(const int32_t *__restrict__ nbr2, int n, int k, int32_t *__restrict__ nodes1,
                                   double *__restrict__ ts1, int32_t *__restrict__ idx2, int32_t *__restrict__ n1) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *n1 = n * (1 + k);
  if (i >= n * k) return;
  const int v = nbr2[i];
  nodes1[n + i] = v;
  ts1[n + i] = ts1[i / k];
  idx2[i] = v != 0 ? n + i : 0;
}

// ---- direct exchange of the layer-1 rows between the GPUs of a node (peer stores over NVLink)
struct Peers {
  float *rows[ORCA_MAX_WORLD];
  int32_t *flags[ORCA_MAX_WORLD];
};

// Every rank copies its live layer-1 rows into slot `rank` of every rank's exchange buffer (its own
// included), then -- once the last block's stores are fenced system-wide -- posts the batch sequence
// number in word `rank` of every rank's flag array.  flags[rank][ORCA_MAX_WORLD] of the own array counts
// the finished blocks.
__global__ void __launch_bounds__(256)
exchange_fanout_kernel(const float *__restrict__ src, const int32_t *__restrict__ n_loc, int rpr, Peers p,
                       int world, int rank, long long off, int seq) {
  dep_trigger();
  dep_wait();
  const int n = min(*n_loc, rpr);
  const long long total = (long long)n * (D / 4);
  const float4 *s4 = reinterpret_cast<const float4 *>(src);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = s4[i];
    for (int q = 0; q < world; ++q) reinterpret_cast<float4 *>(p.rows[q] + off)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t *counter = p.flags[rank] + ORCA_MAX_WORLD;
    const int prev = atomicAdd(counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      for (int q = 0; q < world; ++q)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flags[q] + rank), "r"(seq) : "memory");
    }
  }
}

// Waits (bounded: `limit` SM clocks) until every rank has posted `seq`; a rank that did not sets
// ORCA_E_TIMEOUT in the status word, and the kernels behind this one leave the tables alone.
__global__ void exchange_wait_kernel(const int32_t *__restrict__ flags, int world, int seq, int32_t *status,
                                     long long limit) {
  dep_trigger();
  dep_wait();
  const int q = threadIdx.x;
  if (q < world) {
    const long long t0 = clock64();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + q) : "memory");
      if (v >= seq) break;
      if (clock64() - t0 > limit) {
        report(status, ORCA_E_TIMEOUT, 500 + q);
        break;
      }
    }
  }
}

// Split by layer: a top-layer rank tells the layer-1 ranks that it has finished reading batch `seq` out of
// its exchange and memory-row buffers (word ORCA_FLAG_CONSUMED + rank of their flag arrays).
__global__ void post_consumed_kernel(Peers p, int first, int count, int rank, int seq) {
  dep_trigger();
  dep_wait();
  __threadfence_system();
  const int q = first + (int)threadIdx.x;
  if ((int)threadIdx.x < count)
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flags[q] + ORCA_FLAG_CONSUMED + rank), "r"(seq)
                 : "memory");
}

__global__ void publish_counts_kernel(const int32_t *n1, const int32_t *n_win, int32_t *status) {
  dep_wait();
  status[1] = *n1;
  status[2] = *n_win;
}

// ---- stream plumbing
// `to` waits for what `from` has been given so far (no-op when they are the same stream)
static int link(cudaStream_t from, cudaStream_t to, cudaEvent_t ev) {
  if (from == to) return ORCA_OK;
  ORCA_CUDA(cudaEventRecord(ev, from));
  ORCA_CUDA(cudaStreamWaitEvent(to, ev, 0));
  return ORCA_OK;
}
static int wait_on(cudaStream_t waiter, cudaStream_t recorded_on, cudaEvent_t ev) {
  if (waiter == recorded_on) return ORCA_OK;
  ORCA_CUDA(cudaStreamWaitEvent(waiter, ev, 0));
  return ORCA_OK;
}

}  // namespace orca

using namespace orca;

#define ORCA_TRY(call)        \
  do {                        \
    int rc_ = (call);         \
    if (rc_ != ORCA_OK) return rc_; \
  } while (0)

namespace orca {

static Ctx *ctx_of(const orca_tgn_t *m) {
  return m->ctx != nullptr ? reinterpret_cast<Ctx *>(m->ctx) : default_ctx();
}

// The one-layer model and the recursions without a cache budget: one stream, except for the raw-message /
// GRU chain, which may run on the side stream once layer 1 no longer reads the memory table.
static int eval_serial(const orca_tgn_t *m, Ctx *c, const int32_t *d_batch_i32, const double *d_batch_ts, int b,
                       int u_cap, Workspace &w, float *d_prob, float *d_emb_out, int32_t *d_status, cudaStream_t s) {
  const int k = m->k;
  const int mode = m->n_layers == 2 ? m->mode : ORCA_MODE_BUDGET;
  const int N = 3 * b, R1 = N + u_cap;
  IdxBuf &x = w.idx[0];
  LaneBuf &l = w.lane[0];
  Tracer &tr = c->trace;
  int32_t *tk = c->d_words + CTX_TICKET_MAIN;
  int64_t *lp_push = m->last_pos, *lp_msg = m->last_pos + 2 * m->n_nodes;
  c->last_parity = 0;
  // the batch arrays may have been made ready on another stream
  if (m->input_stream != nullptr) ORCA_TRY(link((cudaStream_t)m->input_stream, s, c->ev_in));

  ORCA_TRY(tr.mark(-1, s));
  batch_prep_kernel<<<ceil_div(N, 256), 256, 0, s>>>(d_batch_i32, d_batch_ts, b, x.nodes1, x.ts1, x.cat_dst, x.n1);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  ORCA_TRY(tr.mark(PH_PREP, s));

  float *emb_top = d_emb_out ? d_emb_out : w.emb2;
  bool forked = false;
  if (m->n_layers == 1) {
    ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, x.nodes1, x.ts1, N,
                              nullptr, k, x.nbr1, x.eid1, nullptr, x.dt1, d_status, s));
    ORCA_TRY(tr.mark(PH_SAMPLE_TOP, s));
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, x.nodes1, N, nullptr, l.qt, s));
    ORCA_TRY(tr.mark(PH_QUERY_L2, s));
    ORCA_TRY(launch_attn_gather(l.qt, m->mem.memory, m->edge_table, m->time_w, x.nbr1, x.eid1, x.dt1, k, N, nullptr,
                                0, nullptr, l.ctx, l.valid, tk, s));
    ORCA_TRY(tr.mark(PH_GATHER_L2, s));
    ORCA_TRY(orca_attn_output(&m->attn[0], l.ctx, l.valid, m->mem.memory, x.nodes1, N, nullptr, emb_top,
                              nullptr, nullptr, nullptr, l.hidden, s));
    ORCA_TRY(tr.mark(PH_OUTPUT_L2, s));
  } else {
    // top-level neighbour table; then the row list of layer 1 by recursion mode
    const int32_t *nbr1 = x.nbr1, *eid1 = x.eid1, *gather2 = x.nbr2;
    const float *dt1 = x.dt1;
    const float *table2 = m->hist_emb;
    const int32_t *d_n1 = x.n1;
    ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, x.nodes1, x.ts1, N,
                              nullptr, k, x.nbr2, x.eid2, nullptr, x.dt2, d_status, s));
    ORCA_TRY(tr.mark(PH_SAMPLE_TOP, s));
    if (mode == ORCA_MODE_NO_REUSE) {
      expand_rows_kernel<<<ceil_div(N * k, 256), 256, 0, s>>>(x.nbr2, N, k, x.nodes1, x.ts1, x.nbr2_loc, x.n1);
      ORCA_COUNT_LAUNCH();
      ORCA_LAUNCH_CHECK();
      gather2 = x.nbr2_loc;
      table2 = w.emb1[0];
    }
    ORCA_TRY(tr.mark(PH_UNCACHED, s));
    if (mode == ORCA_MODE_REUSE_ALL) {
      // layer 1 covers the batch rows only and shares the top-level neighbour table
      nbr1 = x.nbr2, eid1 = x.eid2, dt1 = x.dt2;
      d_n1 = nullptr;
    } else {
      ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, x.nodes1, x.ts1, R1,
                                x.n1, k, x.nbr1, x.eid1, nullptr, x.dt1, d_status, s));
    }
    ORCA_TRY(tr.mark(PH_SAMPLE_L1, s));
    const bool push1 = mode == ORCA_MODE_REUSE_ALL;
    if (push1) {
      ORCA_TRY(orca_last_occurrence(x.nodes1, R1, d_n1, m->n_nodes, lp_push, *m->epoch_base, w.win1, nullptr,
                                    nullptr, s));
      *m->epoch_base += R1;
    }
    ORCA_TRY(tr.mark(PH_LAST_OCC_L1, s));
    // layer 1 over memory rows; with unlimited reuse its output rows are pushed into the history table
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, x.nodes1, R1, d_n1, l.qt, s));
    ORCA_TRY(tr.mark(PH_QUERY_L1, s));
    ORCA_TRY(launch_attn_gather(l.qt, m->mem.memory, m->edge_table, m->time_w, nbr1, eid1, dt1, k, R1, d_n1,
                                mode == ORCA_MODE_NO_REUSE ? R1 : N, nullptr, l.ctx, l.valid, tk, s));
    ORCA_TRY(tr.mark(PH_GATHER_L1, s));
    ORCA_TRY(attn_output_impl(&m->attn[0], l.ctx, l.valid, m->mem.memory, x.nodes1, R1, d_n1, w.emb1[0],
                              push1 ? m->hist_emb : nullptr, push1 ? x.nodes1 : nullptr, push1 ? w.win1 : nullptr,
                              nullptr, 0, N, l.hidden, mode == ORCA_MODE_NO_REUSE ? R1 : N, s));
    ORCA_TRY(tr.mark(PH_OUTPUT_L1, s));
    if (c->overlap && !tr.on) {
      ORCA_TRY(link(s, c->aux, c->fork));
      forked = true;
    }
    ORCA_TRY(tr.mark(PH_FLAGS, s));
    // layer 2 over the history rows (or, without reuse, the fresh layer-1 rows) of the top-level neighbours
    ORCA_TRY(orca_attn_query(&m->attn[1], w.emb1[0], nullptr, N, nullptr, l.qt, s));
    ORCA_TRY(tr.mark(PH_QUERY_L2, s));
    ORCA_TRY(launch_attn_gather(l.qt, table2, m->edge_table, m->time_w, gather2, x.eid2, x.dt2, k, N, nullptr, 0,
                                nullptr, l.ctx, l.valid, tk, s));
    ORCA_TRY(tr.mark(PH_GATHER_L2, s));
    ORCA_TRY(orca_attn_output(&m->attn[1], l.ctx, l.valid, w.emb1[0], nullptr, N, nullptr, emb_top, nullptr,
                              nullptr, nullptr, l.hidden, s));
    ORCA_TRY(tr.mark(PH_OUTPUT_L2, s));
  }
  ORCA_TRY(orca_score(&m->score, emb_top, b, d_prob, s));
  ORCA_TRY(tr.mark(PH_SCORE, s));

  // raw messages of the batch (last occurrence per node in [src|dst]) and the memory update
  cudaStream_t ms = forked ? c->aux : s;
  ORCA_TRY(launch_last_occ_compact(d_batch_i32, 2 * b, m->n_nodes, lp_msg, *m->epoch_base, x.win_pos, x.n_win,
                                   d_status, ms));
  *m->epoch_base += 2 * b;
  ORCA_TRY(tr.mark(PH_LAST_OCC_MSG, s));
  ORCA_TRY(orca_message_store(&m->mem, m->edge_table, m->time_w, d_batch_i32, x.cat_dst, d_batch_ts,
                              d_batch_i32 + 3 * b, b, x.win_pos, 2 * b, x.n_win, x.win_nodes, ms));
  ORCA_TRY(tr.mark(PH_MESSAGE, s));
  ORCA_TRY(orca_gru_update(&m->gru, &m->mem, x.win_nodes, 2 * b, x.n_win, 1, w.gru_h, ms));
  ORCA_TRY(tr.mark(PH_GRU, s));
  if (forked) ORCA_TRY(link(c->aux, s, c->join));
  publish_counts_kernel<<<1, 1, 0, s>>>(x.n1, x.n_win, d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

// The budgeted two-layer batch over the lanes described at the top of the file, on one GPU (world == 1)
// or as one rank of the multi-GPU split.  phases: bit 0 = everything up to and including layer 1 (and,
// sharded, the delivery of its rows), bit 1 = the rest.
static int eval_budget(const orca_tgn_t *m, Ctx *c, int phases, const int32_t *d_batch_i32,
                       const double *d_batch_ts, int b, const int32_t *d_plan, int n_plan, int u_cap, Workspace &w,
                       float *d_emb1_local, const float *d_emb1_all, float *d_prob, float *d_emb_out,
                       int32_t *d_status, cudaStream_t s) {
  const int k = m->k, world = m->world > 1 ? m->world : 1, rank = world > 1 ? m->rank : 0;
  const bool sharded = world > 1;
  const int N = 3 * b, R1 = N + u_cap;
  // split by layer: ranks [0, wa) own the layer-1 rows and the memory update, ranks [wa, world) the top layer
  const bool staged = sharded && m->layer1_ranks > 0;
  const int wa = staged ? m->layer1_ranks : world, wb = staged ? world - m->layer1_ranks : world;
  const bool in_a = !staged || rank < wa, in_b = !staged || rank >= wa;
  const int rb = staged ? rank - wa : rank;
  const int rpr = ceil_div(R1, wa);
  const int b_loc = in_b ? (b - rb + wb - 1) / wb : 0;
  Tracer &tr = c->trace;
  const bool lanes = c->lookahead && c->overlap && !tr.on;
  cudaStream_t si = lanes ? c->idx : s;                       // index lane
  cudaStream_t sa = lanes ? c->lane1 : s;                     // layer-1 lane
  cudaStream_t sx = (c->overlap && !tr.on) ? c->aux : s;      // raw messages + GRU
  const bool direct = sharded && m->peer_rows[rank] != nullptr;   // rows exchanged by peer stores
  if (direct) {
    ORCA_CHECK_ARG(world <= ORCA_MAX_WORLD && m->exchange_seq != nullptr && m->peer_flags[rank] != nullptr);
    if ((int64_t)wa * rpr * D > m->exchange_cap)
      return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch_sharded: exchange buffer of %lld floats, %lld needed",
                       (long long)m->exchange_cap, (long long)wa * rpr * D);
  }
  if (staged) ORCA_CHECK_ARG(direct && wa < world && m->peer_gru[rank] != nullptr && projections_on_tensor_cores());

  const bool gru_split = direct && m->peer_gru[rank] != nullptr && projections_on_tensor_cores();
  if (gru_split && (int64_t)2 * b * D > m->gru_cap)
    return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch_sharded: memory-row buffer of %lld floats, %lld needed",
                     (long long)m->gru_cap, (long long)2 * b * D);
  if (phases & 1) {
    if (direct) c->xseq = ++*m->exchange_seq;   // sequence number of this batch in the ranks' flag words
    c->parity = (int)(c->seq++ & 1);
    c->base1 = *m->epoch_base;
    *m->epoch_base += R1;
    c->base_msg = *m->epoch_base;
    *m->epoch_base += 2 * b;
  }
  const int p = c->parity;
  c->last_parity = p;
  IdxBuf &x = w.idx[p];
  LaneBuf &l1 = w.lane[0], &l2 = w.lane[lanes ? 1 : 0];
  int64_t *lp_push = m->last_pos + (size_t)p * m->n_nodes, *lp_msg = m->last_pos + 2 * (size_t)m->n_nodes;
  const long long base1 = c->base1;
  float *emb1 = d_emb1_local != nullptr ? d_emb1_local : w.emb1[p];
  cudaStream_t s_in = m->input_stream != nullptr ? (cudaStream_t)m->input_stream : s;

  if (phases & 1) {
    ORCA_TRY(tr.mark(-1, s));
    ORCA_TRY(tr.mark(PH_PREP, s));
    // ------------------------------------------------------------------ index lane
    ORCA_CUDA(cudaEventRecord(c->ev_in, s_in));
    ORCA_TRY(wait_on(si, s_in, c->ev_in));
    if (lanes && c->done_recorded[p]) ORCA_CUDA(cudaStreamWaitEvent(si, c->ev_done[p], 0));
    // another batch size (a stream's short last batch) or workspace lays the buffers out differently: the
    // batch in flight must drain before this one touches them
    if (lanes && (c->layout_b != b || c->layout_u != u_cap || c->layout_k != k || c->layout_ws != w.idx[0].nodes1) &&
        c->done_recorded[p ^ 1])
      ORCA_CUDA(cudaStreamWaitEvent(si, c->ev_done[p ^ 1], 0));
    c->layout_b = b, c->layout_u = u_cap, c->layout_k = k, c->layout_ws = w.idx[0].nodes1;
    // One launch builds the row list of the batch and its neighbour table -- which is both the top-level
    // table and the layer-1 table of the same rows (same node, same query time) -- marks the uncached
    // candidates and records the last occurrence of every row's node.  The uncached out-of-batch
    // neighbours then join the row list and only those rows are sampled by a second launch.
    int32_t *top_nbr = sharded ? x.nbr2 : x.nbr1, *top_eid = sharded ? x.eid2 : x.eid1;
    float *top_dt = sharded ? x.dt2 : x.dt1;
    ORCA_TRY(launch_batch_head(m, d_batch_i32, d_batch_ts, b, x.nodes1, x.ts1, x.cat_dst, top_nbr, top_eid, top_dt,
                               d_status, lp_push, base1, si));
    ORCA_TRY(tr.mark(PH_SAMPLE_TOP, s));
    ORCA_TRY(launch_uncached_finish(m, N, x.nodes1, x.ts1, u_cap, x.n1, x.n_unc, d_status, lp_push, base1, si));
    ORCA_TRY(tr.mark(PH_UNCACHED, s));
    if (sharded) {
      // this rank's layer-1 rows, and the top-layer tables of its edges
      if (in_a) {
        shard_l1_kernel<<<ceil_div(rpr, 256), 256, 0, si>>>(x.nodes1, x.ts1, x.n1, rank, wa, rpr, x.loc_nodes,
                                                            x.loc_ts, x.n1_loc);
        ORCA_COUNT_LAUNCH();
        ORCA_LAUNCH_CHECK();
        ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, x.loc_nodes, x.loc_ts,
                                  rpr, x.n1_loc, k, x.nbr1, x.eid1, nullptr, x.dt1, d_status, si));
      }
      if (b_loc > 0) {
        shard_l2_kernel<<<ceil_div(3 * b_loc, 8), 256, 0, si>>>(x.nbr2, x.eid2, x.dt2, b, k, rb, wb, wa, rpr, b_loc,
                                                                x.feat_idx, x.nbr2_loc, x.eid2_loc, x.dt2_loc);
        ORCA_COUNT_LAUNCH();
        ORCA_LAUNCH_CHECK();
      }
    } else if (u_cap > 0) {
      ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, x.nodes1 + N, x.ts1 + N,
                                u_cap, x.n_unc, k, x.nbr1 + (size_t)N * k, x.eid1 + (size_t)N * k, nullptr,
                                x.dt1 + (size_t)N * k, d_status, si));
    }
    // the order in which the two gather launches hand out their rows (heaviest first)
    if (sharded)
      ORCA_TRY(launch_row_order(x.nbr1, in_a ? rpr : 0, x.n1_loc, x.order1, x.nbr2_loc, 3 * b_loc, nullptr, x.order2, k,
                                si));
    else
      ORCA_TRY(launch_row_order(x.nbr1, R1, x.n1, x.order1, x.nbr1, N, nullptr, x.order2, k, si));
    ORCA_TRY(tr.mark(PH_SAMPLE_L1, s));
    // winners of the raw messages: last occurrence per node in [src|dst] (model/tgn_model.py:172-176)
    ORCA_TRY(launch_last_occ_compact(d_batch_i32, 2 * b, m->n_nodes, lp_msg, c->base_msg, x.win_pos, x.n_win,
                                     d_status, si));
    ORCA_TRY(tr.mark(PH_LAST_OCC_MSG, s));
    if (si != s) ORCA_CUDA(cudaEventRecord(c->ev_idx[p], si));
    // cache flags of this batch (History.update_flag): read next by the next batch's head kernel
    if (d_plan != nullptr) {
      const int n_prev = *m->n_prev_plan >= 0 ? *m->n_prev_plan : 0;
      if (*m->n_prev_plan < 0) ORCA_CUDA(cudaMemsetAsync(m->cache_flag, 0, (size_t)m->n_nodes, si));
      plan_flags_kernel<<<1, 1024, 0, si>>>(m->cache_flag, m->n_nodes, m->prev_plan, n_prev, d_plan, n_plan);
      ORCA_COUNT_LAUNCH();
      ORCA_LAUNCH_CHECK();
      *m->n_prev_plan = n_plan;
    } else {
      // plan-less rule: the flags of the pushed ids are set and never cleared
      set_flags_counted_kernel<<<std::min(ceil_div(R1, 256), 1024), 256, 0, si>>>(m->cache_flag, m->n_nodes,
                                                                                  x.nodes1, R1, x.n1);
      ORCA_COUNT_LAUNCH();
      ORCA_LAUNCH_CHECK();
      *m->n_prev_plan = -1;
    }
    if (si != s) ORCA_CUDA(cudaEventRecord(c->ev_flags, si));
    ORCA_TRY(tr.mark(PH_FLAGS, s));

    // ------------------------------------------------------------------ side lane: raw messages, GRU projection
    // (reads the memory table as the previous batch's scatter -- the operation before it in this lane --
    // left it; replicated on every rank of the multi-GPU split)
    if (sx != si) {
      if (si != s) ORCA_CUDA(cudaStreamWaitEvent(sx, c->ev_idx[p], 0));
      else ORCA_TRY(link(s, sx, c->fork));
    }
    ORCA_TRY(orca_message_store(&m->mem, m->edge_table, m->time_w, d_batch_i32, x.cat_dst, d_batch_ts,
                                d_batch_i32 + 3 * b, b, x.win_pos, 2 * b, x.n_win, x.win_nodes, sx));
    ORCA_TRY(tr.mark(PH_MESSAGE, s));
    if (gru_split && !in_a) {
      // (split by layer: the layer-1 ranks compute the memory update; this rank only receives the rows)
    } else if (gru_split) {
      // the memory update is split by node: this rank computes every wa-th unique positive and stores the
      // new rows into every rank's buffer; the scatter (phase 2) waits for all computing ranks' rows
      if (staged) {
        // (the top-layer ranks run behind: their buffers of two batches ago must have been read)
        ORCA_CUDA(launch_dep(exchange_wait_kernel, 1, 32, 0, sx,
                             (const int32_t *)(m->peer_flags[rank] + ORCA_FLAG_CONSUMED + wa), wb, (int)c->xseq - 2,
                             d_status, c->wait_limit));
        ORCA_COUNT_LAUNCH();
      }
      tc::PeerOut po{};
      for (int q = 0; q < world; ++q) {
        ORCA_CHECK_ARG(m->peer_gru[q] != nullptr && m->peer_flags[q] != nullptr);
        po.rows[q] = m->peer_gru[q];
        po.flags[q] = m->peer_flags[q] + 16;
      }
      po.counter = m->peer_flags[rank] + 24;
      po.off = (c->xseq & 1) * m->gru_cap;
      po.world = world, po.rank = rank, po.seq = (int)c->xseq;
      ORCA_TRY(gru_project(&m->gru, &m->mem, x.win_nodes, 2 * b, x.n_win, w.gru_h, sx, &po, wa));
    } else {
      ORCA_TRY(gru_project(&m->gru, &m->mem, x.win_nodes, 2 * b, x.n_win, w.gru_h, sx));
    }
    ORCA_TRY(tr.mark(PH_GRU, s));

    // ------------------------------------------------------------------ layer-1 lane
    ORCA_TRY(wait_on(sa, si, c->ev_idx[p]));
    if (sa != sx && c->state_recorded) ORCA_CUDA(cudaStreamWaitEvent(sa, c->ev_state, 0));
    if (in_a) {
    const int32_t *rows1 = sharded ? x.loc_nodes : x.nodes1;
    const int32_t *d_n1 = sharded ? x.n1_loc : x.n1;
    const int cap1 = sharded ? rpr : R1;
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, rows1, cap1, d_n1, l1.qt, sa));
    ORCA_TRY(tr.mark(PH_QUERY_L1, s));
    ORCA_TRY(launch_attn_gather(l1.qt, m->mem.memory, m->edge_table, m->time_w, x.nbr1, x.eid1, x.dt1, k, cap1, d_n1,
                                sharded ? rpr : N, x.order1, l1.ctx, l1.valid, c->d_words + CTX_TICKET_MAIN, sa));
    ORCA_TRY(tr.mark(PH_GATHER_L1, s));
    if (!sharded) {
      // the push into the history table waits for the previous batch's top layer to have read it
      if (sa != s && c->g2_recorded) ORCA_CUDA(cudaStreamWaitEvent(sa, c->ev_g2, 0));
      // (winners of the push come from the records of the head kernel; the appended rows are distinct
      // out-of-batch nodes, so each of them wins)
      ORCA_TRY(attn_output_impl(&m->attn[0], l1.ctx, l1.valid, m->mem.memory, x.nodes1, R1, x.n1, emb1, m->hist_emb,
                                x.nodes1, w.win1, lp_push, base1, N, l1.hidden, N, sa));
    } else if (direct && projections_on_tensor_cores()) {
      // the LayerNorm epilogue of layer 1 delivers the rows itself: one kernel computes and exchanges
      const long long seq = c->xseq;
      tc::PeerOut po{};
      for (int q = 0; q < world; ++q) {
        ORCA_CHECK_ARG(m->peer_rows[q] != nullptr && m->peer_flags[q] != nullptr);
        po.rows[q] = m->peer_rows[q];
        po.flags[q] = m->peer_flags[q];
      }
      po.counter = m->peer_flags[rank] + ORCA_MAX_WORLD;
      po.off = (seq % ORCA_EXCHANGE_SLOTS) * m->exchange_cap + (long long)rank * rpr * D;
      po.world = world, po.rank = rank, po.seq = (int)seq;
      if (staged) {
        ORCA_CUDA(launch_dep(exchange_wait_kernel, 1, 32, 0, sa,
                             (const int32_t *)(m->peer_flags[rank] + ORCA_FLAG_CONSUMED + wa), wb, (int)seq - 2,
                             d_status, c->wait_limit));
        ORCA_COUNT_LAUNCH();
      }
      ORCA_TRY(attn_output_impl(&m->attn[0], l1.ctx, l1.valid, m->mem.memory, x.loc_nodes, rpr, x.n1_loc, emb1,
                                nullptr, nullptr, nullptr, nullptr, 0, 0, l1.hidden, 0, sa, &po));
    } else {
      ORCA_TRY(orca_attn_output(&m->attn[0], l1.ctx, l1.valid, m->mem.memory, x.loc_nodes, rpr, x.n1_loc, emb1,
                                nullptr, nullptr, nullptr, l1.hidden, sa));
      if (direct) {
        // (fp32 debug projections: a separate kernel fans the rows out)
        const long long seq = c->xseq;
        Peers pr{};
        for (int q = 0; q < world; ++q) {
          ORCA_CHECK_ARG(m->peer_rows[q] != nullptr && m->peer_flags[q] != nullptr);
          pr.rows[q] = m->peer_rows[q];
          pr.flags[q] = m->peer_flags[q];
        }
        const long long off = (seq % ORCA_EXCHANGE_SLOTS) * m->exchange_cap + (long long)rank * rpr * D;
        ORCA_CUDA(launch_dep(exchange_fanout_kernel, std::min(ceil_div(rpr * (D / 4), 256), c->sm_count), 256, 0, sa,
                             (const float *)emb1, (const int32_t *)x.n1_loc, rpr, pr, world, rank, off, (int)seq));
        ORCA_COUNT_LAUNCH();
      }
    }
    }   // in_a
    ORCA_TRY(tr.mark(PH_OUTPUT_L1, s));
    if (sa != s || sx != s) ORCA_CUDA(cudaEventRecord(c->ev_o1, sa));

    // ------------------------------------------------------------------ side lane: the memory table is written
    if (!gru_split) {
      ORCA_TRY(wait_on(sx, sa, c->ev_o1));
      ORCA_TRY(gru_scatter(&m->mem, x.win_nodes, 2 * b, x.n_win, 1, w.gru_h, sx));
      if (sx != s) {
        ORCA_CUDA(cudaEventRecord(c->ev_state, sx));
        c->state_recorded = true;
      }
    }
    // the caller's stream carries on after layer 1 (the caller may exchange the rows between the phases)
    ORCA_TRY(wait_on(s, sa, c->ev_o1));
  }

  if ((phases & 2) && gru_split) {
    // ------------------------------------------------------------------ side lane: all ranks' memory rows
    ORCA_TRY(wait_on(sx, sa, c->ev_o1));
    ORCA_CUDA(launch_dep(exchange_wait_kernel, 1, 32, 0, sx, (const int32_t *)(m->peer_flags[rank] + 16), wa,
                         (int)c->xseq, d_status, c->wait_limit));
    ORCA_COUNT_LAUNCH();
    ORCA_TRY(gru_scatter(&m->mem, x.win_nodes, 2 * b, x.n_win, 1, m->peer_gru[rank] + (c->xseq & 1) * m->gru_cap, sx,
                         d_status));
    if (sx != s) {
      ORCA_CUDA(cudaEventRecord(c->ev_state, sx));
      c->state_recorded = true;
    }
  }
  if (phases & 2) {
    // ------------------------------------------------------------------ caller's stream: layer 2 and the scores
    const float *feat2 = emb1;
    const int32_t *feat2_idx = nullptr;
    const int32_t *nbr2 = x.nbr1, *eid2 = x.eid1;
    const float *dt2 = x.dt1;
    int rows2 = N, b2 = b;
    if (sharded) {
      if (direct) {
        const long long seq = c->xseq;
        ORCA_CUDA(launch_dep(exchange_wait_kernel, 1, 32, 0, s, (const int32_t *)m->peer_flags[rank], wa, (int)seq,
                             d_status, c->wait_limit));
        ORCA_COUNT_LAUNCH();
        d_emb1_all = m->peer_rows[rank] + (seq % ORCA_EXCHANGE_SLOTS) * m->exchange_cap;
      }
      ORCA_CHECK_ARG(d_emb1_all != nullptr);
      // every replica of the history table receives every layer-1 row (winners by the head kernel's records)
      // (measured with the split by layer on 2 GPUs: moving this push to the layer-1 stream costs 9 us per
      // batch on the layer-1 rank, whose lane is the critical one; on the top-layer rank it gains nothing)
      push_gathered_kernel<<<std::min(ceil_div(R1, 4), c->sm_count * 8), 256, 0, s>>>(m->hist_emb, d_emb1_all, x.nodes1,
                                                           reinterpret_cast<const unsigned long long *>(lp_push),
                                                           base1, N, x.n1, wa, rpr, d_status);
      ORCA_COUNT_LAUNCH();
      ORCA_LAUNCH_CHECK();
      feat2 = d_emb1_all, feat2_idx = x.feat_idx;
      nbr2 = x.nbr2_loc, eid2 = x.eid2_loc, dt2 = x.dt2_loc;
      rows2 = 3 * b_loc, b2 = b_loc;
    }
    if (rows2 > 0) {
      ORCA_CHECK_ARG(d_prob != nullptr);
      float *emb_top = d_emb_out ? d_emb_out : w.emb2;
      ORCA_TRY(orca_attn_query(&m->attn[1], feat2, feat2_idx, rows2, nullptr, l2.qt, s));
      ORCA_TRY(tr.mark(PH_QUERY_L2, s));
      ORCA_TRY(launch_attn_gather(l2.qt, m->hist_emb, m->edge_table, m->time_w, nbr2, eid2, dt2, k, rows2, nullptr, 0,
                                  x.order2, l2.ctx, l2.valid, c->d_words + CTX_TICKET_SIDE, s));
      ORCA_TRY(tr.mark(PH_GATHER_L2, s));
      if (!sharded && sa != s) {
        ORCA_CUDA(cudaEventRecord(c->ev_g2, s));
        c->g2_recorded = true;
      }
      ORCA_TRY(orca_attn_output(&m->attn[1], l2.ctx, l2.valid, feat2, feat2_idx, rows2, nullptr, emb_top, nullptr,
                                nullptr, nullptr, l2.hidden, s));
      ORCA_TRY(tr.mark(PH_OUTPUT_L2, s));
      ORCA_TRY(orca_score(&m->score, emb_top, b2, d_prob, s));
      ORCA_TRY(tr.mark(PH_SCORE, s));
    }
    // the batch is complete on the caller's stream once the other lanes' parts of it are
    if (sx != s) ORCA_CUDA(cudaStreamWaitEvent(s, c->ev_state, 0));
    if (si != s) ORCA_CUDA(cudaStreamWaitEvent(s, c->ev_flags, 0));
    if (staged && !in_a) {
      Peers pr{};
      for (int q = 0; q < world; ++q) pr.flags[q] = m->peer_flags[q];
      ORCA_CUDA(launch_dep(post_consumed_kernel, 1, 32, 0, s, pr, 0, wa, rank, (int)c->xseq));
      ORCA_COUNT_LAUNCH();
    }
    if (lanes) {
      ORCA_CUDA(cudaEventRecord(c->ev_done[p], s));
      c->done_recorded[p] = true;
    }
  }
  return ORCA_OK;
}

}  // namespace orca

extern "C" {

int64_t orca_eval_workspace_bytes(int32_t b_cap, int32_t u_cap, int32_t k, int64_t n_nodes) {
  if (b_cap <= 0 || u_cap < 0 || k < 1 || k > ORCA_MAX_K || n_nodes <= 0) return -1;
  return (int64_t)carve(nullptr, b_cap, u_cap, k, n_nodes).bytes;
}

int64_t orca_eval_workspace_row_list(int32_t b_cap, int32_t u_cap, int32_t k, int64_t n_nodes, int32_t parity) {
  if (b_cap <= 0 || u_cap < 0 || k < 1 || k > ORCA_MAX_K || n_nodes <= 0 || parity < 0 || parity > 1) return -1;
  char base = 0;
  Workspace w = carve(&base, b_cap, u_cap, k, n_nodes);
  return (int64_t)((char *)w.idx[parity].nodes1 - &base);
}

int orca_tgn_eval_batch(const orca_tgn_t *m, const int32_t *d_batch_i32, const double *d_batch_ts,
                        int32_t b, const int32_t *d_plan, int32_t n_plan, int32_t u_cap,
                        void *d_workspace, int64_t workspace_bytes, float *d_prob,
                        float *d_emb_out, int32_t *d_status, void *stream) {
  ORCA_CHECK_ARG(m && d_batch_i32 && d_batch_ts && d_workspace && d_prob && d_status);
  ORCA_CHECK_ARG(b > 0 && u_cap >= 0 && n_plan >= 0);
  ORCA_CHECK_ARG(m->n_layers == 1 || m->n_layers == 2);
  ORCA_CHECK_ARG(m->k >= 1 && m->k <= ORCA_MAX_K);
  ORCA_CHECK_ARG(m->last_pos && m->epoch_base && *m->epoch_base > 0);
  if (m->n_layers == 2 && m->mode == ORCA_MODE_BUDGET) {
    ORCA_CHECK_ARG(m->hist_emb && m->cache_flag && m->n_prev_plan && (n_plan == 0 || m->prev_plan));
    ORCA_CHECK_ARG(n_plan <= m->plan_cap && m->cand_bitmap);
  }
  if (m->n_layers == 2 && m->mode == ORCA_MODE_REUSE_ALL) ORCA_CHECK_ARG(m->hist_emb != nullptr);
  const int k = m->k;
  const int mode = m->n_layers == 2 ? m->mode : ORCA_MODE_BUDGET;
  ORCA_CHECK_ARG(mode == ORCA_MODE_BUDGET || mode == ORCA_MODE_REUSE_ALL || mode == ORCA_MODE_NO_REUSE);
  if (m->n_layers == 1 || mode == ORCA_MODE_REUSE_ALL) u_cap = 0;
  if (m->n_layers == 2 && mode == ORCA_MODE_NO_REUSE) u_cap = 3 * b * k;
  Workspace w = carve(d_workspace, b, u_cap, k, m->n_nodes);
  if ((int64_t)w.bytes > workspace_bytes)
    return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch: workspace of %lld bytes, %lld needed",
                     (long long)workspace_bytes, (long long)w.bytes);
  Ctx *c = ctx_of(m);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_tgn_eval_batch: no context for the current device");
  CtxScope scope(c);
  int32_t *saved_status = c->status_word;
  c->status_word = d_status;
  launch_counter() = 0;
  int rc;
  if (m->n_layers == 2 && mode == ORCA_MODE_BUDGET) {
    orca_tgn_t one = *m;
    one.world = 1, one.rank = 0;
    rc = eval_budget(&one, c, 3, d_batch_i32, d_batch_ts, b, d_plan, n_plan, u_cap, w, nullptr, nullptr, d_prob,
                     d_emb_out, d_status, (cudaStream_t)stream);
  } else {
    rc = eval_serial(m, c, d_batch_i32, d_batch_ts, b, u_cap, w, d_prob, d_emb_out, d_status, (cudaStream_t)stream);
  }
  c->status_word = saved_status;
  c->last_batch_launches = launch_counter();
  return rc;
}

int orca_tgn_eval_batch_sharded(const orca_tgn_t *m, int32_t phase, const int32_t *d_batch_i32,
                                const double *d_batch_ts, int32_t b, const int32_t *d_plan, int32_t n_plan,
                                int32_t u_cap, void *d_workspace, int64_t workspace_bytes,
                                float *d_emb1_local, const float *d_emb1_all, float *d_prob_local,
                                float *d_emb2_local, int32_t *d_status, void *stream) {
  ORCA_CHECK_ARG(m && d_batch_i32 && d_batch_ts && d_workspace && d_status);
  ORCA_CHECK_ARG(phase == 0 || phase == 1 || phase == 2);
  ORCA_CHECK_ARG(b > 0 && u_cap >= 0 && n_plan >= 0 && m->n_layers == 2);
  ORCA_CHECK_ARG(m->world >= 2 && m->rank >= 0 && m->rank < m->world);
  ORCA_CHECK_ARG(m->k >= 1 && m->k <= ORCA_MAX_K && m->last_pos && m->epoch_base && *m->epoch_base > 0);
  ORCA_CHECK_ARG(m->hist_emb && m->cache_flag && m->n_prev_plan && (n_plan == 0 || m->prev_plan) && n_plan <= m->plan_cap && m->cand_bitmap);
  const bool direct = m->peer_rows[m->rank] != nullptr;
  ORCA_CHECK_ARG(phase != 0 || direct);                       // one call only when the library exchanges the rows
  ORCA_CHECK_ARG(phase == 2 || direct || d_emb1_local != nullptr);
  ORCA_CHECK_ARG(phase == 1 || d_prob_local != nullptr);
  Workspace w = carve(d_workspace, b, u_cap, m->k, m->n_nodes);
  if ((int64_t)w.bytes > workspace_bytes)
    return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch_sharded: workspace of %lld bytes, %lld needed",
                     (long long)workspace_bytes, (long long)w.bytes);
  Ctx *c = ctx_of(m);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_tgn_eval_batch_sharded: no context for the current device");
  CtxScope scope(c);
  int32_t *saved_status = c->status_word;
  c->status_word = d_status;
  if (phase != 2) launch_counter() = 0;
  const int rc = eval_budget(m, c, phase == 0 ? 3 : phase, d_batch_i32, d_batch_ts, b, d_plan, n_plan, u_cap, w,
                             d_emb1_local, d_emb1_all, d_prob_local, d_emb2_local, d_status, (cudaStream_t)stream);
  c->status_word = saved_status;
  if (phase != 1) c->last_batch_launches = launch_counter();
  return rc;
}

int orca_tgn_eval_epoch(const orca_tgn_t *m, const orca_epoch_t *e, int32_t u_cap, void *d_workspace,
                        int64_t workspace_bytes, void *d_stage, int64_t stage_bytes, float *d_prob, float *h_prob,
                        int32_t *d_status, void *stream) {
  ORCA_CHECK_ARG(m && e && d_workspace && d_stage && d_prob && d_status);
  ORCA_CHECK_ARG(e->n_batches >= 0 && (e->n_batches == 0 || (e->h_i32 && e->h_ts && e->off_i32 && e->off_ts && e->b &&
                                                             e->n_plan && e->off_prob)));
  Ctx *c = ctx_of(m);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_tgn_eval_epoch: no context for the current device");
  const bool sharded = m->world > 1;
  if (sharded && m->peer_rows[m->rank] == nullptr)
    return set_error(ORCA_E_UNSUPPORTED, "orca_tgn_eval_epoch: the multi-GPU split needs the direct exchange");
  cudaStream_t s = (cudaStream_t)stream;
  constexpr int kSlots = Ctx::kStageSlots;
  const int64_t slot_bytes = (stage_bytes / kSlots) & ~(int64_t)255;
  orca_tgn_t mm = *m;
  mm.input_stream = c->copy;
  for (int64_t i = 0; i < e->n_batches; ++i) {
    const int b = e->b[i], n_plan = e->n_plan[i];
    ORCA_CHECK_ARG(b > 0);
    const int64_t bytes_i32 = ((int64_t)4 * b + (n_plan > 0 ? n_plan : 0)) * 4;
    const int64_t off_ts = (bytes_i32 + 15) & ~(int64_t)15;
    if (off_ts + 8ll * b > slot_bytes)
      return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_epoch: staging slot of %lld bytes, batch %lld needs %lld",
                       (long long)slot_bytes, (long long)i, (long long)(off_ts + 8ll * b));
    const int slot = (int)(c->stage_seq++ % kSlots);   // (the ring carries over from call to call)
    char *d_slot = (char *)d_stage + slot * slot_bytes;
    // the copy of batch i runs on the copy stream, ahead of the kernels of the batches before it; a slot is
    // refilled once the batch that read it has completed
    if (c->slot_used[slot]) ORCA_CUDA(cudaStreamWaitEvent(c->copy, c->ev_slot[slot], 0));
    ORCA_CUDA(cudaMemcpyAsync(d_slot, e->h_i32 + e->off_i32[i], (size_t)bytes_i32, cudaMemcpyHostToDevice, c->copy));
    ORCA_CUDA(cudaMemcpyAsync(d_slot + off_ts, e->h_ts + e->off_ts[i], (size_t)8 * b, cudaMemcpyHostToDevice, c->copy));
    const int32_t *d_i32 = reinterpret_cast<const int32_t *>(d_slot);
    const double *d_ts = reinterpret_cast<const double *>(d_slot + off_ts);
    const int32_t *d_plan = n_plan >= 0 ? d_i32 + 4 * (size_t)b : nullptr;
    float *prob = d_prob + e->off_prob[i];
    int n_scores;
    if (sharded) {
      ORCA_TRY(orca_tgn_eval_batch_sharded(&mm, 0, d_i32, d_ts, b, d_plan, n_plan > 0 ? n_plan : 0, u_cap, d_workspace,
                                           workspace_bytes, nullptr, nullptr, prob, nullptr, d_status, stream));
      // (split by layer: only the top-layer ranks hold scores)
      const int wa = m->layer1_ranks > 0 ? m->layer1_ranks : 0;
      const int wb = m->world - wa, rb = m->rank - wa;
      n_scores = rb < 0 ? 0 : 2 * ((b - rb + wb - 1) / wb);
    } else {
      ORCA_TRY(orca_tgn_eval_batch(&mm, d_i32, d_ts, b, d_plan, n_plan > 0 ? n_plan : 0, u_cap, d_workspace,
                                   workspace_bytes, prob, nullptr, d_status, stream));
      n_scores = 2 * b;
    }
    if (h_prob != nullptr && n_scores > 0)
      ORCA_CUDA(cudaMemcpyAsync(h_prob + e->off_prob[i], prob, (size_t)n_scores * 4, cudaMemcpyDeviceToHost, s));
    ORCA_CUDA(cudaEventRecord(c->ev_slot[slot], s));
    c->slot_used[slot] = true;
  }
  return ORCA_OK;
}

int orca_ipc_export(const void *d_ptr, void *h_handle, int64_t *h_offset) {
  ORCA_CHECK_ARG(d_ptr && h_handle && h_offset);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaPointerAttributes attr;
  ORCA_CUDA(cudaPointerGetAttributes(&attr, d_ptr));
  ORCA_CHECK_ARG(attr.type == cudaMemoryTypeDevice);
  // d_ptr may sit inside a pooled allocation: the handle names the allocation, the offset finds the buffer.
  // The range query lives in the driver API; the runtime hands out its entry point.
  typedef int (*range_fn)(unsigned long long *, size_t *, unsigned long long);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qr;
  ORCA_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr));
  ORCA_CHECK_ARG(fn != nullptr);
  unsigned long long base = 0;
  size_t size = 0;
  if (((range_fn)fn)(&base, &size, (unsigned long long)(uintptr_t)d_ptr) != 0)
    return set_error(ORCA_E_CUDA, "orca_ipc_export: address range query failed");
  cudaIpcMemHandle_t h;
  ORCA_CUDA(cudaIpcGetMemHandle(&h, (void *)(uintptr_t)base));
  memcpy(h_handle, &h, sizeof(h));
  *h_offset = (int64_t)((unsigned long long)(uintptr_t)d_ptr - base);
  return ORCA_OK;
}

int orca_ipc_open(const void *h_handle, int64_t offset, void **h_ptr_out) {
  ORCA_CHECK_ARG(h_handle && h_ptr_out && offset >= 0);
  cudaIpcMemHandle_t h;
  memcpy(&h, h_handle, sizeof(h));
  void *base = nullptr;
  // opened from the calling process's current device: peer access to the owner is enabled on the way
  ORCA_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *h_ptr_out = (char *)base + offset;
  return ORCA_OK;
}

int orca_ipc_close(void *h_ptr, int64_t offset) {
  ORCA_CHECK_ARG(h_ptr && offset >= 0);
  ORCA_CUDA(cudaIpcCloseMemHandle((char *)h_ptr - offset));
  return ORCA_OK;
}

int orca_stage_h2d(void *d_dst, const void *h_src, int64_t bytes, void *stream) {
  ORCA_CHECK_ARG(d_dst && h_src && bytes >= 0);
  if (bytes == 0) return ORCA_OK;
  ORCA_CUDA(cudaMemcpyAsync(d_dst, h_src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return ORCA_OK;
}

int orca_read_status(orca_ctx_t *ctx, int32_t *d_status, int32_t *h_counts, void *stream) {
  ORCA_CHECK_ARG(d_status);
  Ctx *c = ctx != nullptr ? reinterpret_cast<Ctx *>(ctx) : default_ctx();
  int32_t h[4] = {0, 0, 0, 0};
  cudaStream_t s = (cudaStream_t)stream;
  ORCA_CUDA(cudaMemcpyAsync(h, d_status, sizeof(h), cudaMemcpyDeviceToHost, s));
  ORCA_CUDA(cudaStreamSynchronize(s));
  if (h_counts) {
    h_counts[0] = h[0];
    h_counts[1] = h[1];
    h_counts[2] = h[2];
    h_counts[3] = c != nullptr ? c->last_batch_launches : 0;
  }
  if (h[0] != 0) {
    ORCA_CUDA(cudaMemsetAsync(d_status, 0, sizeof(h), s));
    return set_error(h[0], "device status %d (detail %d)", h[0], h[3]);
  }
  return ORCA_OK;
}

}  // extern "C"
