// One eval batch of the budgeted-reuse path, enqueued on a stream without host synchronisation:
// sample -> find uncached -> sample -> attention layer 1 (memory rows) -> history push / flags ->
// attention layer 2 (history rows) -> link scores -> raw messages -> GRU memory update.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "index_ops.cuh"
#include "tc_gemm.cuh"

namespace orca {

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct Workspace {
  int32_t *nodes1; double *ts1; int32_t *n1; int32_t *n_unc;
  int32_t *nbr2, *eid2; float *dt2;
  int32_t *nbr1, *eid1; float *dt1;
  uint8_t *win1, *valid;
  float *qt, *ctx, *emb1, *emb2;
  int32_t *cat_dst; uint8_t *is_last2; int32_t *win_pos; int32_t *n_win; int32_t *win_nodes;
  float *gru_h;
  float *hidden;
  int32_t *loc_nodes; double *loc_ts; int32_t *n1_loc;      // sharded layer 1
  int32_t *feat_idx; int32_t *nbr2_loc, *eid2_loc; float *dt2_loc;  // sharded layer 2
  void *bitmap;
  size_t bytes;
};

static Workspace carve(void *base, int b_cap, int u_cap, int k, int64_t n_nodes) {
  Workspace w{};
  size_t off = 0;
  char *p = (char *)base;
  const size_t N = 3 * (size_t)b_cap, R1 = N + (size_t)u_cap;
  auto take = [&](size_t bytes) { void *r = p ? p + off : nullptr; off += align_up(bytes); return r; };
  w.nodes1 = (int32_t *)take(R1 * 4);
  w.ts1 = (double *)take(R1 * 8);
  w.n1 = (int32_t *)take(4);
  w.n_unc = (int32_t *)take(4);
  w.nbr2 = (int32_t *)take(N * k * 4);
  w.eid2 = (int32_t *)take(N * k * 4);
  w.dt2 = (float *)take(N * k * 4);
  w.nbr1 = (int32_t *)take(R1 * k * 4);
  w.eid1 = (int32_t *)take(R1 * k * 4);
  w.dt1 = (float *)take(R1 * k * 4);
  w.win1 = (uint8_t *)take(R1);
  w.valid = (uint8_t *)take(R1);
  w.qt = (float *)take(R1 * QT_LD * 4);
  w.ctx = (float *)take(R1 * QT * 4);
  w.emb1 = (float *)take(R1 * D * 4);
  w.emb2 = (float *)take(N * D * 4);
  w.cat_dst = (int32_t *)take(2 * (size_t)b_cap * 4);
  w.is_last2 = (uint8_t *)take(2 * (size_t)b_cap);
  w.win_pos = (int32_t *)take(2 * (size_t)b_cap * 4);
  w.n_win = (int32_t *)take(4);
  w.win_nodes = (int32_t *)take(2 * (size_t)b_cap * 4);
  w.gru_h = (float *)take(2 * (size_t)b_cap * D * 4);
  w.hidden = (float *)take(R1 * D * 4);
  w.loc_nodes = (int32_t *)take(R1 * 4);
  w.loc_ts = (double *)take(R1 * 8);
  w.n1_loc = (int32_t *)take(4);
  w.feat_idx = (int32_t *)take(N * 4);
  w.nbr2_loc = (int32_t *)take(N * k * 4);
  w.eid2_loc = (int32_t *)take(N * k * 4);
  w.dt2_loc = (float *)take(N * k * 4);
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
// (i % world) * rpr + i / world
__global__ void push_gathered_kernel(float *__restrict__ table, const float *__restrict__ emb_all,
                                     const int32_t *__restrict__ ids, const unsigned long long *__restrict__ last_pos,
                                     long long base, int all_from, const int32_t *__restrict__ n1, int world,
                                     int rpr) {
  const int n = *n1;
  const int i = blockIdx.x * 4 + threadIdx.x / 64;
  const int t = threadIdx.x % 64;
  if (i >= n || t >= D / 4) return;
  // the last occurrence of an id wins; the appended rows are distinct and always win
  if (i < all_from && last_pos[ids[i]] != (unsigned long long)(base + i)) return;
  const size_t slot = (size_t)(i % world) * rpr + i / world;
  reinterpret_cast<float4 *>(table + (size_t)ids[i] * D)[t] =
      reinterpret_cast<const float4 *>(emb_all + slot * D)[t];
}

// top-layer rows of the local edges e = rank + j * world: local row p * b_loc + j <- batch row p * b + e
__global__ void shard_l2_kernel(const int32_t *__restrict__ nbr2, const int32_t *__restrict__ eid2,
                                const float *__restrict__ dt2, int b, int k, int rank, int world, int rpr,
                                int b_loc, int32_t *__restrict__ feat_idx, int32_t *__restrict__ nbr_loc,
                                int32_t *__restrict__ eid_loc, float *__restrict__ dt_loc) {
  const int lr = blockIdx.x * blockDim.x / 32 + threadIdx.x / 32;   // one warp per local row
  const int lane = threadIdx.x % 32;
  if (lr >= 3 * b_loc) return;
  const int p = lr / b_loc, j = lr - p * b_loc;
  const int row = p * b + rank + j * world;
  if (lane == 0) feat_idx[lr] = (row % world) * rpr + row / world;
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

// Waits (bounded: about a second of SM clocks) until every rank has posted `seq`; a rank that did not
// sets ORCA_E_TIMEOUT in the status word and the batch goes on with whatever the buffer holds.
__global__ void exchange_wait_kernel(const int32_t *__restrict__ flags, int world, int seq, int32_t *status) {
  dep_trigger();
  dep_wait();
  const int q = threadIdx.x;
  if (q < world) {
    const long long t0 = clock64();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + q) : "memory");
      if (v >= seq) break;
      if (clock64() - t0 > 2000000000ll) {
        report(status, ORCA_E_TIMEOUT, 500 + q);
        break;
      }
    }
  }
}

__global__ void publish_counts_kernel(const int32_t *n1, const int32_t *n_win, int32_t *status) {
  dep_wait();
  status[1] = *n1;
  status[2] = *n_win;
}

static thread_local int g_last_batch_launches = 0;

// Optional per-phase timing of the eval batch: CUDA events at the phase boundaries, summed per phase.
enum Phase { PH_PREP, PH_SAMPLE_TOP, PH_UNCACHED, PH_SAMPLE_L1, PH_LAST_OCC_L1, PH_QUERY_L1, PH_GATHER_L1,
             PH_OUTPUT_L1, PH_FLAGS, PH_QUERY_L2, PH_GATHER_L2, PH_OUTPUT_L2, PH_SCORE, PH_LAST_OCC_MSG,
             PH_MESSAGE, PH_GRU, PH_COUNT };
static const char *kPhaseNames[PH_COUNT] = {"prep", "sample_top", "find_uncached", "sample_l1", "last_occurrence_l1",
                                            "attn_query_l1", "attn_gather_l1", "attn_output_l1", "set_flags",
                                            "attn_query_l2", "attn_gather_l2", "attn_output_l2", "score",
                                            "last_occurrence_msg", "message_store", "gru_update"};
struct Tracer {
  bool on = false;
  std::vector<cudaEvent_t> ev;        // PH_COUNT + 1 events per traced batch
  std::vector<int> phase_of;          // phase that ENDS at event i (or -1 for a batch's first event)
  size_t used = 0;
  int mark(int phase, cudaStream_t s) {
    if (!on) return ORCA_OK;
    if (used == ev.size()) {
      cudaEvent_t e;
      ORCA_CUDA(cudaEventCreate(&e));
      ev.push_back(e);
      phase_of.push_back(-1);
    }
    phase_of[used] = phase;
    ORCA_CUDA(cudaEventRecord(ev[used++], s));
    return ORCA_OK;
  }
};
static Tracer g_trace;

// The raw-message / GRU chain of a batch only needs the memory table to be no longer read by the
// batch's attention layers, so it runs on a second stream next to the top attention layer and the
// scorer.  One auxiliary stream and two events per device, created on first use.
struct Overlap {
  bool enabled = true;
  int device = -1;
  cudaStream_t aux = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  int ensure() {
    int dev = 0;
    ORCA_CUDA(cudaGetDevice(&dev));
    if (dev == device && aux != nullptr) return ORCA_OK;
    ORCA_CUDA(cudaStreamCreateWithFlags(&aux, cudaStreamNonBlocking));
    ORCA_CUDA(cudaEventCreateWithFlags(&fork, cudaEventDisableTiming));
    ORCA_CUDA(cudaEventCreateWithFlags(&join, cudaEventDisableTiming));
    device = dev;
    return ORCA_OK;
  }
};
static Overlap g_overlap;

}  // namespace orca

using namespace orca;

#define ORCA_TRY(call)        \
  do {                        \
    int rc_ = (call);         \
    if (rc_ != ORCA_OK) return rc_; \
  } while (0)

extern "C" {

int64_t orca_eval_workspace_bytes(int32_t b_cap, int32_t u_cap, int32_t k, int64_t n_nodes) {
  if (b_cap <= 0 || u_cap < 0 || k < 1 || k > ORCA_MAX_K || n_nodes <= 0) return -1;
  return (int64_t)carve(nullptr, b_cap, u_cap, k, n_nodes).bytes;
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
  cudaStream_t s = (cudaStream_t)stream;
  orca_set_status_word(d_status);
  launch_counter() = 0;
  const int N = 3 * b, R1 = N + u_cap;
  const bool push1 = mode != ORCA_MODE_NO_REUSE;

  ORCA_TRY(g_trace.mark(-1, s));
  const bool fused_head = m->n_layers == 2 && mode == ORCA_MODE_BUDGET;   // the head kernel builds the row list
  if (!fused_head) {
    batch_prep_kernel<<<ceil_div(N, 256), 256, 0, s>>>(d_batch_i32, d_batch_ts, b, w.nodes1, w.ts1, w.cat_dst, w.n1);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
  }
  ORCA_TRY(g_trace.mark(PH_PREP, s));

  float *emb_top = d_emb_out ? d_emb_out : w.emb2;
  bool forked = false;
  bool side_flags = false;   // History.update_flag with a plan rides on the message-winner launch
  int side_prev = 0;
  if (m->n_layers == 1) {
    ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, w.nodes1, w.ts1, N,
                              nullptr, k, w.nbr1, w.eid1, nullptr, w.dt1, d_status, s));
    ORCA_TRY(g_trace.mark(PH_SAMPLE_TOP, s));
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, w.nodes1, N, nullptr, w.qt, s));
    ORCA_TRY(g_trace.mark(PH_QUERY_L2, s));
    ORCA_TRY(orca_attn_gather(w.qt, m->mem.memory, m->edge_table, m->time_w, w.nbr1, w.eid1, w.dt1, k, N,
                              nullptr, w.ctx, w.valid, d_status, s));
    ORCA_TRY(g_trace.mark(PH_GATHER_L2, s));
    ORCA_TRY(orca_attn_output(&m->attn[0], w.ctx, w.valid, m->mem.memory, w.nodes1, N, nullptr, emb_top,
                              nullptr, nullptr, nullptr, w.hidden, s));
    ORCA_TRY(g_trace.mark(PH_OUTPUT_L2, s));
  } else {
    // top-level neighbour table; then the row list of layer 1 by recursion mode
    const int32_t *nbr1 = w.nbr1, *eid1 = w.eid1, *gather2 = w.nbr2, *eid2 = w.eid2;
    const float *dt1 = w.dt1, *dt2 = w.dt2;
    const float *table2 = m->hist_emb;
    const int32_t *d_n1 = w.n1;
    const long long base1 = *m->epoch_base;   // layer-1 row i holds the record base1 + i
    if (mode == ORCA_MODE_BUDGET) {
      // One launch builds the row list of the batch and its neighbour table -- which is both the top-level
      // table and the layer-1 table of the same rows (same node, same query time) -- marks the uncached
      // candidates and records the last occurrence of every row's node.  The uncached out-of-batch
      // neighbours then join the row list and only those rows are sampled by a second launch.
      ORCA_TRY(launch_batch_head(m, d_batch_i32, d_batch_ts, b, w.nodes1, w.ts1, w.cat_dst, w.nbr1, w.eid1, w.dt1,
                                 d_status, base1, s));
      ORCA_TRY(g_trace.mark(PH_SAMPLE_TOP, s));
      ORCA_TRY(launch_uncached_finish(m, N, w.nodes1, w.ts1, u_cap, w.n1, w.n_unc, d_status, base1, s));
      ORCA_TRY(g_trace.mark(PH_UNCACHED, s));
      if (u_cap > 0)
        ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, w.nodes1 + N, w.ts1 + N,
                                  u_cap, w.n_unc, k, w.nbr1 + (size_t)N * k, w.eid1 + (size_t)N * k, nullptr,
                                  w.dt1 + (size_t)N * k, d_status, s));
      gather2 = w.nbr1, eid2 = w.eid1, dt2 = w.dt1;
      *m->epoch_base += R1;
    } else {
      ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, w.nodes1, w.ts1, N,
                                nullptr, k, w.nbr2, w.eid2, nullptr, w.dt2, d_status, s));
      ORCA_TRY(g_trace.mark(PH_SAMPLE_TOP, s));
      if (mode == ORCA_MODE_NO_REUSE) {
        expand_rows_kernel<<<ceil_div(N * k, 256), 256, 0, s>>>(w.nbr2, N, k, w.nodes1, w.ts1, w.nbr2_loc, w.n1);
        ORCA_COUNT_LAUNCH();
        ORCA_LAUNCH_CHECK();
        gather2 = w.nbr2_loc;
        table2 = w.emb1;
      }
      ORCA_TRY(g_trace.mark(PH_UNCACHED, s));
      if (mode == ORCA_MODE_REUSE_ALL) {
        // layer 1 covers the batch rows only and shares the top-level neighbour table
        nbr1 = w.nbr2, eid1 = w.eid2, dt1 = w.dt2;
        d_n1 = nullptr;
      } else {
        ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, w.nodes1, w.ts1, R1,
                                  w.n1, k, w.nbr1, w.eid1, nullptr, w.dt1, d_status, s));
      }
    }
    ORCA_TRY(g_trace.mark(PH_SAMPLE_L1, s));
    if (mode == ORCA_MODE_REUSE_ALL) {
      ORCA_TRY(orca_last_occurrence(w.nodes1, R1, d_n1, m->n_nodes, m->last_pos, *m->epoch_base, w.win1,
                                    nullptr, nullptr, s));
      *m->epoch_base += R1;
    }
    ORCA_TRY(g_trace.mark(PH_LAST_OCC_L1, s));
    // layer 1 over memory rows; its output rows are pushed into the history table
    // (projecting the batch's own rows on the side stream beside the index kernels was measured: no gain,
    // one more launch)
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, w.nodes1, R1, d_n1, w.qt, s));
    ORCA_TRY(g_trace.mark(PH_QUERY_L1, s));
    ORCA_TRY(orca_attn_gather(w.qt, m->mem.memory, m->edge_table, m->time_w, nbr1, eid1, dt1, k, R1,
                              d_n1, w.ctx, w.valid, d_status, s));
    ORCA_TRY(g_trace.mark(PH_GATHER_L1, s));
    // (budget mode: the winners of the push come from the records of the head kernel; the appended
    // rows are distinct out-of-batch nodes, so each of them wins)
    ORCA_TRY(attn_output_impl(&m->attn[0], w.ctx, w.valid, m->mem.memory, w.nodes1, R1, d_n1, w.emb1,
                              push1 ? m->hist_emb : nullptr, push1 ? w.nodes1 : nullptr, push1 ? w.win1 : nullptr,
                              mode == ORCA_MODE_BUDGET ? m->last_pos : nullptr, base1, N, w.hidden,
                              mode == ORCA_MODE_NO_REUSE ? R1 : N, s));
    ORCA_TRY(g_trace.mark(PH_OUTPUT_L1, s));
    if (g_overlap.enabled && !g_trace.on) {
      ORCA_TRY(g_overlap.ensure());
      ORCA_CUDA(cudaEventRecord(g_overlap.fork, s));
      ORCA_CUDA(cudaStreamWaitEvent(g_overlap.aux, g_overlap.fork, 0));
      forked = true;
    }
    // cache flags follow the plan of this batch (History.update_flag); the next reader of the flags is
    // the next batch's head kernel, so this runs beside the top layer
    cudaStream_t fs = forked ? g_overlap.aux : s;
    if (mode != ORCA_MODE_BUDGET) {
      // no flags outside the budgeted recursion
    } else if (d_plan != nullptr) {
      // (done by the message-winner launch below, which is the next single-block kernel of that stream)
      side_prev = *m->n_prev_plan >= 0 ? *m->n_prev_plan : 0;
      if (*m->n_prev_plan < 0) ORCA_CUDA(cudaMemsetAsync(m->cache_flag, 0, (size_t)m->n_nodes, fs));
      side_flags = true;
      *m->n_prev_plan = n_plan;
    } else {
      // plan-less rule: the flags of the pushed ids are set and never cleared
      set_flags_counted_kernel<<<std::min(ceil_div(R1, 256), 1024), 256, 0, fs>>>(m->cache_flag, m->n_nodes,
                                                                                  w.nodes1, R1, w.n1);
      ORCA_COUNT_LAUNCH();
      *m->n_prev_plan = -1;
    }
    ORCA_TRY(g_trace.mark(PH_FLAGS, s));
    // layer 2 over the history rows of the top-level neighbours
    ORCA_TRY(orca_attn_query(&m->attn[1], w.emb1, nullptr, N, nullptr, w.qt, s));
    ORCA_TRY(g_trace.mark(PH_QUERY_L2, s));
    ORCA_TRY(orca_attn_gather(w.qt, table2, m->edge_table, m->time_w, gather2, eid2, dt2, k, N,
                              nullptr, w.ctx, w.valid, d_status, s));
    ORCA_TRY(g_trace.mark(PH_GATHER_L2, s));
    ORCA_TRY(orca_attn_output(&m->attn[1], w.ctx, w.valid, w.emb1, nullptr, N, nullptr, emb_top, nullptr,
                              nullptr, nullptr, w.hidden, s));
    ORCA_TRY(g_trace.mark(PH_OUTPUT_L2, s));
  }

  ORCA_TRY(orca_score(&m->score, emb_top, b, d_prob, s));
  ORCA_TRY(g_trace.mark(PH_SCORE, s));

  // raw messages of the batch (last occurrence per node in [src|dst]) and the memory update; on the
  // auxiliary stream when the fork event was recorded after the last reader of the memory table
  cudaStream_t ms = forked ? g_overlap.aux : s;
  ORCA_TRY(launch_last_occ_compact(d_batch_i32, 2 * b, m->n_nodes, m->last_pos, *m->epoch_base, w.win_pos, w.n_win,
                                   d_status, side_flags ? m->cache_flag : nullptr, m->prev_plan, side_prev, d_plan,
                                   n_plan, ms));
  *m->epoch_base += 2 * b;
  ORCA_TRY(g_trace.mark(PH_LAST_OCC_MSG, s));
  ORCA_TRY(orca_message_store(&m->mem, m->edge_table, m->time_w, d_batch_i32, w.cat_dst, d_batch_ts,
                              d_batch_i32 + 3 * b, b, w.win_pos, 2 * b, w.n_win, w.win_nodes, ms));
  ORCA_TRY(g_trace.mark(PH_MESSAGE, s));
  ORCA_TRY(orca_gru_update(&m->gru, &m->mem, w.win_nodes, 2 * b, w.n_win, 1, w.gru_h, ms));
  ORCA_TRY(g_trace.mark(PH_GRU, s));
  if (forked) {
    ORCA_CUDA(cudaEventRecord(g_overlap.join, g_overlap.aux));
    ORCA_CUDA(cudaStreamWaitEvent(s, g_overlap.join, 0));
  }

  // (the budgeted two-layer batch has its counters written by the kernels that produce them)
  if (!fused_head) {
    publish_counts_kernel<<<1, 1, 0, s>>>(w.n1, w.n_win, d_status);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
  }
  g_last_batch_launches = launch_counter();
  return ORCA_OK;
}

int orca_tgn_eval_batch_sharded(const orca_tgn_t *m, int32_t phase, const int32_t *d_batch_i32,
                                const double *d_batch_ts, int32_t b, const int32_t *d_plan, int32_t n_plan,
                                int32_t u_cap, void *d_workspace, int64_t workspace_bytes,
                                float *d_emb1_local, const float *d_emb1_all, float *d_prob_local,
                                float *d_emb2_local, int32_t *d_status, void *stream) {
  ORCA_CHECK_ARG(m && d_batch_i32 && d_batch_ts && d_workspace && d_status);
  ORCA_CHECK_ARG(phase == 1 || phase == 2);
  ORCA_CHECK_ARG(b > 0 && u_cap >= 0 && n_plan >= 0 && m->n_layers == 2);
  ORCA_CHECK_ARG(m->world >= 1 && m->rank >= 0 && m->rank < m->world);
  ORCA_CHECK_ARG(m->k >= 1 && m->k <= ORCA_MAX_K && m->last_pos && m->epoch_base && *m->epoch_base > 0);
  ORCA_CHECK_ARG(m->hist_emb && m->cache_flag && m->n_prev_plan && (n_plan == 0 || m->prev_plan) && n_plan <= m->plan_cap && m->cand_bitmap);
  const int k = m->k, world = m->world, rank = m->rank;
  Workspace w = carve(d_workspace, b, u_cap, k, m->n_nodes);
  if ((int64_t)w.bytes > workspace_bytes)
    return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch_sharded: workspace of %lld bytes, %lld needed",
                     (long long)workspace_bytes, (long long)w.bytes);
  cudaStream_t s = (cudaStream_t)stream;
  orca_set_status_word(d_status);
  const int N = 3 * b, R1 = N + u_cap;
  const int rpr = ceil_div(R1, world);
  const int b_loc = (b - rank + world - 1) / world;

  const bool direct = m->peer_rows[rank] != nullptr;   // rows exchanged by peer stores, not by the caller
  if (direct) {
    ORCA_CHECK_ARG(world <= ORCA_MAX_WORLD && m->exchange_seq != nullptr && m->peer_flags[rank] != nullptr);
    if ((int64_t)world * rpr * D > m->exchange_cap)
      return set_error(ORCA_E_CAPACITY, "orca_tgn_eval_batch_sharded: exchange buffer of %lld floats, %lld needed",
                       (long long)m->exchange_cap, (long long)world * rpr * D);
  }
  if (phase == 1) {
    ORCA_CHECK_ARG(direct || d_emb1_local != nullptr);
    if (d_emb1_local == nullptr) d_emb1_local = w.emb1;
    launch_counter() = 0;
    // replicated index work: every rank must find the same uncached set and the same winners (row list,
    // top-level table, candidates and last-occurrence records in one launch, as on one GPU)
    const long long base1 = *m->epoch_base;
    ORCA_TRY(launch_batch_head(m, d_batch_i32, d_batch_ts, b, w.nodes1, w.ts1, w.cat_dst, w.nbr2, w.eid2, w.dt2,
                               d_status, base1, s));
    ORCA_TRY(launch_uncached_finish(m, N, w.nodes1, w.ts1, u_cap, w.n1, w.n_unc, d_status, base1, s));
    *m->epoch_base += R1;
    // this rank's layer-1 rows
    shard_l1_kernel<<<ceil_div(rpr, 256), 256, 0, s>>>(w.nodes1, w.ts1, w.n1, rank, world, rpr, w.loc_nodes,
                                                       w.loc_ts, w.n1_loc);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
    ORCA_TRY(orca_sample_topk(m->indptr, m->adj_nbr, m->adj_eid, m->adj_ts, m->n_nodes, w.loc_nodes, w.loc_ts,
                              rpr, w.n1_loc, k, w.nbr1, w.eid1, nullptr, w.dt1, d_status, s));
    ORCA_TRY(orca_attn_query(&m->attn[0], m->mem.memory, w.loc_nodes, rpr, w.n1_loc, w.qt, s));
    ORCA_TRY(orca_attn_gather(w.qt, m->mem.memory, m->edge_table, m->time_w, w.nbr1, w.eid1, w.dt1, k, rpr,
                              w.n1_loc, w.ctx, w.valid, d_status, s));
    if (direct && projections_on_tensor_cores()) {
      // the LayerNorm epilogue of layer 1 delivers the rows itself: one kernel computes and exchanges
      const long long seq = ++*m->exchange_seq;
      tc::PeerOut po{};
      for (int q = 0; q < world; ++q) {
        ORCA_CHECK_ARG(m->peer_rows[q] != nullptr && m->peer_flags[q] != nullptr);
        po.rows[q] = m->peer_rows[q];
        po.flags[q] = m->peer_flags[q];
      }
      po.counter = m->peer_flags[rank] + ORCA_MAX_WORLD;
      po.off = (seq & 1) * m->exchange_cap + (long long)rank * rpr * D;
      po.world = world, po.rank = rank, po.seq = (int)seq;
      ORCA_TRY(attn_output_impl(&m->attn[0], w.ctx, w.valid, m->mem.memory, w.loc_nodes, rpr, w.n1_loc, d_emb1_local,
                                nullptr, nullptr, nullptr, nullptr, 0, 0, w.hidden, 0, s, &po));
      return ORCA_OK;
    }
    ORCA_TRY(orca_attn_output(&m->attn[0], w.ctx, w.valid, m->mem.memory, w.loc_nodes, rpr, w.n1_loc,
                              d_emb1_local, nullptr, nullptr, nullptr, w.hidden, s));
    if (direct) {
      // (fp32 debug projections: a separate kernel fans the rows out)
      const long long seq = ++*m->exchange_seq;
      Peers p{};
      for (int q = 0; q < world; ++q) {
        ORCA_CHECK_ARG(m->peer_rows[q] != nullptr && m->peer_flags[q] != nullptr);
        p.rows[q] = m->peer_rows[q];
        p.flags[q] = m->peer_flags[q];
      }
      const long long off = (seq & 1) * m->exchange_cap + (long long)rank * rpr * D;
      ORCA_CUDA(launch_dep(exchange_fanout_kernel, std::min(ceil_div(rpr * (D / 4), 256), 148), 256, 0, s,
                           (const float *)d_emb1_local, (const int32_t *)w.n1_loc, rpr, p, world, rank, off,
                           (int)seq));
      ORCA_COUNT_LAUNCH();
    }
    return ORCA_OK;
  }

  if (direct) {
    const long long seq = *m->exchange_seq;
    ORCA_CUDA(launch_dep(exchange_wait_kernel, 1, 32, 0, s, (const int32_t *)m->peer_flags[rank], world, (int)seq,
                         d_status));
    ORCA_COUNT_LAUNCH();
    d_emb1_all = m->peer_rows[rank] + (seq & 1) * m->exchange_cap;
  }
  ORCA_CHECK_ARG(d_emb1_all != nullptr && d_prob_local != nullptr);
  // every replica of the history table receives every layer-1 row
  // (winners by the records phase 1 made: it advanced the epoch by R1 and nothing recorded since)
  push_gathered_kernel<<<ceil_div(R1, 4), 256, 0, s>>>(m->hist_emb, d_emb1_all, w.nodes1,
                                                       reinterpret_cast<const unsigned long long *>(m->last_pos),
                                                       *m->epoch_base - R1, N, w.n1, world, rpr);
  ORCA_COUNT_LAUNCH();
  bool side_flags = false;   // History.update_flag with a plan rides on the message-winner launch below
  int side_prev = 0;
  if (d_plan != nullptr) {
    side_prev = *m->n_prev_plan >= 0 ? *m->n_prev_plan : 0;
    if (*m->n_prev_plan < 0) ORCA_CUDA(cudaMemsetAsync(m->cache_flag, 0, (size_t)m->n_nodes, s));
    side_flags = true;
    *m->n_prev_plan = n_plan;
  } else {
    set_flags_counted_kernel<<<std::min(ceil_div(R1, 256), 1024), 256, 0, s>>>(m->cache_flag, m->n_nodes,
                                                                               w.nodes1, R1, w.n1);
    ORCA_COUNT_LAUNCH();
    *m->n_prev_plan = -1;
  }
  // the memory table was last read in phase 1: the replicated raw-message / GRU chain can run aside
  bool forked = false;
  if (g_overlap.enabled) {
    ORCA_TRY(g_overlap.ensure());
    ORCA_CUDA(cudaEventRecord(g_overlap.fork, s));
    ORCA_CUDA(cudaStreamWaitEvent(g_overlap.aux, g_overlap.fork, 0));
    forked = true;
  }
  cudaStream_t ms = forked ? g_overlap.aux : s;
  ORCA_TRY(launch_last_occ_compact(d_batch_i32, 2 * b, m->n_nodes, m->last_pos, *m->epoch_base, w.win_pos, w.n_win,
                                   nullptr, side_flags ? m->cache_flag : nullptr, m->prev_plan, side_prev, d_plan,
                                   n_plan, ms));
  *m->epoch_base += 2 * b;
  ORCA_TRY(orca_message_store(&m->mem, m->edge_table, m->time_w, d_batch_i32, w.cat_dst, d_batch_ts,
                              d_batch_i32 + 3 * b, b, w.win_pos, 2 * b, w.n_win, w.win_nodes, ms));
  ORCA_TRY(orca_gru_update(&m->gru, &m->mem, w.win_nodes, 2 * b, w.n_win, 1, w.gru_h, ms));
  if (b_loc > 0) {
    // top layer and scores of this rank's edges
    shard_l2_kernel<<<ceil_div(3 * b_loc, 8), 256, 0, s>>>(w.nbr2, w.eid2, w.dt2, b, k, rank, world, rpr, b_loc,
                                                           w.feat_idx, w.nbr2_loc, w.eid2_loc, w.dt2_loc);
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
    float *emb2 = d_emb2_local ? d_emb2_local : w.emb2;
    ORCA_TRY(orca_attn_query(&m->attn[1], d_emb1_all, w.feat_idx, 3 * b_loc, nullptr, w.qt, s));
    ORCA_TRY(orca_attn_gather(w.qt, m->hist_emb, m->edge_table, m->time_w, w.nbr2_loc, w.eid2_loc, w.dt2_loc, k,
                              3 * b_loc, nullptr, w.ctx, w.valid, d_status, s));
    ORCA_TRY(orca_attn_output(&m->attn[1], w.ctx, w.valid, d_emb1_all, w.feat_idx, 3 * b_loc, nullptr, emb2,
                              nullptr, nullptr, nullptr, w.hidden, s));
    ORCA_TRY(orca_score(&m->score, emb2, b_loc, d_prob_local, s));
  }
  if (forked) {
    ORCA_CUDA(cudaEventRecord(g_overlap.join, g_overlap.aux));
    ORCA_CUDA(cudaStreamWaitEvent(s, g_overlap.join, 0));
  }
  publish_counts_kernel<<<1, 1, 0, s>>>(w.n1, w.n_win, d_status);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  g_last_batch_launches = launch_counter();
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

int orca_stage_h2d(void *d_dst, const void *h_src, int64_t bytes, void *stream) {
  ORCA_CHECK_ARG(d_dst && h_src && bytes >= 0);
  if (bytes == 0) return ORCA_OK;
  ORCA_CUDA(cudaMemcpyAsync(d_dst, h_src, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return ORCA_OK;
}

int orca_set_dependent_launch(int32_t enable) {
  dependent_launch_enabled() = enable != 0;
  return ORCA_OK;
}

int orca_set_overlap(int32_t enable) {
  g_overlap.enabled = enable != 0;
  return ORCA_OK;
}

int orca_trace(int32_t enable) {
  g_trace.on = enable != 0;
  g_trace.used = 0;
  return ORCA_OK;
}

int orca_trace_phases(void) { return PH_COUNT; }
const char *orca_trace_phase_name(int32_t phase) {
  return (phase >= 0 && phase < PH_COUNT) ? kPhaseNames[phase] : "";
}

int orca_trace_read(double *h_ms_per_phase) {
  ORCA_CHECK_ARG(h_ms_per_phase);
  for (int i = 0; i < PH_COUNT; ++i) h_ms_per_phase[i] = 0.0;
  for (size_t i = 1; i < g_trace.used; ++i) {
    const int ph = g_trace.phase_of[i];
    if (ph < 0) continue;  // first event of a batch
    ORCA_CUDA(cudaEventSynchronize(g_trace.ev[i]));
    float ms = 0.f;
    ORCA_CUDA(cudaEventElapsedTime(&ms, g_trace.ev[i - 1], g_trace.ev[i]));
    h_ms_per_phase[ph] += ms;
  }
  g_trace.used = 0;
  return ORCA_OK;
}

int orca_read_status(int32_t *d_status, int32_t *h_counts, void *stream) {
  ORCA_CHECK_ARG(d_status);
  int32_t h[4] = {0, 0, 0, 0};
  cudaStream_t s = (cudaStream_t)stream;
  ORCA_CUDA(cudaMemcpyAsync(h, d_status, sizeof(h), cudaMemcpyDeviceToHost, s));
  ORCA_CUDA(cudaStreamSynchronize(s));
  if (h_counts) {
    h_counts[0] = h[0];
    h_counts[1] = h[1];
    h_counts[2] = h[2];
    h_counts[3] = g_last_batch_launches;
  }
  if (h[0] != 0) {
    ORCA_CUDA(cudaMemsetAsync(d_status, 0, sizeof(h), s));
    return set_error(h[0], "device status %d (detail %d)", h[0], h[3]);
  }
  return ORCA_OK;
}

}  // extern "C"
