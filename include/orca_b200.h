/*
 * orca_b200 -- C ABI of the B200 (sm_100a) implementation of Orca's per-batch temporal-embedding
 * path.  Every entry point replaces one function of the reference (LuckyLYM/Orca, pure Python +
 * numba); the reference location is cited beside each declaration.
 *
 * Conventions
 *   - All functions return 0 on success or one of the ORCA_E_* codes; orca_last_error() gives the
 *     message of the calling thread's last failure.
 *   - Pointers named d_* are device pointers, h_* host pointers.  `stream` is a cudaStream_t passed
 *     as void*.  Unless stated otherwise a function only enqueues work on `stream`, allocates
 *     nothing and keeps no pointer after it returns (the reference replaces its state tensors
 *     on restore, modules/memory.py:43, so state is passed per call).
 *   - Row counts that are only known on the device (the number of uncached neighbours, the number
 *     of unique positive nodes) are passed as a capacity `*_cap` plus a device pointer
 *     `d_n_*`; kernels launched for the capacity read the count and idle beyond it.
 *   - Feature width is fixed at 172 floats (node = memory = time = edge dimension) and the number
 *     of heads at 2, the only widths the headline workloads use; ORCA_E_UNSUPPORTED otherwise.
 *   - Ids are int32 on the device (node 0 and edge 0 are padding), times are float64 where the
 *     reference keeps float64.
 */
#ifndef ORCA_B200_H
#define ORCA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORCA_OK 0
#define ORCA_E_BADARG 1      /* null pointer, negative size, K out of range            */
#define ORCA_E_UNSUPPORTED 2 /* dimension or mode this build has no kernel for          */
#define ORCA_E_CUDA 3        /* a CUDA runtime call failed (message has the CUDA error) */
#define ORCA_E_CAPACITY 4    /* a device-side count exceeded the capacity it was given  */
#define ORCA_E_BOUNDS 5      /* a kernel met an id outside its table (debug checks)     */
#define ORCA_E_TIMEOUT 6     /* a bounded device-side wait gave up                      */

#define ORCA_DIM 172
#define ORCA_HEADS 2
#define ORCA_MAX_K 32
#define ORCA_MAX_WORLD 8   /* GPUs of one node */
#define ORCA_FLAG_WORDS 48    /* flag words of one rank's exchange buffer: [0,8) layer-1 rows posted by rank q, [8]
                                 check-out counter of the layer-1 kernel, [16,24) memory rows posted by rank q,
                                 [24] check-out counter of the memory-update kernel, [32,40) (split by layer)
                                 last batch whose buffers top-layer rank q has finished reading */
#define ORCA_FLAG_CONSUMED 32
#define ORCA_EXCHANGE_SLOTS 4 /* batches whose layer-1 rows an exchange buffer holds: with the lanes of the
                                 batch pipeline a rank's layer 1 may be two batches ahead of a peer's layer 2 */
#define ORCA_CAND_CAP 2048 /* listed candidates of the uncached set; more fall back to a bitmap scan */
#define ORCA_MSG_DIM (4 * ORCA_DIM)          /* [mem_src | mem_dst | edge feat | time enc] */
#define ORCA_KEY_DIM (3 * ORCA_DIM)          /* [neighbour | edge feat | time enc]         */
#define ORCA_QT_DIM (ORCA_HEADS * ORCA_KEY_DIM)
#define ORCA_QT_LD 1056                      /* row stride of the projected query: 2 heads x 528 */

const char *orca_last_error(void);
int orca_version(void);

/* ------------------------------------------------------------------------------------------
 * Contexts (no counterpart in the reference, which is a single Python process on one device).
 * A context owns what a caller of the batch entry points would otherwise share with every other
 * caller in the process: three auxiliary CUDA streams and the events that tie them to the caller's
 * stream, the switches below, the device status word the projection kernels report to, the phase
 * tracer and 1 KB of zeroed device words (work tickets).  orca_ctx_create works on the current
 * device and is the one call of the library that allocates device memory.  A model descriptor
 * (orca_tgn_t.ctx) names its context; two models with contexts of their own share nothing.
 * Entry points without a descriptor, and descriptors with ctx == NULL, use the default context of
 * the current device, created on first use; `ctx == NULL` below means that context.
 */
typedef struct orca_ctx orca_ctx_t;
int orca_ctx_create(orca_ctx_t **out);
int orca_ctx_destroy(orca_ctx_t *ctx);
/* Projection kernels: 0 (default) = tcgen05 tensor cores, every fp32 operand split into a bf16 head
 * and a bf16 tail (three MMAs per product, layer error 3-5e-4), 1 = plain fp32 SIMT tiles (debug
 * reference for the tensor-core path, ~5e-5). */
#define ORCA_OPT_PROJECTION_MODE 0
/* 1 (default): the raw-message / GRU chain of a batch runs on an auxiliary stream beside the
 * attention layers; 0: everything on the caller's stream. */
#define ORCA_OPT_OVERLAP 1
/* 1 (default): kernels are enqueued with programmatic stream serialisation: a kernel's blocks may be
 * scheduled and run their set-up while the kernel before it in the stream drains, and wait
 * (griddepcontrol.wait) before touching anything it produced.  Results are identical either way. */
#define ORCA_OPT_DEPENDENT_LAUNCH 2
/* 1 (default, needs OVERLAP): the budgeted two-layer batch is spread over four streams -- index work
 * (sampling, uncached set, message winners, cache flags) a batch ahead, layer 1, raw messages + GRU,
 * and layer 2 + scores on the caller's stream beside the next batch's layer 1.  0: one batch after
 * the other.  Results are identical either way. */
#define ORCA_OPT_LOOKAHEAD 3
/* SM clocks a device-side wait (mbarrier of the projection kernels, peer flags of the multi-GPU
 * exchange) may spin before it gives up with ORCA_E_TIMEOUT in the status word; default 2e9 (about a
 * second). */
#define ORCA_OPT_WAIT_LIMIT 4
/* 1: CUDA events are recorded at the phase boundaries of every batch (which then runs on the caller's
 * stream alone); see orca_trace_read. */
#define ORCA_OPT_TRACE 5
int orca_ctx_set(orca_ctx_t *ctx, int32_t option, int64_t value);
/* Device status word (int32[4], see orca_read_status) to which projection kernels launched through the
 * stand-alone entry points report a bounded wait that gave up; NULL (default) = not reported.  The
 * batch entry points report to their own d_status. */
int orca_ctx_set_status_word(orca_ctx_t *ctx, int32_t *d_status);
/* Which of the two index-buffer sets of the workspace the last batch of the context used (see
 * orca_eval_workspace_row_list). */
int orca_ctx_last_parity(orca_ctx_t *ctx);

/* ------------------------------------------------------------------------------------------
 * Time-sorted adjacency.  Replaces get_neighbor_finder (utils/util.py:91-105): every edge is
 * listed under both endpoints; each node's list is stably sorted by timestamp with insertion
 * order = stream order, the source-side entry of an edge ahead of its destination-side entry.
 * Host function (runs on the CPU, once per graph).  indptr has n_nodes+1 entries, the other
 * three outputs 2*n_edges entries.
 */
int orca_csr_build_host(const int64_t *h_src, const int64_t *h_dst, const int64_t *h_eidx,
                        const double *h_ts, int64_t n_edges, int64_t n_nodes, int64_t *h_indptr,
                        int32_t *h_nbr, int32_t *h_eid, double *h_adj_ts);

/* The same adjacency built on the device from device arrays: a stable radix sort of the 2*n_edges
 * records by (node, timestamp), least significant byte first (8 passes over the timestamp's bytes, then
 * the bytes of the node id), so any stream order and any ties come out as the reference's stable sort
 * leaves them.  Outputs are device arrays of the sizes above; ids outside [0, n_nodes) are reported in
 * d_status (ORCA_E_BOUNDS).  Enqueues on `stream`; the workspace (256-byte aligned) is sized by
 * orca_csr_build_workspace_bytes. */
int64_t orca_csr_build_workspace_bytes(int64_t n_edges, int64_t n_nodes);
int orca_csr_build(const int64_t *d_src, const int64_t *d_dst, const int64_t *d_eidx, const double *d_ts,
                   int64_t n_edges, int64_t n_nodes, int64_t *d_indptr, int32_t *d_nbr, int32_t *d_eid,
                   double *d_adj_ts, int32_t *d_status, void *d_workspace, int64_t workspace_bytes,
                   void *stream);

/* ------------------------------------------------------------------------------------------
 * Temporal neighbour sampling.  Replaces NeighborFinder.get_temporal_neighbor and find_before
 * (utils/util.py:129-151): per query the interactions strictly before the query time, the last k
 * of them, right-aligned, zero-padded on the left.  Outputs are [n_query_cap, k] row-major;
 * d_edge_times (float32, the reference's return dtype) and d_delta may be NULL.  d_delta is the
 * fused time difference of modules/embedding_module.py:266-267: float32(t_query - float64(
 * float32(t_edge))), and t_query itself on padded slots.
 * d_n_query may be NULL (then all n_query_cap rows are queries).
 */
int orca_sample_topk(const int64_t *d_indptr, const int32_t *d_adj_nbr, const int32_t *d_adj_eid,
                     const double *d_adj_ts, int64_t n_nodes, const int32_t *d_nodes,
                     const double *d_ts, int32_t n_query_cap, const int32_t *d_n_query, int32_t k,
                     int32_t *d_nbr, int32_t *d_eid, float *d_edge_times, float *d_delta,
                     int32_t *d_status, void *stream);

/* orca_sample_topk that also prepares find_uncached_out_of_batch_neighbors
 * (modules/embedding_module.py:200-212): every sampled neighbour id (the padding node 0 for an empty
 * slot) whose cache flag is 0 gets its bit set in d_cand_bitmap ((n_nodes+31)/32 words, all zero on
 * entry); orca_find_uncached_marked turns the bitmap into the uncached set. */
int orca_sample_topk_mark(const int64_t *d_indptr, const int32_t *d_adj_nbr, const int32_t *d_adj_eid,
                          const double *d_adj_ts, int64_t n_nodes, const int32_t *d_nodes,
                          const double *d_ts, int32_t n_query_cap, const int32_t *d_n_query, int32_t k,
                          int32_t *d_nbr, int32_t *d_eid, float *d_edge_times, float *d_delta,
                          int32_t *d_status, const uint8_t *d_cache_flag, uint32_t *d_cand_bitmap,
                          void *stream);

/* find_before (utils/util.py:129-131) on its own: the number of interactions of d_nodes[i]
 * strictly before d_ts[i]. */
int orca_find_before(const int64_t *d_indptr, const double *d_adj_ts, int64_t n_nodes,
                     const int32_t *d_nodes, const double *d_ts, int32_t n_query,
                     int32_t *d_count, void *stream);

/* ------------------------------------------------------------------------------------------
 * Uncached out-of-batch neighbours.  Replaces find_uncached_out_of_batch_neighbors
 * (modules/embedding_module.py:200-212): ascending unique ids of the neighbour table that are not
 * query nodes and whose cache flag is 0, minus the first entry.  The ids are APPENDED to the
 * query list: d_nodes_io[n_query .. n_query+|U|) = U, d_ts_io likewise = max over the n_query
 * timestamps (modules/embedding_module.py:253-257), and *d_n_total = n_query + |U|.
 * If |U| > u_cap the surplus is dropped and ORCA_E_CAPACITY is written to *d_status.
 * d_bitmap: scratch of orca_find_uncached_scratch_bytes(n_nodes) bytes.
 */
int64_t orca_find_uncached_scratch_bytes(int64_t n_nodes);
int orca_find_uncached(const int32_t *d_nbr, int32_t n_query, int32_t k, const uint8_t *d_cache_flag,
                       int64_t n_nodes, int32_t *d_nodes_io, double *d_ts_io, int32_t u_cap,
                       int32_t *d_n_total, void *d_bitmap, int32_t *d_status, void *stream);

/* orca_find_uncached on a bitmap filled by orca_sample_topk_mark: same outputs; the bitmap is all
 * zero again when the kernel has run. */
int orca_find_uncached_marked(uint32_t *d_cand_bitmap, int32_t n_query, int64_t n_nodes, int32_t *d_nodes_io,
                              double *d_ts_io, int32_t u_cap, int32_t *d_n_total, int32_t *d_status,
                              void *stream);

/* ------------------------------------------------------------------------------------------
 * Last-occurrence selection.  Replaces the np.unique(np.flip(nodes), return_index=True) rule of
 * TGN.get_raw_messages (model/tgn_model.py:172-176) and gives History.push its deterministic
 * winner (modules/history.py:38-40 under deterministic execution): d_is_last[i] = 1 iff no
 * j > i has d_ids[j] == d_ids[i].
 * d_last_pos: int64 [n_nodes] scratch owned by the caller, zero-initialised once; `epoch_base`
 * must grow by at least n_cap between calls that share the scratch (no clearing is needed).
 * If d_compact is non-NULL the positions with is_last == 1 are also written there in ascending
 * position order and their number to *d_n_compact.
 */
int orca_last_occurrence(const int32_t *d_ids, int32_t n_cap, const int32_t *d_n, int64_t n_nodes,
                         int64_t *d_last_pos, int64_t epoch_base, uint8_t *d_is_last,
                         int32_t *d_compact, int32_t *d_n_compact, void *stream);

/* ------------------------------------------------------------------------------------------
 * Prepared weights of one attention layer (host side composes them once per weight update from
 * the reference's parameters; see orca_b200/weights.py for the algebra):
 *   qt   = h_src . Mq + cq                                  [*, 2 x 528] (scaled, K-projected query;
 *                                                            516 used per head, stride ORCA_QT_LD)
 *   hid  = relu([ctx | h_src] . G + b1 + valid * g)         [*, 172]
 *   out  = LayerNorm(hid . W2t + b2) * ln_w + ln_b          [*, 172]
 * All matrices are row-major [in, out] float32.  The *_tc members hold the same matrices split into
 * a bf16 head and a bf16 tail and packed into the stage images of the tensor-core kernel
 * (orca_b200/weights.py: pack_tc).
 */
typedef struct {
  const float *Mq;   /* [172, 1056]  */
  const float *cq;   /* [1056]       */
  const float *G;    /* [1204, 172]  */
  const float *b1;   /* [172]        */
  const float *g;    /* [172]        */
  const float *W2t;  /* [172, 172]   */
  const float *b2;   /* [172]        */
  const float *ln_w; /* [172]        */
  const float *ln_b; /* [172]        */
  const float *Mq_tc, *G_tc, *W2t_tc;
} orca_attn_weights_t;

/* Step 1 of TemporalAttentionLayer.forward (model/temporal_attention.py:41-48, the query side of
 * nn.MultiheadAttention): qt[r] = feat[idx ? idx[r] : r] . Mq + cq. */
int orca_attn_query(const orca_attn_weights_t *w, const float *d_feat, const int32_t *d_idx,
                    int32_t n_rows_cap, const int32_t *d_n_rows, float *d_qt, void *stream);

/* Step 2, the fused gather-attention kernel (model/temporal_attention.py:43-53 with
 * model/time_encoding.py:23-28 and the gathers of modules/embedding_module.py:262-270 and
 * modules/history.py:32-36): per row, gather the k neighbour rows of d_nbr_table and edge-feature
 * rows, encode cos(delta * w_time), masked 2-head softmax over the slots, weighted key sum.
 *   d_qt    [n_rows_cap, ORCA_QT_LD]
 *   d_ctx   [n_rows_cap, 1032]   sum_j a_hj * [nbr_j | efeat_j | tenc_j] per head
 *   d_valid [n_rows_cap]         0 where every slot is padding (the layer output of such a row
 *                                ignores the attention term, model/temporal_attention.py:46,52)
 */
int orca_attn_gather(const float *d_qt, const float *d_nbr_table, const float *d_edge_table,
                     const float *d_time_w, const int32_t *d_nbr, const int32_t *d_eid,
                     const float *d_delta, int32_t k, int32_t n_rows_cap, const int32_t *d_n_rows,
                     float *d_ctx, uint8_t *d_valid, int32_t *d_status, void *stream);

/* Benchmark support for the kernel above (no counterpart in the reference): while enabled, every
 * orca_attn_gather launch is bracketed by CUDA events on its stream and adds {rows that gathered,
 * neighbour slots gathered} to the two uint64 device counters.  _read synchronises on the recorded
 * events, returns their summed duration and count, and forgets them. */
int orca_attn_gather_profile(orca_ctx_t *ctx, int32_t enable, void *d_counters);
int orca_attn_gather_profile_read(orca_ctx_t *ctx, double *h_ms_total, int64_t *h_launches);

/* Step 3 (out-projection, merger and LayerNorm, model/temporal_attention.py:48-55 and
 * utils/util.py:21-24): d_out[r] = LN(fc2(relu(fc1([attn | h_src])))).  If d_push_table is
 * non-NULL the row is also written to d_push_table[d_push_ids[r]] when d_push_win[r] != 0, which
 * is History.push (modules/history.py:38-40) with the last occurrence of an id winning.
 * d_scratch_hidden: no longer used (both projection kernels keep the merger's hidden tile on the SM); may be
 * NULL. */
int orca_attn_output(const orca_attn_weights_t *w, const float *d_ctx, const uint8_t *d_valid,
                     const float *d_feat, const int32_t *d_idx, int32_t n_rows_cap,
                     const int32_t *d_n_rows, float *d_out, float *d_push_table,
                     const int32_t *d_push_ids, const uint8_t *d_push_win, float *d_scratch_hidden,
                     void *stream);

/* ------------------------------------------------------------------------------------------
 * Historical-embedding cache.  Replace History.pull / push / update_flag
 * (modules/history.py:25-40).
 */
int orca_history_pull(const float *d_emb, const int32_t *d_ids, int64_t n, float *d_out, void *stream);
/* rows with d_win[i] == 0 are skipped (pass the is_last flags of orca_last_occurrence) */
int orca_history_push(float *d_emb, const float *d_x, const int32_t *d_ids, const uint8_t *d_win,
                      int32_t n_cap, const int32_t *d_n, void *stream);
/* cache_flag = 0 everywhere, then 1 on d_plan; the previous plan is passed so that only its
 * entries are cleared (NULL/0 clears all n_nodes flags).  With d_plan == NULL the flags of
 * d_ids are set and nothing is cleared (the reference's plan-less branch). */
int orca_history_set_flags(uint8_t *d_cache_flag, int64_t n_nodes, const int32_t *d_prev_plan,
                           int32_t n_prev, const int32_t *d_plan, int32_t n_plan, void *stream);

/* ------------------------------------------------------------------------------------------
 * Link scorer.  Replaces affinity_score + sigmoid of TGN.compute_edge_probabilities
 * (model/tgn_model.py:154-157; MergeLayer utils/util.py:12-24).  d_emb is [3*b, 172] =
 * [src | dst | neg]; d_prob is [2*b] = [pos | neg].
 */
typedef struct {
  const float *W1t; /* [344, 172] */
  const float *b1;  /* [172]      */
  const float *w2;  /* [172]      */
  float b2;
  const float *W1t_tc;
} orca_score_weights_t;
int orca_score(const orca_score_weights_t *w, const float *d_emb, int32_t b, float *d_prob, void *stream);

/* ------------------------------------------------------------------------------------------
 * Raw messages and memory update.
 */
typedef struct {
  float *memory;       /* [n_nodes, 172]                    modules/memory.py:18 */
  float *last_update;  /* [n_nodes]                         modules/memory.py:19 */
  float *messages;     /* [n_nodes, 688]                    modules/memory.py:22 */
  float *msg_ts;       /* [n_nodes]                         modules/memory.py:23 */
  uint8_t *msg_flag;   /* [n_nodes], the `nodes` bool array modules/memory.py:21 */
  int64_t n_nodes;
} orca_memory_t;

/* Replaces TGN.get_raw_messages + Memory.store_raw_messages (model/tgn_model.py:172-191,
 * modules/memory.py:25-28).  d_cat_src/d_cat_dst are the 2*b concatenations [src|dst], [dst|src];
 * position p carries time d_ts[p % b] and edge d_eidx[p % b].  d_win_pos/d_n_win are the compact
 * winner positions from orca_last_occurrence.  Message of node a = cat_src[p]:
 * [memory[a] | memory[cat_dst[p]] | efeat[e] | cos((float32(t) - last_update[a]) * w_time)].
 * d_win_nodes (may be NULL) receives the node id of every winner, the list the memory update runs
 * over. */
int orca_message_store(const orca_memory_t *mem, const float *d_edge_table, const float *d_time_w,
                       const int32_t *d_cat_src, const int32_t *d_cat_dst, const double *d_ts,
                       const int32_t *d_eidx, int32_t b, const int32_t *d_win_pos, int32_t n_win_cap,
                       const int32_t *d_n_win, int32_t *d_win_nodes, void *stream);

/* GRU weights: Wg is [860, 688] = [message 688 ; memory 172] x [172 units x 4 gate columns
 * (r, z, n_input, n_hidden) interleaved], bg [688] likewise. */
typedef struct {
  const float *Wg;
  const float *bg;     /* padded to 704 entries */
  const float *Wg_tc;
} orca_gru_weights_t;

/* Replaces SequenceMemoryUpdater.update_memory / update_memory_in_test with nn.GRUCell
 * (modules/memory_updater.py:25-53,86): for every listed node whose msg_flag is set:
 * last_update = msg_ts, memory = GRU(messages, memory); if clear_flags the flag is cleared
 * afterwards (Memory.clear_messages, modules/memory.py:49-50).  d_nodes may hold duplicates only if
 * they are flagged once (the callers pass unique ids). */
int orca_gru_update(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes,
                    int32_t n_cap, const int32_t *d_n, int32_t clear_flags, float *d_scratch_h,
                    void *stream);
int64_t orca_gru_scratch_bytes(int32_t n_cap);

/* The same update for callers that cannot allocate device memory (no counterpart in the reference,
 * which allocates freely through PyTorch): the scratch is a fixed array inside the library, so the
 * call takes no scratch pointer and is limited to ORCA_GRU_STATIC_MAX_ROWS listed nodes
 * (ORCA_E_CAPACITY beyond that).  The first call on each device resolves the array's device address
 * and should be made outside stream capture.  Calls share the array: do not let two of them overlap
 * on the GPU. */
#define ORCA_GRU_STATIC_MAX_ROWS 4096
int orca_gru_update_static(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes,
                           int32_t n_cap, const int32_t *d_n, int32_t clear_flags, void *stream);

/* ------------------------------------------------------------------------------------------
 * Offline cache planning.  Replaces read_batches + MRD_numba / LRU_numba / TwoQ_numba
 * (utils/cache.py:19-89, 92-166, 338-403, 175-333).  The neighbour tables of ALL batches are
 * sampled beforehand with one orca_sample_topk launch over the query list in which batch b (edges
 * [s, e) of the stream, s = b*bs) contributes rows 2*s .. 2*s+(e-s)-1 = its sources and the next
 * (e-s) rows = its destinations, each at the edge's own timestamp; h_nbr is that table copied to
 * the host ([2*n_edges, k] int32).  The batch-sequential policy then runs on the host.
 * strategy: 0 = MRD, 1 = LRU, 2 = 2Q.  `seed` seeds the Mersenne Twister behind the random
 * evictions of LRU / 2Q (the reference's numba generator seeded with np.random.seed(seed) from
 * jitted code).  Plan of batch b = h_plan_flat[h_plan_off[b] .. h_plan_off[b+1]) in the reference's
 * order (MRD: argsort order; LRU: ascending; 2Q: FIFO half ascending then LRU half ascending).
 * h_plan_off has n_batches+1 entries; plan_cap >= n_batches*(budget+2) always suffices.
 * h_stats = {n_reuse, n_recompute, sum of reuse distances} (utils/cache.py:427).
 * Host function.
 */
int orca_plan_host(int32_t strategy, const int64_t *h_src, const int64_t *h_dst, int64_t n_edges,
                   int32_t bs, int32_t k, const int32_t *h_nbr, int64_t n_nodes, int32_t budget,
                   uint32_t seed, int32_t *h_plan_flat, int64_t plan_cap, int64_t *h_plan_off,
                   double *h_stats);

/* The MRD plan computed on the device (utils/cache.py:19-89 and 92-166, one call for both).
 * d_nodes: the query list described above ([2*n_edges] int32, batch b = its sources, then its
 * destinations); d_nbr: the neighbour table sampled for it ([2*n_edges, k] int32).  Two kernels walk
 * the batches, one backwards (next use of every node at every batch) and one forwards (candidates from
 * bitmaps in ascending order, keys, the first `budget` places of numba's argsort with its order among
 * equal keys, statistics).  Outputs, all on the device: d_plan_flat / d_plan_off as in orca_plan_host
 * (plan_cap >= n_batches * budget always suffices), d_stats = int64 {n_reuse, n_recompute, sum of
 * reuse distances}, d_status (int32[4], ORCA_E_CAPACITY when d_plan_flat is too small).
 * Enqueues on `stream`; the workspace (256-byte aligned) is sized by orca_plan_mrd_workspace_bytes. */
int64_t orca_plan_mrd_workspace_bytes(int64_t n_edges, int32_t bs, int32_t k, int64_t n_nodes, int32_t budget);
int orca_plan_mrd(const int32_t *d_nodes, int64_t n_edges, int32_t bs, int32_t k, const int32_t *d_nbr,
                  int64_t n_nodes, int32_t budget, int32_t *d_plan_flat, int64_t plan_cap,
                  int64_t *d_plan_off, int64_t *d_stats, int32_t *d_status, void *d_workspace,
                  int64_t workspace_bytes, void *stream);

/* Any of the three plans on the device: strategy 0 = MRD (the call above), 1 = LRU (utils/cache.py:338-403),
 * 2 = 2Q (:175-333).  LRU and 2Q run as one thread block: their random evictions are a serial Fisher-Yates
 * shuffle per batch, driven by numba's Mersenne Twister (`seed` as in orca_plan_host) and walked by one
 * thread; the split of the tables, the statistics, the ascending member lists of the sets and the
 * least-recently-used evictions (first entries of numba's argsort of the last-use times) are data parallel
 * around it.  Arguments, outputs and plan order as in orca_plan_mrd / orca_plan_host
 * (plan_cap >= n_batches * budget always suffices). */
int64_t orca_plan_device_workspace_bytes(int32_t strategy, int64_t n_edges, int32_t bs, int32_t k,
                                         int64_t n_nodes, int32_t budget);
int orca_plan_device(int32_t strategy, const int32_t *d_nodes, int64_t n_edges, int32_t bs, int32_t k,
                     const int32_t *d_nbr, int64_t n_nodes, int32_t budget, uint32_t seed,
                     int32_t *d_plan_flat, int64_t plan_cap, int64_t *d_plan_off, int64_t *d_stats,
                     int32_t *d_status, void *d_workspace, int64_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------------------------
 * One whole eval batch: TGN.compute_edge_probabilities(..., reuse=True, train=False, cache_plan)
 * with budget != 0 (model/tgn_model.py:95-157 over modules/embedding_module.py:215-285), enqueued
 * on `stream` without any host synchronisation.
 */
/* The three recursions TGN.compute_temporal_embeddings chooses between (model/tgn_model.py:114-120),
 * for the two-layer model; with one layer they coincide.
 *   ORCA_MODE_BUDGET    reuse=True, budget != 0: compute_embedding_budget_reuse
 *                       (modules/embedding_module.py:215-285) -- cached rows come from the history table,
 *                       uncached out-of-batch neighbours join the layer-1 row list.
 *   ORCA_MODE_REUSE_ALL reuse=True, budget == 0: compute_embedding_reuse
 *                       (modules/embedding_module.py:154-182) -- layer 1 covers the 3b batch rows only,
 *                       pushes them, and the top layer reads every neighbour from the history table.
 *   ORCA_MODE_NO_REUSE  reuse=False: compute_embedding (modules/embedding_module.py:116-147) -- layer 1
 *                       covers the 3b rows and each of their 3b*k neighbour slots; no table is written.
 *                       The workspace must be sized with u_cap = 3*b*k. */
#define ORCA_MODE_BUDGET 0
#define ORCA_MODE_REUSE_ALL 1
#define ORCA_MODE_NO_REUSE 2

typedef struct {
  /* graph */
  const int64_t *indptr; const int32_t *adj_nbr; const int32_t *adj_eid; const double *adj_ts;
  const float *edge_table; int64_t n_nodes; int64_t n_edge_rows;
  /* weights */
  const float *time_w;
  orca_attn_weights_t attn[2];
  orca_score_weights_t score;
  orca_gru_weights_t gru;
  int32_t n_layers; int32_t k;
  /* state */
  orca_memory_t mem;
  float *hist_emb;          /* [n_nodes,172] (n_layers == 2) */
  uint8_t *cache_flag;      /* [n_nodes]                     */
  int32_t *prev_plan;       /* [plan_cap] device copy of the plan whose flags are set */
  int32_t *n_prev_plan;     /* host-resident counter owned by the caller              */
  int32_t plan_cap;
  int64_t *last_pos;        /* [3 * n_nodes] last-occurrence records, zero-initialised once: push  */
                            /* winners of even / odd batches, message winners                     */
  int64_t *epoch_base;      /* host-resident counter owned by the caller              */
  int32_t rank, world;      /* orca_tgn_eval_batch_sharded only; world <= 1 means one GPU */
  uint32_t *cand_bitmap;    /* (n_nodes+31)/32 + 1 + ORCA_CAND_CAP words (candidate bitmap, list    */
                            /* length, list), zero-initialised once by the caller                */
  int32_t mode;             /* ORCA_MODE_*: which recursion of the embedding module runs        */
  /* Direct exchange of the layer-1 rows between the GPUs of one node (orca_tgn_eval_batch_sharded; all
   * NULL / 0: the caller all-gathers).  peer_rows[r] / peer_flags[r]: rank r's exchange buffer
   * (ORCA_EXCHANGE_SLOTS slots of exchange_cap floats, used in turn) and flag words
   * (int32[ORCA_FLAG_WORDS], zero-initialised) as mapped into THIS process (own rank included, peers
   * through CUDA IPC). */
  float *peer_rows[ORCA_MAX_WORLD];
  int32_t *peer_flags[ORCA_MAX_WORLD];   /* int32[ORCA_FLAG_WORDS] per rank */
  int64_t exchange_cap;
  /* The same for the memory update, which is split by node: of the batch's unique positive nodes (in list
   * order) rank r computes every world-th from r and stores the new memory rows into every rank's buffer
   * peer_gru[q] (2 halves of gru_cap floats, used alternately; gru_cap >= 2 * b * 172); all ranks then write
   * all rows into their replica of the memory table.  All NULL: every rank computes every row. */
  float *peer_gru[ORCA_MAX_WORLD];
  int64_t gru_cap;
  int64_t *exchange_seq;    /* host-resident batch sequence counter owned by the caller (starts at 0) */
  orca_ctx_t *ctx;          /* context of this model; NULL = default context of the current device   */
  void *input_stream;       /* cudaStream_t on which the batch arrays (and the plan) of a call were made */
                            /* ready, e.g. a copy stream; NULL = the call's `stream`.  Only with an    */
                            /* input stream of its own can the index work of a batch run ahead of the  */
                            /* previous batch's kernels on `stream`.                                   */
  /* Split by layer (direct exchange only): 0 = every rank computes its share of both layers' rows.
   * layer1_ranks = a (0 < a < world): ranks 0..a-1 compute layer 1 (row i on rank i % a) and the memory
   * update (node split over the same ranks) and deliver the rows to ALL ranks; ranks a..world-1 compute
   * the top layer and the scores (edge e on rank a + e % (world - a)).  Every rank still applies all
   * rows to its replicas of the history and memory tables.  The two halves of a batch's kernel chain
   * then run on different GPUs, a batch apart. */
  int32_t layer1_ranks;
} orca_tgn_t;

/* Workspace sizing: bytes needed for batches of up to b_cap edges with at most u_cap uncached
 * neighbours per batch. */
int64_t orca_eval_workspace_bytes(int32_t b_cap, int32_t u_cap, int32_t k, int64_t n_nodes);
/* Byte offset, inside a workspace of those parameters, of the layer-1 row list (int32 node ids:
 * [src | dst | neg | uncached]) of the index-buffer set `parity` (0 or 1; orca_ctx_last_parity tells
 * which one the last batch used).  For tests and debugging. */
int64_t orca_eval_workspace_row_list(int32_t b_cap, int32_t u_cap, int32_t k, int64_t n_nodes, int32_t parity);

/* d_batch_i32: [src | dst | neg | eidx] (4*b int32), d_batch_ts: [b] float64, d_plan: ids of the
 * batch's cache plan (NULL = plan-less flag rule).  Outputs: d_prob [2*b] = [pos | neg] and, if
 * non-NULL, d_emb_out [3*b,172] = [src | dst | neg] embeddings.  d_status: int32[4] device words
 * (0 = ok; see orca_read_status). */
int orca_tgn_eval_batch(const orca_tgn_t *m, const int32_t *d_batch_i32, const double *d_batch_ts,
                        int32_t b, const int32_t *d_plan, int32_t n_plan, int32_t u_cap,
                        void *d_workspace, int64_t workspace_bytes, float *d_prob,
                        float *d_emb_out, int32_t *d_status, void *stream);

/* ------------------------------------------------------------------------------------------
 * The same batch with its rows split over `world` GPUs of one node (no counterpart in the reference,
 * which is single-device).  Every rank holds a full replica of the graph, the tables and the weights
 * and receives the full batch.  Index work (top-level sampling, uncached set, last occurrences) and the
 * raw-message / GRU chain are replicated -- they are cheap and keep every replica identical -- while
 * the two attention layers and the scorer are sharded:
 *   phase 0: both phases in one call (only with the direct exchange, where the library moves the rows).
 *   phase 1: layer-1 row i of [src|dst|neg|U] belongs to rank i % world; a rank computes its rows
 *            into d_emb1_local [rows_per_rank, 172], rows_per_rank = ceil((3b + u_cap) / world),
 *            local slot i / world.
 *   -- the caller all-gathers d_emb1_local into d_emb1_all [world, rows_per_rank, 172] (NCCL) --
 *   phase 2: every rank pushes ALL layer-1 rows into its history replica, sets the cache flags, then
 *            computes the top layer and the link scores of its edges (edge e belongs to rank
 *            e % world, local slot e / world): d_prob_local [2 * b_local] = [pos | neg] and, if
 *            non-NULL, d_emb2_local [3 * b_local, 172] = [src | dst | neg], b_local = number of local
 *            edges = (b - rank + world - 1) / world.
 * Workspace: orca_eval_workspace_bytes (same size as the single-GPU call).
 */
int orca_tgn_eval_batch_sharded(const orca_tgn_t *m, int32_t phase, const int32_t *d_batch_i32,
                                const double *d_batch_ts, int32_t b, const int32_t *d_plan, int32_t n_plan,
                                int32_t u_cap, void *d_workspace, int64_t workspace_bytes,
                                float *d_emb1_local, const float *d_emb1_all, float *d_prob_local,
                                float *d_emb2_local, int32_t *d_status, void *stream);

/* ------------------------------------------------------------------------------------------
 * A whole stream of batches in one call: the loop of evaluation/evaluation.py:18-37 (one
 * compute_edge_probabilities per batch, scores brought back to the host) without a host round trip per
 * batch.  The batches lie packed in PINNED host memory; the call enqueues, per batch, the host-to-device
 * copy of its arrays (on a copy stream of the model's context, into a ring of 4 staging slots, ahead of the
 * kernels), the batch itself (orca_tgn_eval_batch, or both phases of orca_tgn_eval_batch_sharded when
 * m->world > 1 with the direct exchange) and the device-to-host copy of its scores.  Nothing is
 * synchronised: the scores are complete in `stream` order.
 *   h_i32 + off_i32[i]  [src | dst | neg | eidx | plan] of batch i: 4*b[i] + max(n_plan[i], 0) int32
 *   h_ts + off_ts[i]    b[i] float64
 *   n_plan[i] < 0       batch i has no plan (the cumulative flag rule of modules/history.py:29-30)
 *   off_prob[i]         where batch i's scores go in d_prob / h_prob (floats): [pos | neg], 2*b[i] of them, or
 *                       2*b_local of this rank's edges when sharded (edge e belongs to rank e % world)
 * d_stage: device memory for the staging ring, 4 slots of stage_bytes/4 each (a slot holds one batch:
 * 16*b + 4*n_plan + 8*b bytes, rounded up to 256).  d_prob: device floats; h_prob (pinned, may be NULL):
 * the same layout on the host.  The workspace must be sized for the largest batch.
 */
typedef struct {
  const int32_t *h_i32;
  const double *h_ts;
  const int64_t *off_i32, *off_ts, *off_prob;
  const int32_t *b, *n_plan;
  int64_t n_batches;
} orca_epoch_t;
int orca_tgn_eval_epoch(const orca_tgn_t *m, const orca_epoch_t *e, int32_t u_cap, void *d_workspace,
                        int64_t workspace_bytes, void *d_stage, int64_t stage_bytes, float *d_prob, float *h_prob,
                        int32_t *d_status, void *stream);

/* Sharing the exchange buffer of the multi-GPU split between the processes of one node (no counterpart
 * in the reference).  orca_ipc_export: the 64-byte CUDA IPC handle of the allocation that holds d_ptr and
 * d_ptr's offset inside it; orca_ipc_open (in another process, on its own GPU): the address of the same
 * memory there, with peer access enabled.  A handle may be opened once per process. */
int orca_ipc_export(const void *d_ptr, void *h_handle64, int64_t *h_offset);
int orca_ipc_open(const void *h_handle64, int64_t offset, void **h_ptr_out);
/* unmaps what orca_ipc_open returned (same offset) */
int orca_ipc_close(void *h_ptr, int64_t offset);

/* Asynchronous copy of a staged batch from pinned host memory to the device on `stream` (what
 * `tensor.to(device)` does for the batch arrays in evaluation/evaluation.py:34 of the reference; here
 * one copy per batch). */
int orca_stage_h2d(void *d_dst, const void *h_src, int64_t bytes, void *stream);

/* Phase tracing of the batch entry points (the reference only has wall-clock deltas around whole
 * epochs, train.py:189-341): while ORCA_OPT_TRACE is on, CUDA events are recorded at the phase
 * boundaries of every batch; orca_trace_read synchronises on them, returns the summed milliseconds per
 * phase (orca_trace_phases() entries, names from orca_trace_phase_name) and forgets them. */
int orca_trace_phases(void);
const char *orca_trace_phase_name(int32_t phase);
int orca_trace_read(orca_ctx_t *ctx, double *h_ms_per_phase);

/* Copies the device status words to the host (synchronises `stream`), returns the first nonzero
 * code and resets the device words. h_counts (may be NULL) receives {status, n_layer1_rows,
 * n_unique_positives, kernels launched by the last batch}. */
int orca_read_status(orca_ctx_t *ctx, int32_t *d_status, int32_t *h_counts, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ORCA_B200_H */
