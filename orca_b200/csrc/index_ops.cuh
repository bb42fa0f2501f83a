// Launchers shared between the translation units of the batch pipeline.
#pragma once

#include "common.cuh"

namespace orca {

// rows [src | dst | neg] of the batch with their query times, the [dst | src] partner list, the
// neighbour table of those rows, candidate marking (bitmap + list) and the last-occurrence record of
// every row's node in d_last_pos (record = base + row)
int launch_batch_head(const orca_tgn_t *m, const int32_t *d_batch, const double *d_bts, int b, int32_t *nodes1,
                      double *ts1, int32_t *cat_dst, int32_t *o_nbr, int32_t *o_eid, float *o_dt, int32_t *status,
                      int64_t *d_last_pos, long long base, cudaStream_t s);

// appends the uncached set to the row list: *d_n_total = n_query + |U|, *d_n_unc = |U|; d_last_pos / base:
// the records launch_batch_head made for the batch rows
int launch_uncached_finish(const orca_tgn_t *m, int n_query, int32_t *nodes_io, double *ts_io, int u_cap,
                           int32_t *d_n_total, int32_t *d_n_unc, int32_t *status, const int64_t *d_last_pos,
                           long long base, cudaStream_t s);

// positions of the last occurrence of every id, in position order (single block; n up to a few
// thousand); d_status (optional): the count is also written to status word 2
int launch_last_occ_compact(const int32_t *d_ids, int n, int64_t n_nodes, int64_t *d_last_pos, long long base,
                            int32_t *d_compact, int32_t *d_n_compact, int32_t *d_status, cudaStream_t s);

// the fused gather-attention kernel (attention.cu); d_ticket: two zeroed device words that the launch
// leaves at zero (launches that may overlap on the GPU need words of their own); rows_hint > 0: the live
// row count the caller expects (n_rows_cap is a capacity); d_order (optional): the row ids in the order the
// warps should take them (launch_row_order)
int launch_attn_gather(const float *d_qt, const float *d_nbr_table, const float *d_edge_table,
                       const float *d_time_w, const int32_t *d_nbr, const int32_t *d_eid, const float *d_delta,
                       int k, int n_rows_cap, const int32_t *d_n_rows, int rows_hint, const int32_t *d_order,
                       float *d_ctx, uint8_t *d_valid, int32_t *d_ticket, cudaStream_t stream);
// rows of two neighbour tables sorted by falling number of valid slots (one launch, one block per table)
int launch_row_order(const int32_t *d_nbr_a, int n_cap_a, const int32_t *d_n_a, int32_t *d_order_a,
                     const int32_t *d_nbr_b, int n_cap_b, const int32_t *d_n_b, int32_t *d_order_b, int k,
                     cudaStream_t stream);

// the two halves of orca_gru_update (gemm.cu): the projection + gates into d_scratch_h reads the tables
// only; the scatter writes memory / last_update and clears the message flags
// (peer, multi-GPU: this rank computes every world-th listed node from its rank and stores the rows into
// every rank's buffer peer->rows[q] + peer->off instead of d_scratch_h, then posts peer->seq; split > 0: the
// nodes are split over the first `split` ranks only, the rows still go to all peer->world ranks)
namespace tc { struct PeerOut; }
int gru_project(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes, int32_t n_cap,
                const int32_t *d_n, float *d_scratch_h, cudaStream_t s, const tc::PeerOut *peer = nullptr,
                int split = 0);
// (d_skip_if_set, optional: a device status word; the scatter leaves the table alone when it is non-zero)
int gru_scatter(const orca_memory_t *mem, const int32_t *d_nodes, int32_t n_cap, const int32_t *d_n,
                int32_t clear_flags, const float *d_scratch_h, cudaStream_t s, const int32_t *d_skip_if_set = nullptr);

}  // namespace orca
