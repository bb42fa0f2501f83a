// Launchers of the fused index kernels of the eval batch (sampler.cu), used by the batch pipeline.
#pragma once

#include "common.cuh"

namespace orca {

// rows [src | dst | neg] of the batch with their query times, the [dst | src] partner list, the
// neighbour table of those rows, candidate marking (bitmap + list) and the last-occurrence record
int launch_batch_head(const orca_tgn_t *m, const int32_t *d_batch, const double *d_bts, int b, int32_t *nodes1,
                      double *ts1, int32_t *cat_dst, int32_t *o_nbr, int32_t *o_eid, float *o_dt, int32_t *status,
                      long long base, cudaStream_t s);

// appends the uncached set to the row list: *d_n_total = n_query + |U|, *d_n_unc = |U|; `base` is the
// epoch base that launch_batch_head recorded the batch rows with
int launch_uncached_finish(const orca_tgn_t *m, int n_query, int32_t *nodes_io, double *ts_io, int u_cap,
                           int32_t *d_n_total, int32_t *d_n_unc, int32_t *status, long long base, cudaStream_t s);

// positions of the last occurrence of every id, in position order (single block; n up to a few
// thousand); d_status (optional): the count is also written to status word 2.  With d_flag given the
// block first applies History.update_flag for the plan (clear d_prev_plan[0..n_prev), set
// d_plan[0..n_plan), copy the plan to d_prev_plan).
int launch_last_occ_compact(const int32_t *d_ids, int n, int64_t n_nodes, int64_t *d_last_pos, long long base,
                            int32_t *d_compact, int32_t *d_n_compact, int32_t *d_status, uint8_t *d_flag,
                            int32_t *d_prev_plan, int n_prev, const int32_t *d_plan, int n_plan, cudaStream_t s);

}  // namespace orca
