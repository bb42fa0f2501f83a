// State-table kernels: historical-embedding cache (pull / push / flags) and raw-message build.
// All of them move 688-byte rows with 128-bit accesses; a row is handled by 43 lanes of a 64-lane
// group so that four rows share a 256-thread block.
#include <algorithm>

#include "common.cuh"

namespace orca {

constexpr int ROW_F4 = D / 4;  // 43

__global__ void pull_rows_kernel(const float *__restrict__ table, const int32_t *__restrict__ ids, int64_t n,
                                 float *__restrict__ out) {
  const int64_t row = (int64_t)blockIdx.x * 4 + threadIdx.x / 64;
  const int t = threadIdx.x % 64;
  if (row >= n || t >= ROW_F4) return;
  reinterpret_cast<float4 *>(out + row * D)[t] =
      __ldg(reinterpret_cast<const float4 *>(table + (size_t)ids[row] * D) + t);
}

__global__ void push_rows_kernel(float *__restrict__ table, const float *__restrict__ x,
                                 const int32_t *__restrict__ ids, const uint8_t *__restrict__ win, int n_cap,
                                 const int32_t *d_n) {
  const int n = rows_of(n_cap, d_n);
  const int row = blockIdx.x * 4 + threadIdx.x / 64;
  const int t = threadIdx.x % 64;
  if (row >= n || t >= ROW_F4 || win[row] == 0) return;
  reinterpret_cast<float4 *>(table + (size_t)ids[row] * D)[t] =
      reinterpret_cast<const float4 *>(x + (size_t)row * D)[t];
}

__global__ void set_flags_kernel(uint8_t *__restrict__ flag, int64_t n_nodes, const int32_t *__restrict__ ids,
                                 int n, uint8_t value) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int v = ids[i];
    if (v >= 0 && v < n_nodes) flag[v] = value;
  }
}

// One 256-thread block per winner position: the four 172-float quarters of the message are
// produced by four 64-lane groups (memory of the node, memory of the other endpoint, edge
// features, time encoding of the gap since the node's last update).
__global__ void __launch_bounds__(256)
message_store_kernel(orca_memory_t mem, const float *__restrict__ edge_table, const float *__restrict__ time_w,
                     const int32_t *__restrict__ cat_src, const int32_t *__restrict__ cat_dst,
                     const double *__restrict__ ts, const int32_t *__restrict__ eidx, int b,
                     const int32_t *__restrict__ win_pos, int n_cap, const int32_t *d_n,
                     int32_t *__restrict__ win_nodes) {
  dep_trigger();
  dep_wait();
  const int n = rows_of(n_cap, d_n);
  const int w = blockIdx.x;
  if (w >= n) return;
  const int p = win_pos[w];
  const int node = cat_src[p];
  const int other = cat_dst[p];
  const int e = eidx[p % b];
  const float t = (float)ts[p % b];
  const int part = threadIdx.x / 64, lane = threadIdx.x % 64;
  float *dst = mem.messages + (size_t)node * MSG + part * D;
  if (part < 3) {
    const float *src = part == 0 ? mem.memory + (size_t)node * D
                     : part == 1 ? mem.memory + (size_t)other * D
                                 : edge_table + (size_t)e * D;
    if (lane < ROW_F4) reinterpret_cast<float4 *>(dst)[lane] = reinterpret_cast<const float4 *>(src)[lane];
  } else {
    const float gap = t - mem.last_update[node];
    for (int d = lane; d < D; d += 64) dst[d] = cos_any(gap * __ldg(time_w + d));
  }
  if (threadIdx.x == 0) {
    mem.msg_ts[node] = t;
    mem.msg_flag[node] = 1;
    if (win_nodes) win_nodes[w] = node;
  }
}

}  // namespace orca

using namespace orca;

extern "C" {

int orca_history_pull(const float *d_emb, const int32_t *d_ids, int64_t n, float *d_out, void *stream) {
  ORCA_CHECK_ARG(d_emb && d_ids && d_out && n >= 0);
  if (n == 0) return ORCA_OK;
  pull_rows_kernel<<<(unsigned)((n + 3) / 4), 256, 0, (cudaStream_t)stream>>>(d_emb, d_ids, n, d_out);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_history_push(float *d_emb, const float *d_x, const int32_t *d_ids, const uint8_t *d_win,
                      int32_t n_cap, const int32_t *d_n, void *stream) {
  ORCA_CHECK_ARG(d_emb && d_x && d_ids && d_win && n_cap >= 0);
  if (n_cap == 0) return ORCA_OK;
  push_rows_kernel<<<ceil_div(n_cap, 4), 256, 0, (cudaStream_t)stream>>>(d_emb, d_x, d_ids, d_win, n_cap, d_n);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_history_set_flags(uint8_t *d_cache_flag, int64_t n_nodes, const int32_t *d_prev_plan,
                           int32_t n_prev, const int32_t *d_plan, int32_t n_plan, void *stream) {
  ORCA_CHECK_ARG(d_cache_flag && n_nodes > 0 && n_prev >= 0 && n_plan >= 0);
  cudaStream_t s = (cudaStream_t)stream;
  if (d_prev_plan == nullptr) {
    ORCA_CUDA(cudaMemsetAsync(d_cache_flag, 0, (size_t)n_nodes, s));
  } else if (n_prev > 0) {
    set_flags_kernel<<<std::min(ceil_div(n_prev, 256), 1024), 256, 0, s>>>(d_cache_flag, n_nodes, d_prev_plan,
                                                                           n_prev, 0);
    ORCA_COUNT_LAUNCH();
  }
  if (d_plan != nullptr && n_plan > 0) {
    set_flags_kernel<<<std::min(ceil_div(n_plan, 256), 1024), 256, 0, s>>>(d_cache_flag, n_nodes, d_plan,
                                                                           n_plan, 1);
    ORCA_COUNT_LAUNCH();
  }
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_message_store(const orca_memory_t *mem, const float *d_edge_table, const float *d_time_w,
                       const int32_t *d_cat_src, const int32_t *d_cat_dst, const double *d_ts,
                       const int32_t *d_eidx, int32_t b, const int32_t *d_win_pos, int32_t n_win_cap,
                       const int32_t *d_n_win, int32_t *d_win_nodes, void *stream) {
  ORCA_CHECK_ARG(mem && mem->memory && mem->last_update && mem->messages && mem->msg_ts && mem->msg_flag);
  ORCA_CHECK_ARG(d_edge_table && d_time_w && d_cat_src && d_cat_dst && d_ts && d_eidx && d_win_pos);
  ORCA_CHECK_ARG(b >= 0 && n_win_cap >= 0);
  if (n_win_cap == 0 || b == 0) return ORCA_OK;
  ORCA_CUDA(launch_dep(message_store_kernel, n_win_cap, 256, 0, (cudaStream_t)stream, *mem, d_edge_table, d_time_w,
                       d_cat_src, d_cat_dst, d_ts, d_eidx, b, d_win_pos, n_win_cap, d_n_win, d_win_nodes));
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // extern "C"
