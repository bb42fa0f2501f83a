// Dense projections of the path, fp32 SIMT tiles with gathered A rows and fused epilogues:
//   attn_query   qt  = feat[idx] . Mq + cq
//   attn_output  out = LN(relu([ctx | feat[idx]] . G + b1 + valid*g) . W2t + b2), optional history push
//   score        p   = sigmoid(relu([emb_a | emb_b] . W1t + b1) . w2 + b2)
//   gru          h'  = GRU([message | memory]) with the four gate columns of a unit adjacent
#include <algorithm>

#include "common.cuh"
#include "context.cuh"
#include "index_ops.cuh"
#include "tc_gemm.cuh"

namespace orca {

// ---------------------------------------------------------------------------------------------
// A-row sources: a logical A row is the concatenation of up to two gathered rows.
// ---------------------------------------------------------------------------------------------
struct RowSrc {
  const float *p;      // table base, row stride = width floats
  const int32_t *idx;  // row m reads table row idx[m] (or m + add if idx == nullptr)
  int width;
  int mod;             // if > 0 and idx == nullptr: table row = m % mod + add
  int add;
};

__device__ __forceinline__ const float *src_row(const RowSrc &s, int m) {
  int r;
  if (s.idx) r = s.idx[m];
  else r = (s.mod > 0 ? m % s.mod : m) + s.add;
  return s.p + (size_t)r * s.width;
}

// ---------------------------------------------------------------------------------------------
// F1: C[m_cap, Nc] tiles of 64 x 64, BK = 16, 256 threads, 4 x 4 outputs per thread.
// ---------------------------------------------------------------------------------------------
constexpr int F1_BM = 64, F1_BN = 64, F1_BK = 16, F1_THREADS = 256;

struct F1Args {
  RowSrc a0, a1;  // a1.width == 0 when unused
  int Kd;
  const float *B;  // [Kd, Nc]
  int Nc;
  const float *bias;  // [Nc]
  int m_cap;
  const int32_t *d_m;
  float *C;  // EPI_BIAS: [m_cap, Nc]; EPI_GRU: scratch h' [m_cap, D]
  // GRU extras
  const float *memory;
  const int32_t *nodes;
};

enum { EPI_BIAS = 0, EPI_GRU = 1 };

template <int EPI>
__global__ void __launch_bounds__(F1_THREADS) f1_gemm_kernel(F1Args g) {
  __shared__ float As[2][F1_BK][F1_BM + 4];
  __shared__ __align__(16) float Bs[2][F1_BK][F1_BN];
  const int M = rows_of(g.m_cap, g.d_m);
  const int n0 = blockIdx.x * F1_BN;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;
  // row tiles are strided over gridDim.y so that a large capacity costs no idle blocks
  for (int m0 = blockIdx.y * F1_BM; m0 < M; m0 += gridDim.y * F1_BM) {

  // loader coordinates
  const int ar = tid / 4, akq = (tid % 4) * 4;
  const int am = m0 + ar;
  const float *arow0 = nullptr, *arow1 = nullptr;
  if (am < M) {
    arow0 = src_row(g.a0, am);
    if (g.a1.width) arow1 = src_row(g.a1, am);
  }
  const int bk = tid / 16, bc = (tid % 16) * 4;

  auto load_a = [&](int k0) -> float4 {
    const int col = k0 + akq;
    if (arow0 == nullptr || col >= g.Kd) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < g.a0.width) return *reinterpret_cast<const float4 *>(arow0 + col);
    return *reinterpret_cast<const float4 *>(arow1 + (col - g.a0.width));
  };
  auto load_b = [&](int k0) -> float4 {
    const int kr = k0 + bk, col = n0 + bc;
    if (kr >= g.Kd || col >= g.Nc) return make_float4(0.f, 0.f, 0.f, 0.f);
    return __ldg(reinterpret_cast<const float4 *>(g.B + (size_t)kr * g.Nc + col));
  };
  auto stash = [&](int buf, float4 a, float4 b) {
    As[buf][akq + 0][ar] = a.x;
    As[buf][akq + 1][ar] = a.y;
    As[buf][akq + 2][ar] = a.z;
    As[buf][akq + 3][ar] = a.w;
    *reinterpret_cast<float4 *>(&Bs[buf][bk][bc]) = b;
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int n_k = (g.Kd + F1_BK - 1) / F1_BK;
  float4 ra = load_a(0), rb = load_b(0);
  stash(0, ra, rb);
  __syncthreads();
  for (int kt = 0; kt < n_k; ++kt) {
    const int cur = kt & 1;
    if (kt + 1 < n_k) {
      ra = load_a((kt + 1) * F1_BK);
      rb = load_b((kt + 1) * F1_BK);
    }
#pragma unroll
    for (int kk = 0; kk < F1_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[cur][kk][ty * 4 + i];
      const float4 bv = *reinterpret_cast<const float4 *>(&Bs[cur][kk][tx * 4]);
      b[0] = bv.x; b[1] = bv.y; b[2] = bv.z; b[3] = bv.w;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < n_k) {
      stash(cur ^ 1, ra, rb);
      __syncthreads();
    }
  }

  __syncthreads();
  const int col0 = n0 + tx * 4;
  if (col0 >= g.Nc) continue;
  const float4 bias = __ldg(reinterpret_cast<const float4 *>(g.bias + col0));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    if (EPI == EPI_BIAS) {
      float4 o = make_float4(acc[i][0] + bias.x, acc[i][1] + bias.y, acc[i][2] + bias.z, acc[i][3] + bias.w);
      *reinterpret_cast<float4 *>(g.C + (size_t)m * g.Nc + col0) = o;
    } else {
      // columns col0..col0+3 are (r, z, n_input, n_hidden) of unit j
      const int j = col0 / 4;
      const float hp = g.memory[(size_t)g.nodes[m] * D + j];
      const float r = 1.f / (1.f + expf(-(acc[i][0] + bias.x)));
      const float z = 1.f / (1.f + expf(-(acc[i][1] + bias.y)));
      const float nn = tanhf((acc[i][2] + bias.z) + r * (acc[i][3] + bias.w));
      g.C[(size_t)m * D + j] = (1.f - z) * nn + z * hp;
    }
  }
  }  // row tiles
}

// ---------------------------------------------------------------------------------------------
// F2: full-row tiles, 32 rows x 176 columns (172 used), 256 threads: thread (ty, tx) owns rows
// 2*ty, 2*ty+1 and columns tx + 16*j, j < 11, so a row lives in one half-warp and row reductions
// (LayerNorm, the scorer's dot product) are four shuffles.
// ---------------------------------------------------------------------------------------------
constexpr int F2_BM = 32, F2_BN = 176, F2_BK = 16, F2_THREADS = 256, F2_J = 11;

struct F2Smem {
  float As[F2_BK][F2_BM + 1];
  float Bs[F2_BK][F2_BN];
  float Hs[F2_BM][F2_BN + 1];
};

// acc += A[32, Kd] . B[Kd, 172]; afetch(r, col) returns 4 consecutive A values of tile row r
template <class AFetch>
__device__ __forceinline__ void f2_mainloop(F2Smem &s, AFetch afetch, const float *__restrict__ B, int Kd,
                                            float (&acc)[2][F2_J]) {
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int n_k = (Kd + F2_BK - 1) / F2_BK;
  for (int kt = 0; kt < n_k; ++kt) {
    const int k0 = kt * F2_BK;
    if (tid < 128) {
      const int r = tid / 4, kq = (tid % 4) * 4;
      const float4 a = (k0 + kq < Kd) ? afetch(r, k0 + kq) : make_float4(0.f, 0.f, 0.f, 0.f);
      s.As[kq + 0][r] = a.x;
      s.As[kq + 1][r] = a.y;
      s.As[kq + 2][r] = a.z;
      s.As[kq + 3][r] = a.w;
    }
    for (int i = tid; i < F2_BK * (F2_BN / 4); i += F2_THREADS) {
      const int kr = i / (F2_BN / 4), c4 = (i % (F2_BN / 4)) * 4;
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k0 + kr < Kd && c4 < D) b = __ldg(reinterpret_cast<const float4 *>(B + (size_t)(k0 + kr) * D + c4));
      *reinterpret_cast<float4 *>(&s.Bs[kr][c4]) = b;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < F2_BK; ++kk) {
      const float a0 = s.As[kk][ty * 2], a1 = s.As[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < F2_J; ++j) {
        const float b = s.Bs[kk][tx + 16 * j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
}

__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct OutArgs {
  orca_attn_weights_t w;
  const float *ctx;
  const uint8_t *valid;
  RowSrc feat;
  int m_cap;
  const int32_t *d_m;
  float *out;
  float *push_table;
  const int32_t *push_ids;
  const uint8_t *push_win;
};

__global__ void __launch_bounds__(F2_THREADS) attn_output_kernel(OutArgs g) {
  extern __shared__ __align__(16) unsigned char raw[];
  F2Smem &s = *reinterpret_cast<F2Smem *>(raw);
  const int M = rows_of(g.m_cap, g.d_m);
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  for (int m0 = blockIdx.x * F2_BM; m0 < M; m0 += gridDim.x * F2_BM) {

  float acc[2][F2_J];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < F2_J; ++j) acc[i][j] = 0.f;

  // phase 1: hidden = relu([ctx | feat] . G + b1 + valid * g)
  {
    const int r = tid / 4;
    const int m = m0 + r;
    const bool live = tid < 128 && m < M;
    const bool val = live && g.valid[m] != 0;
    const float *crow = live ? g.ctx + (size_t)m * QT : nullptr;
    const float *frow = live ? src_row(g.feat, m) : nullptr;
    auto afetch = [&](int, int col) -> float4 {
      if (!live) return make_float4(0.f, 0.f, 0.f, 0.f);
      if (col < QT) return val ? *reinterpret_cast<const float4 *>(crow + col) : make_float4(0.f, 0.f, 0.f, 0.f);
      return *reinterpret_cast<const float4 *>(frow + (col - QT));
    };
    f2_mainloop(s, afetch, g.w.G, QT + D, acc);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    const int m = m0 + r;
    const float v = (m < M && g.valid[m] != 0) ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < F2_J; ++j) {
      const int c = tx + 16 * j;
      float h = 0.f;
      if (c < D) h = fmaxf(acc[i][j] + __ldg(g.w.b1 + c) + v * __ldg(g.w.g + c), 0.f);
      s.Hs[r][c] = h;
      acc[i][j] = 0.f;
    }
  }
  __syncthreads();
  // phase 2: y = hidden . W2t + b2
  {
    auto afetch = [&](int r, int col) -> float4 {
      return make_float4(s.Hs[r][col], s.Hs[r][col + 1], s.Hs[r][col + 2], s.Hs[r][col + 3]);
    };
    f2_mainloop(s, afetch, g.w.W2t, D, acc);
  }
  // LayerNorm over the 172 columns of each row (two-pass mean / variance)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + ty * 2 + i;
    float y[F2_J];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < F2_J; ++j) {
      const int c = tx + 16 * j;
      y[j] = (c < D) ? acc[i][j] + __ldg(g.w.b2 + c) : 0.f;
      sum += y[j];
    }
    const float mean = half_warp_sum(sum) * (1.f / D);
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < F2_J; ++j) {
      const int c = tx + 16 * j;
      const float d = (c < D) ? y[j] - mean : 0.f;
      sq += d * d;
    }
    const float var = half_warp_sum(sq) * (1.f / D);
    const float inv = 1.f / sqrtf(var + 1e-5f);
    if (m < M) {
      const bool push = g.push_table != nullptr && g.push_win[m] != 0;
      float *prow = push ? g.push_table + (size_t)g.push_ids[m] * D : nullptr;
#pragma unroll
      for (int j = 0; j < F2_J; ++j) {
        const int c = tx + 16 * j;
        if (c < D) {
          const float o = (y[j] - mean) * inv * __ldg(g.w.ln_w + c) + __ldg(g.w.ln_b + c);
          g.out[(size_t)m * D + c] = o;
          if (push) prow[c] = o;
        }
      }
    }
  }
  __syncthreads();
  }  // row tiles
}

struct ScoreArgs {
  orca_score_weights_t w;
  const float *emb;
  int b;
  float *prob;
};

__global__ void __launch_bounds__(F2_THREADS) score_kernel(ScoreArgs g) {
  extern __shared__ __align__(16) unsigned char raw[];
  F2Smem &s = *reinterpret_cast<F2Smem *>(raw);
  const int M = 2 * g.b;
  const int m0 = blockIdx.x * F2_BM;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[2][F2_J];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < F2_J; ++j) acc[i][j] = 0.f;
  {
    const int r = tid / 4;
    const int m = m0 + r;
    const bool live = tid < 128 && m < M;
    // row m < b pairs (src m, dst m); row m >= b pairs (src m-b, neg m-b): rows m % b and b + m
    const float *arow = live ? g.emb + (size_t)(m % g.b) * D : nullptr;
    const float *brow = live ? g.emb + (size_t)(g.b + m) * D : nullptr;
    auto afetch = [&](int, int col) -> float4 {
      if (!live) return make_float4(0.f, 0.f, 0.f, 0.f);
      if (col < D) return *reinterpret_cast<const float4 *>(arow + col);
      return *reinterpret_cast<const float4 *>(brow + (col - D));
    };
    f2_mainloop(s, afetch, g.w.W1t, 2 * D, acc);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + ty * 2 + i;
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < F2_J; ++j) {
      const int c = tx + 16 * j;
      if (c < D) part += fmaxf(acc[i][j] + __ldg(g.w.b1 + c), 0.f) * __ldg(g.w.w2 + c);
    }
    const float z = half_warp_sum(part) + g.w.b2;
    if (tx == 0 && m < M) g.prob[m] = 1.f / (1.f + expf(-z));
  }
}

// scatter of the GRU result: memory[node] = h', last_update[node] = msg_ts[node], and -- optionally --
// the message flag of the node is cleared once every lane of the row has seen it set (a listed node
// without a pending message is left alone)
__global__ void gru_scatter_kernel(const float *__restrict__ hnew, orca_memory_t mem,
                                   const int32_t *__restrict__ nodes, int n_cap, const int32_t *d_n,
                                   int clear_flags, const int32_t *__restrict__ status) {
  dep_trigger();
  dep_wait();
  // (multi-GPU: rows that the peers did not deliver in time must not reach the memory table)
  if (status != nullptr && *status != 0) return;
  const int n = rows_of(n_cap, d_n);
  const int row = blockIdx.x * (blockDim.x / 64) + threadIdx.x / 64;
  const int t = threadIdx.x % 64;
  int node = 0;
  bool pending = false;
  if (row < n) {
    node = nodes[row];
    pending = mem.msg_flag[node] != 0;
  }
  __syncthreads();
  if (!pending) return;
  if (t < D / 4) {
    reinterpret_cast<float4 *>(mem.memory + (size_t)node * D)[t] =
        reinterpret_cast<const float4 *>(hnew + (size_t)row * D)[t];
  }
  if (t == 63) {
    mem.last_update[node] = mem.msg_ts[node];
    if (clear_flags) mem.msg_flag[node] = 0;
  }
}

}  // namespace orca

using namespace orca;

// projection kernels of the context in effect: 0 = tensor cores (bf16 head/tail split), 1 = fp32 SIMT tiles
static int projection_mode() {
  Ctx *c = cur();
  return c != nullptr ? c->projection_mode : 0;
}
static int sm_count() {
  Ctx *c = cur();
  return c != nullptr ? c->sm_count : 148;
}

static int ensure_f2_smem() {
  static thread_local int configured_device = -1;
  int dev = 0;
  ORCA_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    ORCA_CUDA(cudaFuncSetAttribute(attn_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(F2Smem)));
    ORCA_CUDA(cudaFuncSetAttribute(score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)sizeof(F2Smem)));
    configured_device = dev;
  }
  return ORCA_OK;
}

static inline int kblocks(int k) { return (k + tc::BK - 1) / tc::BK; }

extern "C" {

int orca_attn_query(const orca_attn_weights_t *w, const float *d_feat, const int32_t *d_idx,
                    int32_t n_rows_cap, const int32_t *d_n_rows, float *d_qt, void *stream) {
  ORCA_CHECK_ARG(w && w->Mq && w->cq && d_feat && d_qt && n_rows_cap >= 0);
  if (n_rows_cap == 0) return ORCA_OK;
  if (projection_mode() == 0) {
    ORCA_CHECK_ARG(w->Mq_tc != nullptr);
    tc::Args a{};
    a.a0 = tc::RowSrc{d_feat, d_idx, D, 0, 0};
    a.Kd = D;
    a.w_packed = w->Mq_tc;
    a.n_kblocks = kblocks(D);
    a.m_cap = n_rows_cap;
    a.d_m = d_n_rows;
    a.bias = w->cq;
    a.out = d_qt;
    a.out_ld = QT_LD;
    return tc::launch(tc::EPI_BIAS, a, QT_LD / tc::BN, (cudaStream_t)stream);
  }
  F1Args g{};
  g.a0 = RowSrc{d_feat, d_idx, D, 0, 0};
  g.a1 = RowSrc{nullptr, nullptr, 0, 0, 0};
  g.Kd = D;
  g.B = w->Mq;
  g.Nc = QT_LD;
  g.bias = w->cq;
  g.m_cap = n_rows_cap;
  g.d_m = d_n_rows;
  g.C = d_qt;
  dim3 grid(ceil_div(QT_LD, F1_BN), std::min(ceil_div(n_rows_cap, F1_BM), sm_count()));
  f1_gemm_kernel<EPI_BIAS><<<grid, F1_THREADS, 0, (cudaStream_t)stream>>>(g);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int orca_attn_output(const orca_attn_weights_t *w, const float *d_ctx, const uint8_t *d_valid,
                     const float *d_feat, const int32_t *d_idx, int32_t n_rows_cap,
                     const int32_t *d_n_rows, float *d_out, float *d_push_table,
                     const int32_t *d_push_ids, const uint8_t *d_push_win, float *d_scratch_hidden,
                     void *stream) {
  ORCA_CHECK_ARG(d_push_table == nullptr || (d_push_ids && d_push_win));
  return orca::attn_output_impl(w, d_ctx, d_valid, d_feat, d_idx, n_rows_cap, d_n_rows, d_out, d_push_table,
                                d_push_ids, d_push_win, nullptr, 0, 0, d_scratch_hidden, 0, (cudaStream_t)stream);
}

}  // extern "C"

namespace orca {

// winners of a push from the last-occurrence records (fp32 debug path only; the tensor-core epilogue
// reads the records itself)
__global__ void win_from_last_pos_kernel(const int32_t *__restrict__ ids, int cap, const int32_t *d_n,
                                         const unsigned long long *__restrict__ last_pos, long long base,
                                         int all_from, uint8_t *__restrict__ win) {
  const int n = rows_of(cap, d_n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    win[i] = (i >= all_from || last_pos[ids[i]] == (unsigned long long)(base + i)) ? 1 : 0;
}

bool projections_on_tensor_cores() { return projection_mode() == 0; }

// d_push_win given: rows with a non-zero byte are pushed.  Otherwise (d_last_pos given) row i is
// pushed when i >= all_from or when last_pos[push_ids[i]] == base + i; `d_push_win` is then only
// scratch for the fp32 debug path and may be NULL in tensor-core mode.  rows_hint (> 0): the live row
// count the caller expects (n_rows_cap is a capacity); it only steers how the work is spread.
int attn_output_impl(const orca_attn_weights_t *w, const float *d_ctx, const uint8_t *d_valid, const float *d_feat,
                     const int32_t *d_idx, int32_t n_rows_cap, const int32_t *d_n_rows, float *d_out,
                     float *d_push_table, const int32_t *d_push_ids, const uint8_t *d_push_win,
                     const int64_t *d_last_pos, long long base, int all_from, float *d_scratch_hidden,
                     int rows_hint, cudaStream_t stream, const tc::PeerOut *peer) {
  ORCA_CHECK_ARG(w && w->G && w->b1 && w->g && w->W2t && w->b2 && w->ln_w && w->ln_b);
  ORCA_CHECK_ARG(d_ctx && d_valid && d_feat && d_out && n_rows_cap >= 0);
  if (n_rows_cap == 0) return ORCA_OK;
  if (projection_mode() != 0 && d_push_table != nullptr && d_last_pos != nullptr) {
    ORCA_CHECK_ARG(d_push_win != nullptr);
    win_from_last_pos_kernel<<<std::min(ceil_div(n_rows_cap, 256), 1024), 256, 0, stream>>>(
        d_push_ids, n_rows_cap, d_n_rows, reinterpret_cast<const unsigned long long *>(d_last_pos), base, all_from,
        const_cast<uint8_t *>(d_push_win));
    ORCA_COUNT_LAUNCH();
    ORCA_LAUNCH_CHECK();
  }
  if (projection_mode() == 0) {
    // (the tensor-core kernel zeroes the whole first source of an invalid row: zero_cols == its width)
    ORCA_CHECK_ARG(w->G_tc && w->W2t_tc);
    // One kernel: relu([ctx | feat] . G + b1 + valid * g) stays on the SM as the A operand of the second
    // product (. W2t + b2), whose epilogue is the LayerNorm with the history push.  (The hidden tile never
    // goes to HBM; d_scratch_hidden is not used in this mode.)
    (void)rows_hint;
    (void)d_scratch_hidden;
    tc::Args a{};
    a.a0 = tc::RowSrc{d_ctx, nullptr, QT, 0, 0};
    a.a1 = tc::RowSrc{d_feat, d_idx, D, 0, 0};
    a.Kd = QT + D;
    a.row_valid = d_valid;
    a.zero_cols = QT;
    a.w_packed = w->G_tc;
    a.n_kblocks = kblocks(QT + D);
    a.m_cap = n_rows_cap;
    a.d_m = d_n_rows;
    a.bias = w->b1;
    a.bias2 = w->g;
    a.w2_packed = w->W2t_tc;
    a.bias_out = w->b2;
    a.ln_w = w->ln_w;
    a.ln_b = w->ln_b;
    a.out = d_out;
    a.push_table = d_push_table;
    a.push_ids = d_push_ids;
    a.push_win = d_last_pos ? nullptr : d_push_win;
    a.push_last_pos = reinterpret_cast<const unsigned long long *>(d_last_pos);
    a.push_base = base;
    a.push_all_from = all_from;
    if (peer != nullptr) a.peer = *peer;
    return tc::launch(tc::EPI_MERGER, a, 1, (cudaStream_t)stream);
  }
  int rc = ensure_f2_smem();
  if (rc) return rc;
  OutArgs g{};
  g.w = *w;
  g.ctx = d_ctx;
  g.valid = d_valid;
  g.feat = RowSrc{d_feat, d_idx, D, 0, 0};
  g.m_cap = n_rows_cap;
  g.d_m = d_n_rows;
  g.out = d_out;
  g.push_table = d_push_table;
  g.push_ids = d_push_ids;
  g.push_win = d_push_win;
  attn_output_kernel<<<std::min(ceil_div(n_rows_cap, F2_BM), sm_count() * 4), F2_THREADS, sizeof(F2Smem), (cudaStream_t)stream>>>(g);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace orca

namespace orca {

int gru_project(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes, int32_t n_cap,
                const int32_t *d_n, float *d_scratch_h, cudaStream_t s, const tc::PeerOut *peer, int split) {
  ORCA_CHECK_ARG(w && w->Wg && w->bg && mem && mem->memory && mem->last_update && mem->messages &&
                 mem->msg_ts && mem->msg_flag && d_nodes && d_scratch_h && n_cap >= 0);
  if (n_cap == 0) return ORCA_OK;
  if (projection_mode() == 0) {
    ORCA_CHECK_ARG(w->Wg_tc != nullptr);
    tc::Args a{};
    a.a0 = tc::RowSrc{mem->messages, d_nodes, MSG, 0, 0};
    a.a1 = tc::RowSrc{mem->memory, d_nodes, D, 0, 0};
    a.Kd = MSG + D;
    a.w_packed = w->Wg_tc;
    a.n_kblocks = kblocks(MSG + D);
    a.m_cap = n_cap;
    a.d_m = d_n;
    a.bias = w->bg;
    a.out = d_scratch_h;
    a.memory = mem->memory;
    a.nodes = d_nodes;
    if (peer != nullptr) {
      // one rank of the multi-GPU split: every world-th listed node from `rank`, rows delivered to all ranks
      a.peer = *peer;
      const int stride = split > 0 ? split : peer->world;
      a.row_stride = stride, a.row_off = peer->rank, a.idx_limit = n_cap;
      a.m_cap = ceil_div(n_cap, stride);
    }
    return tc::launch(tc::EPI_GRU, a, 4, s);
  }
  if (peer != nullptr) return set_error(ORCA_E_UNSUPPORTED, "gru_project: the node split needs the tensor-core path");
  F1Args g{};
  g.a0 = RowSrc{mem->messages, d_nodes, MSG, 0, 0};
  g.a1 = RowSrc{mem->memory, d_nodes, D, 0, 0};
  g.Kd = MSG + D;
  g.B = w->Wg;
  g.Nc = 4 * D;
  g.bias = w->bg;
  g.m_cap = n_cap;
  g.d_m = d_n;
  g.C = d_scratch_h;
  g.memory = mem->memory;
  g.nodes = d_nodes;
  dim3 grid(ceil_div(4 * D, F1_BN), std::min(ceil_div(n_cap, F1_BM), sm_count()));
  f1_gemm_kernel<EPI_GRU><<<grid, F1_THREADS, 0, s>>>(g);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int gru_scatter(const orca_memory_t *mem, const int32_t *d_nodes, int32_t n_cap, const int32_t *d_n,
                int32_t clear_flags, const float *d_scratch_h, cudaStream_t s, const int32_t *d_skip_if_set) {
  ORCA_CHECK_ARG(mem && mem->memory && mem->last_update && mem->msg_ts && mem->msg_flag && d_nodes && d_scratch_h &&
                 n_cap >= 0);
  if (n_cap == 0) return ORCA_OK;
  ORCA_CUDA(launch_dep(gru_scatter_kernel, ceil_div(n_cap, 4), 256, 0, s, d_scratch_h, *mem, d_nodes, n_cap, d_n,
                       (int)clear_flags, d_skip_if_set));
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace orca

extern "C" {

int orca_score(const orca_score_weights_t *w, const float *d_emb, int32_t b, float *d_prob, void *stream) {
  ORCA_CHECK_ARG(w && w->W1t && w->b1 && w->w2 && d_emb && d_prob && b >= 0);
  if (b == 0) return ORCA_OK;
  if (projection_mode() == 0) {
    ORCA_CHECK_ARG(w->W1t_tc != nullptr);
    tc::Args a{};
    // row m < b pairs (src m, dst m); row m >= b pairs (src m-b, neg m-b): table rows m % b and b + m
    a.a0 = tc::RowSrc{d_emb, nullptr, D, b, 0};
    a.a1 = tc::RowSrc{d_emb, nullptr, D, 0, b};
    a.Kd = 2 * D;
    a.w_packed = w->W1t_tc;
    a.n_kblocks = kblocks(2 * D);
    a.m_cap = 2 * b;
    a.bias = w->b1;
    a.w2 = w->w2;
    a.b2 = w->b2;
    a.out = d_prob;
    return tc::launch(tc::EPI_SCORE, a, 1, (cudaStream_t)stream);
  }
  int rc = ensure_f2_smem();
  if (rc) return rc;
  ScoreArgs g{*w, d_emb, b, d_prob};
  score_kernel<<<ceil_div(2 * b, F2_BM), F2_THREADS, sizeof(F2Smem), (cudaStream_t)stream>>>(g);
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

int64_t orca_gru_scratch_bytes(int32_t n_cap) { return (int64_t)(n_cap > 0 ? n_cap : 1) * D * 4; }

int orca_gru_update(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes,
                    int32_t n_cap, const int32_t *d_n, int32_t clear_flags, float *d_scratch_h,
                    void *stream) {
  int rc = orca::gru_project(w, mem, d_nodes, n_cap, d_n, d_scratch_h, (cudaStream_t)stream);
  if (rc) return rc;
  return orca::gru_scatter(mem, d_nodes, n_cap, d_n, clear_flags, d_scratch_h, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// orca_gru_update for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand it a scratch buffer: a serving loop that runs under a fixed
// memory budget and treats any cudaMalloc as a fault (it also synchronises the whole device), or a
// plugin whose owner forbids allocator calls after start-up.  For them the [rows, 172] staging
// area of the GRU result lives in the library image itself: a file-scope device array that every GPU
// which loads the library holds until the process exits.  Its size bounds the call:
// ORCA_GRU_STATIC_MAX_ROWS rows (2.8 MB).
//
// In host code `g_gru_static_scratch` is only a stand-in for the symbol, not a device address, so
// the address is looked up with cudaGetSymbolAddress once per device (with that device current) and
// that pointer is what the kernels receive.  The look-up happens on the first call on a device;
// make that first call outside any stream capture.  All calls share the array and it keeps the
// previous call's contents: nothing in it has to start at zero (every row that is read was written
// by the same call first), but two calls that overlap on the GPU (different streams) race on it.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_gru_static_scratch[ORCA_GRU_STATIC_MAX_ROWS * ORCA_DIM];

int orca_gru_update_static(const orca_gru_weights_t *w, const orca_memory_t *mem, const int32_t *d_nodes,
                           int32_t n_cap, const int32_t *d_n, int32_t clear_flags, void *stream) {
  ORCA_CHECK_ARG(n_cap >= 0);
  if (n_cap > ORCA_GRU_STATIC_MAX_ROWS)
    return set_error(ORCA_E_CAPACITY,
                     "orca_gru_update_static: %d rows exceed the built-in scratch of %d rows; "
                     "use orca_gru_update with a caller-provided scratch buffer",
                     n_cap, ORCA_GRU_STATIC_MAX_ROWS);
  constexpr int kMaxDevices = 64;
  static float *scratch_of_device[kMaxDevices] = {nullptr};
  int dev = 0;
  ORCA_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return set_error(ORCA_E_UNSUPPORTED, "orca_gru_update_static: device %d", dev);
  if (scratch_of_device[dev] == nullptr) {
    float *p = nullptr;
    ORCA_CUDA(cudaGetSymbolAddress((void **)&p, g_gru_static_scratch));
    scratch_of_device[dev] = p;
  }
  return orca_gru_update(w, mem, d_nodes, n_cap, d_n, clear_flags, scratch_of_device[dev], stream);
}

}  // extern "C"
