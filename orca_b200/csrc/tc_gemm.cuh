// Interface of the tensor-core projection kernel (tc_gemm.cu).
#pragma once

#include "common.cuh"

namespace orca {
namespace tc {

constexpr int BM = 128;      // tile rows (accumulator lanes)
constexpr int BN = 176;      // tile columns (172 padded to a multiple of 16)
constexpr int BK = 64;       // K elements per stage = 8 chunks of 8 bf16 (16 bytes) = 4 MMA steps of K = 16
constexpr int CHUNKS = BK / 8;
constexpr int STAGES = 2;    // producer group g (warps 0-3 / 6-9) owns stage g
constexpr int THREADS = 320;
constexpr int A_LBO = BM * 16 + 16;   // chunk stride of an A image; +16 keeps the 8-byte stores conflict free
constexpr int A_SBO = 128;
constexpr int A_BYTES = CHUNKS * A_LBO;
constexpr int B_LBO = BN * 16;
constexpr int B_SBO = 128;
constexpr int B_BYTES = CHUNKS * B_LBO;
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;   // A head, A tail, W head, W tail
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
// The merger kernel (EPI_MERGER) runs a second product from shared memory once the first is done: the
// hidden tile as an A image of 22 chunks (176 columns) head + tail at the start of the ring, and the
// three k-blocks of the second weight matrix behind it (the third holds only 6 chunks); k-block 0 sits past
// the ring, so that it can be fetched while the first product still uses the stages.
constexpr int A2_CHUNKS = BN / 8;
constexpr int A2_BYTES = A2_CHUNKS * A_LBO;
constexpr int W2_KB1 = 2 * A2_BYTES;
constexpr int W2_KB2 = W2_KB1 + 2 * B_BYTES;
constexpr int W2_TAIL_CHUNKS = A2_CHUNKS - 2 * CHUNKS;   // chunks of the last k-block that are used
constexpr int W2_KB0 = W2_KB2 + 2 * W2_TAIL_CHUNKS * B_LBO;
constexpr int MERGER_RING_BYTES = W2_KB0 + 2 * B_BYTES;
constexpr int MERGER_SMEM_BYTES = MERGER_RING_BYTES + 1024 + 256;
static_assert(W2_KB0 >= STAGES * STAGE_BYTES, "k-block 0 of the second weights must lie past the stage ring");
constexpr int TMEM_COLS = 512;   // main accumulator at column 0, cross-term accumulator at column 256
constexpr int TMEM_SMALL = 256;
constexpr int TILE_LD = 180;     // floats per row of the epilogue's output tile: 16-byte row-wise stores of a
                                 // warp (one row per lane) then spread over all banks

// A logical A row is the concatenation of up to two gathered table rows
struct RowSrc {
  const float *p;      // table base, row stride = width floats
  const int32_t *idx;  // row m reads table row idx[m]; nullptr: (mod > 0 ? m % mod : m) + add
  int width;
  int mod;
  int add;
};

// LAYERNORM / GRU epilogue that also delivers the rows to the other GPUs of the node (the exchange of the
// multi-GPU split): row m goes to rows[q] + off + m * 172 floats for every rank q (peer stores over
// NVLink; the own buffer is one of them), and the last CTA to finish posts `seq` in word `rank` of every
// rank's flag array.  counter: a zeroed word of the own flag array.
struct PeerOut {
  float *rows[ORCA_MAX_WORLD];
  int32_t *flags[ORCA_MAX_WORLD];
  int32_t *counter;
  long long off;
  int world, rank, seq;
};

// EPI_MERGER: hidden = relu(A . W + bias + valid * bias2) kept on the SM, then LayerNorm(hidden . W2 + bias_out)
// with the LayerNorm epilogue (push, peer fan-out).  EPI_LAYERNORM names that epilogue inside the kernel; it
// is not a kernel of its own (values 1 and 2 were the two separate kernels the merger replaced).
enum Epilogue { EPI_BIAS = 0, EPI_LAYERNORM = 2, EPI_GRU = 3, EPI_SCORE = 4, EPI_MERGER = 5 };

struct Args {
  RowSrc a0, a1;             // a1.width == 0 when unused
  int Kd;                    // a0.width + a1.width
  const uint8_t *row_valid;  // optional: rows with 0 read zeros for the first zero_cols columns
  int zero_cols;
  const void *w_packed;      // [n_tiles][n_kblocks][head | tail] bf16 stage images (weights.pack_tc)
  int n_kblocks;
  int m_cap;
  const int32_t *d_m;
  // optional row map: tile row m stands for entry m * row_stride + row_off of the index lists (a0.idx,
  // a1.idx, nodes; idx_limit entries) and d_m counts the entries of the whole lists; row_stride <= 1: off
  int row_stride, row_off, idx_limit;
  const float *bias;         // [n_tiles * BN]
  float *out;                // BIAS: [m, out_ld]; HIDDEN / LAYERNORM: [m, 172]; GRU: [m, 172]; SCORE: [m]
  int out_ld;
  // MERGER, first product: + valid * bias2; second product: packed weights (3 k-blocks) and bias
  const float *bias2;
  const void *w2_packed;
  const float *bias_out;
  // LAYERNORM
  const float *ln_w, *ln_b;
  float *push_table;
  const int32_t *push_ids;
  const uint8_t *push_win;                  // winners by flag, or (push_win == nullptr) by record:
  const unsigned long long *push_last_pos;  // row m wins if m >= push_all_from or
  long long push_base;                      // push_last_pos[push_ids[m]] == push_base + m
  int push_all_from;
  // GRU
  const float *memory;
  const int32_t *nodes;
  // SCORE
  const float *w2;
  float b2;
  int32_t *status;           // where a wait that gave up is reported (set by launch() from the context)
  long long wait_limit;      // SM clocks a wait on an mbarrier may spin (set by launch() from the context)
  PeerOut peer;              // peer.world == 0: no fan-out
};

// enqueues the kernel: grid = (n_tiles, ceil(m_cap / 128))
int launch(int epilogue, const Args &a, int n_tiles, cudaStream_t stream);

}  // namespace tc

// out-projection + merger + LayerNorm of an attention layer with the optional history push; see gemm.cu
int attn_output_impl(const orca_attn_weights_t *w, const float *d_ctx, const uint8_t *d_valid, const float *d_feat,
                     const int32_t *d_idx, int32_t n_rows_cap, const int32_t *d_n_rows, float *d_out,
                     float *d_push_table, const int32_t *d_push_ids, const uint8_t *d_push_win,
                     const int64_t *d_last_pos, long long base, int all_from, float *d_scratch_hidden,
                     int rows_hint, cudaStream_t stream, const tc::PeerOut *peer = nullptr);
// whether the projections run on the tensor cores (orca_set_projection_mode(0)); the fp32 debug path has
// no peer fan-out
bool projections_on_tensor_cores();

}  // namespace orca
