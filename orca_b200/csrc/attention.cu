// The fused gather-attention kernel: per query row, gather the valid neighbour rows and edge-feature
// rows (688 B each) with direct 128-bit loads, compute the time encoding cos(delta * w) in registers,
// and run the masked two-head attention over the slots on chip.  No weight matrix is touched: the K
// and V projections are folded into the query (qt) and into the output GEMM, so the memory side of
// this kernel is pure HBM traffic:
//   in : qt row (2 x 2064 B) + valid slots x (688 + 688) B of gathered rows + K * 12 B of indices
//   out: ctx row (4128 B) + 1 flag
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "context.cuh"

namespace orca {

#ifndef ORCA_GA_THREADS
#define ORCA_GA_THREADS 256
#endif
constexpr int GA_THREADS = ORCA_GA_THREADS;
constexpr int GA_SMEM_LIMIT = 226 * 1024;   // dynamic shared memory one block may ask for
constexpr int GA_WARPS = GA_THREADS / 32;

// One warp per query row, two passes over its valid neighbour slots:
//   pass 1  every lane owns a fixed set of key columns -- 16-byte pieces l, l+32, l+64 of the
//           gathered [neighbour | edge feature] part, loaded straight from the tables into registers
//           with 128-bit loads (the next slot's pieces are requested before the current slot is
//           processed), and column PAIRS l, l+32, l+64 of the time-encoding part, which is computed
//           (cos of delta * w) two columns at a time with the packed two-wide fp32 instructions of this
//           architecture (fma.rn.f32x2: half the issue slots for the range reduction, the dot products
//           and the weighted sums) and parked in shared memory.  The lane's partial dot products with
//           the two query heads are parked too; no cross-lane work happens inside the slot loop.
//   softmax the 2 * slots partial-sum rows are reduced by 2 * slots lanes at once, the two heads'
//           softmax runs across lanes;
//   pass 2  the gathered pieces are loaded again (they sit in L1/L2 now), the time encodings come back
//           from shared memory, and the weighted key sum is accumulated in registers.
// Keeping the reductions and the exponentials out of the slot loops matters: with one row per warp
// the kernel is bound by the length of each warp's dependent instruction chain, not by bandwidth (a
// single pass with a running softmax needs a warp-wide reduction per slot and measured 15 % slower).
// (The 688-byte rows are not moved by cp.async.bulk: an SM retires only about one small bulk copy
// per ~130 cycles, which capped an earlier version at 1.5 TB/s whatever else it did.)
//
// Work distribution.  Rows differ tenfold in cost (0 to k valid slots, 1 to 14 us) and a launch holds
// only two to three rows per resident warp, so WHO gets WHICH row decides the length of the launch:
//   - rows are handed out by ticket (one atomic per row on a counter the launch leaves at zero again);
//   - a warp draws its next ticket only when it enters pass 2 of the current row: drawing it a whole
//     row ahead commits slow warps to one more row while fast warps run dry (measured: 38 -> 33 us);
//   - tickets walk the rows in the order of `order` (rows sorted by falling number of valid slots,
//     made by row_order_kernel beside the sampling), so that the launch ends on its lightest rows.
// The slot indices of the next row are loaded during pass 2; its projected query (4.2 KB) is read straight
// from global memory when the row starts (staging it in shared memory with cp.async during pass 2 was
// measured 6 % slower: the 4.2 KB per warp are better left free).
// No block-level synchronisation; a block is eight independent warps.
constexpr int GA_MEM_F4 = 2 * D / 4;            // 86 sixteen-byte pieces of [neighbour | edge feature]
constexpr int GA_ROW_F4 = D / 4;                // 43 pieces per table row
constexpr int GA_P_ITERS = 3;                   // pieces / time-column pairs per lane (the third for lanes 0..21)
constexpr int GA_TE_LD = 172;                   // floats per parked time encoding
constexpr int GA_PART_LD = 33;                  // 32 partial sums + 1 pad (conflict-free column reads)
// (a multiple of four floats: every warp's area starts on a 16-byte boundary)
__host__ __device__ constexpr int ga_warp_floats(int k) { return (k * GA_TE_LD + 2 * k * GA_PART_LD + 3) & ~3; }

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 dup2(float v) { return make_float2(v, v); }
__device__ __forceinline__ float2 lo2(const float4 &v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(const float4 &v) { return make_float2(v.z, v.w); }

// cos of two arguments below 2^15 at once: the Cody-Waite reduction of cos_small in packed arithmetic;
// the nearest integer of x / 2pi comes from adding and subtracting 1.5 * 2^23
__device__ __forceinline__ float2 cos_small2(float2 x) {
  const float2 t = mul2(x, dup2(0.15915494309189535f));
  const float2 kk = add2(add2(t, dup2(12582912.f)), dup2(-12582912.f));
  float2 r = fma2(kk, dup2(-6.28125f), x);
  r = fma2(kk, dup2(-0.0019350051879882812f), r);
  r = fma2(kk, dup2(-3.019916050561733e-07f), r);
  return make_float2(__cosf(r.x), __cosf(r.y));
}

// Time encodings of one slot for this lane's column pairs: the first NL pair groups (64 columns each) hold
// large arguments (fixed-point reduction), the others small ones (packed fp32 reduction).  w decreases with
// the column, so "large" groups are always a prefix; NL is uniform over the warp and the body is branch free.
template <int NL>
__device__ __forceinline__ void time_terms(float dt, const float2 (&wt)[GA_P_ITERS], float2 (&te)[GA_P_ITERS]) {
#pragma unroll
  for (int i = 0; i < GA_P_ITERS; ++i) {
    const float2 x = mul2(dup2(dt), wt[i]);
    te[i] = i < NL ? make_float2(cos_fixed(x.x), cos_fixed(x.y)) : cos_small2(x);
  }
}

// Rows sorted by falling number of valid slots (counting sort, one block): order[0 .. n) = row ids.  The
// tables are right-aligned (padding first), so a row's count is k minus the position of its first neighbour.
__global__ void __launch_bounds__(1024)
row_order_kernel(const int32_t *__restrict__ nbr_a, int n_cap_a, const int32_t *__restrict__ d_n_a,
                 int32_t *__restrict__ order_a, const int32_t *__restrict__ nbr_b, int n_cap_b,
                 const int32_t *__restrict__ d_n_b, int32_t *__restrict__ order_b, int k) {
  __shared__ int s_bin[ORCA_MAX_K + 1];
  dep_trigger();
  dep_wait();
  // block 0 orders table a, block 1 table b
  const int32_t *nbr = blockIdx.x == 0 ? nbr_a : nbr_b;
  int32_t *order = blockIdx.x == 0 ? order_a : order_b;
  const int n = blockIdx.x == 0 ? rows_of(n_cap_a, d_n_a) : rows_of(n_cap_b, d_n_b);
  const int tid = threadIdx.x;
  if (tid <= ORCA_MAX_K) s_bin[tid] = 0;
  __syncthreads();
  auto count = [&](int r) {
    const int32_t *row = nbr + (size_t)r * k;
    int c = 0;
    for (int j = 0; j < k; ++j) c += row[j] != 0 ? 1 : 0;
    return c;
  };
  for (int r = tid; r < n; r += 1024) atomicAdd(&s_bin[count(r)], 1);
  __syncthreads();
  if (tid == 0) {   // bins -> first position, heaviest bin first
    int pos = 0;
    for (int c = k; c >= 0; --c) {
      const int m = s_bin[c];
      s_bin[c] = pos;
      pos += m;
    }
  }
  __syncthreads();
  for (int r = tid; r < n; r += 1024) order[atomicAdd(&s_bin[count(r)], 1)] = r;
}

__global__ void __launch_bounds__(GA_THREADS, 2)
attn_gather_kernel(const float *__restrict__ qt, const float *__restrict__ nbr_table,
                   const float *__restrict__ edge_table, const float *__restrict__ time_w,
                   const int32_t *__restrict__ nbr, const int32_t *__restrict__ eid,
                   const float *__restrict__ delta, int k, int n_cap, const int32_t *__restrict__ d_n,
                   const int32_t *__restrict__ order, float *__restrict__ ctx, uint8_t *__restrict__ valid_out,
                   int32_t *__restrict__ ticket, unsigned long long *__restrict__ prof) {
  extern __shared__ __align__(128) float smem[];
  constexpr unsigned FULL = 0xffffffffu;
  dep_trigger();
  dep_wait();
  const int n = rows_of(n_cap, d_n);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *s_te = smem + warp * ga_warp_floats(k);  // [k][172]
  float *s_part = s_te + k * GA_TE_LD;            // [2k][33]
  const bool third = lane + 64 < GA_MEM_F4;       // lanes 0..21 own a third piece / pair
  // this lane's time-encoding frequencies, as column pairs, and the largest frequency of each pair group
  float2 wt[GA_P_ITERS];
#pragma unroll
  for (int i = 0; i < GA_P_ITERS; ++i)
    wt[i] = (i < 2 || third) ? __ldg(reinterpret_cast<const float2 *>(time_w) + lane + 32 * i) : make_float2(0.f, 0.f);
  const float wg0 = __ldg(time_w), wg1 = __ldg(time_w + 64), wg2 = __ldg(time_w + 128);
  unsigned long long prof_rows = 0, prof_slots = 0;

  auto row_of_ticket = [&](int t) -> int { return order != nullptr ? order[t] : t; };
  auto load_indices = [&](int r, int &o_nbr, int &o_eid, float &o_dt) {
    o_nbr = 0, o_eid = 0, o_dt = 0.f;
    if (lane < k) {
      const size_t o = (size_t)r * k + lane;
      o_nbr = nbr[o];
      o_eid = eid[o];
      o_dt = delta[o];
    }
  };
  int tkt = 0;
  if (lane == 0) tkt = atomicAdd(&ticket[0], 1);
  tkt = __shfl_sync(FULL, tkt, 0);
  int row = tkt < n ? row_of_ticket(tkt) : -1;
  int my_nbr = 0, my_eid = 0;
  float my_dt = 0.f;
  if (row >= 0) load_indices(row, my_nbr, my_eid, my_dt);
  while (row >= 0) {
    int next = -1, nx_nbr = 0, nx_eid = 0;
    float nx_dt = 0.f;
    const unsigned vmask = __ballot_sync(FULL, my_nbr != 0);
    if (vmask == 0) {
      // every slot is padding: the layer ignores the attention term for this row
      if (lane == 0) valid_out[row] = 0;
      if (lane == 0) tkt = atomicAdd(&ticket[0], 1);
      tkt = __shfl_sync(FULL, tkt, 0);
      if (tkt < n) {
        next = row_of_ticket(tkt);
        load_indices(next, nx_nbr, nx_eid, nx_dt);
      }
    } else {
      const int n_valid = __popc(vmask);
      // this lane's pieces of a slot: piece l of the neighbour row; piece l+32 of the concatenation
      // (neighbour row for l < 11, else edge row piece l-11); piece l+64 (edge row piece l+21, l < 22).
      // Addresses are selected, loads are unconditional (lanes without a third piece re-read piece 0
      // of the edge row; their third accumulator is never written out).
      auto load_slot = [&](int j, float4(&x)[3]) {
        const int nb = __shfl_sync(FULL, my_nbr, j), ei = __shfl_sync(FULL, my_eid, j);
        const float4 *nrow = reinterpret_cast<const float4 *>(nbr_table + (size_t)nb * D);
        const float4 *erow = reinterpret_cast<const float4 *>(edge_table + (size_t)ei * D);
        const float4 *p1 = lane < GA_ROW_F4 - 32 ? nrow + lane + 32 : erow + lane - (GA_ROW_F4 - 32);
        const float4 *p2 = third ? erow + lane + 64 - GA_ROW_F4 : erow;
        x[0] = __ldg(nrow + lane);
        x[1] = __ldg(p1);
        x[2] = __ldg(p2);
      };
      // two slot buffers used alternately (no register copies): while one slot is processed the next one
      // is in flight
      float4 xa[3], xb[3];
      unsigned todo = vmask;
      int j0 = __ffs(todo) - 1;
      todo &= todo - 1;
      load_slot(j0, xa);
      // which pair groups of this lane's slot need the fixed-point cosine (see time_terms)
      int my_nl;
      {
        const float adt = fabsf(my_dt);
        my_nl = (adt * wg0 >= 32768.f ? 1 : 0) + (adt * wg1 >= 32768.f ? 1 : 0) + (adt * wg2 >= 32768.f ? 1 : 0);
        if (!(adt * wg0 < 1073741824.f)) my_nl = -1;   // beyond the fixed-point range (or not finite)
      }
      // the lane's pieces of the two query heads
      float4 qa[3], qb[3];
      float2 qta[GA_P_ITERS], qtb[GA_P_ITERS];
      const float *q_src = qt + (size_t)row * QT_LD;
#pragma unroll
      for (int i = 0; i < GA_P_ITERS; ++i) {
        const int f = (i < 2 || third) ? lane + 32 * i : 0;
        qa[i] = __ldg(reinterpret_cast<const float4 *>(q_src) + f);
        qb[i] = __ldg(reinterpret_cast<const float4 *>(q_src + QT_HEAD) + f);
        qta[i] = __ldg(reinterpret_cast<const float2 *>(q_src + 2 * D) + f);
        qtb[i] = __ldg(reinterpret_cast<const float2 *>(q_src + QT_HEAD + 2 * D) + f);
      }

      // ---- pass 1: time encodings and partial logits, slot by slot
      auto pass1_slot = [&](int it, int j, const float4(&x)[3]) {
        const float dt = __shfl_sync(FULL, my_dt, j);
        const int nl = __shfl_sync(FULL, my_nl, j);
        float2 te[GA_P_ITERS];
        switch (nl) {
          case 0: time_terms<0>(dt, wt, te); break;
          case 1: time_terms<1>(dt, wt, te); break;
          case 2: time_terms<2>(dt, wt, te); break;
          case 3: time_terms<3>(dt, wt, te); break;
          default:
#pragma unroll
            for (int i = 0; i < GA_P_ITERS; ++i) te[i] = make_float2(cos_any(dt * wt[i].x), cos_any(dt * wt[i].y));
        }
        float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);   // head 0 / head 1, two partial sums each
#pragma unroll
        for (int i = 0; i < GA_P_ITERS; ++i) {
          if (i < 2 || third) {
            reinterpret_cast<float2 *>(s_te + it * GA_TE_LD)[lane + 32 * i] = te[i];
            a0 = fma2(te[i], qta[i], a0);
            a1 = fma2(te[i], qtb[i], a1);
            a0 = fma2(lo2(x[i]), lo2(qa[i]), a0);
            a0 = fma2(hi2(x[i]), hi2(qa[i]), a0);
            a1 = fma2(lo2(x[i]), lo2(qb[i]), a1);
            a1 = fma2(hi2(x[i]), hi2(qb[i]), a1);
          }
        }
        s_part[(2 * it) * GA_PART_LD + lane] = a0.x + a0.y;
        s_part[(2 * it + 1) * GA_PART_LD + lane] = a1.x + a1.y;
      };
      for (int it = 0; it < n_valid; it += 2) {
        int j1 = -1;
        if (todo) {
          j1 = __ffs(todo) - 1;
          todo &= todo - 1;
          load_slot(j1, xb);
        }
        pass1_slot(it, j0, xa);
        if (j1 < 0) break;
        if (todo) {
          j0 = __ffs(todo) - 1;
          todo &= todo - 1;
          load_slot(j0, xa);
        }
        pass1_slot(it + 1, j1, xb);
      }
      __syncwarp();
      // the next ticket is drawn now, not a row ahead; pass 2's first slot goes out before the softmax
      if (lane == 0) tkt = atomicAdd(&ticket[0], 1);
      todo = vmask;
      load_slot(__ffs(todo) - 1, xa);
      todo &= todo - 1;

      // ---- softmax: lane p reduces partial row p = 2 * slot + head; heads live on even / odd lanes
      // (k <= 16 keeps all 2k rows on the 32 lanes; for larger k a lane takes rows p and p + 32)
      float prob_lo = 0.f, prob_hi = 0.f;
      {
        float lg_lo = -INFINITY, lg_hi = -INFINITY;
        if (lane < 2 * n_valid) {
          float a = 0.f, b = 0.f;
#pragma unroll 8
          for (int t = 0; t < 32; t += 2) {
            a += s_part[lane * GA_PART_LD + t];
            b += s_part[lane * GA_PART_LD + t + 1];
          }
          lg_lo = a + b;
        }
        if (lane + 32 < 2 * n_valid) {
          float a = 0.f, b = 0.f;
#pragma unroll 8
          for (int t = 0; t < 32; t += 2) {
            a += s_part[(lane + 32) * GA_PART_LD + t];
            b += s_part[(lane + 32) * GA_PART_LD + t + 1];
          }
          lg_hi = a + b;
        }
        float m = fmaxf(lg_lo, lg_hi);               // lanes of equal parity hold the same head
#pragma unroll
        for (int o = 2; o < 32; o <<= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, o));
        const float e_lo = lane < 2 * n_valid ? expf(lg_lo - m) : 0.f;
        const float e_hi = lane + 32 < 2 * n_valid ? expf(lg_hi - m) : 0.f;
        float sum = e_lo + e_hi;
#pragma unroll
        for (int o = 2; o < 32; o <<= 1) sum += __shfl_xor_sync(FULL, sum, o);
        const float inv = 1.f / sum;
        prob_lo = e_lo * inv;
        prob_hi = e_hi * inv;
      }
      // the next row of this warp: its indices are requested now and land during pass 2
      tkt = __shfl_sync(FULL, tkt, 0);
      if (tkt < n) {
        next = row_of_ticket(tkt);
        load_indices(next, nx_nbr, nx_eid, nx_dt);
      }

      // ---- pass 2: weighted key sum
      float4 am0[3], am1[3];                         // gathered part, heads 0 / 1
      float2 at0[GA_P_ITERS], at1[GA_P_ITERS];       // time part
#pragma unroll
      for (int i = 0; i < 3; ++i) am0[i] = am1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < GA_P_ITERS; ++i) at0[i] = at1[i] = make_float2(0.f, 0.f);
      auto pass2_slot = [&](int it, const float4(&x)[3]) {
        const int p = 2 * it;
        const float p0 = p < 32 ? __shfl_sync(FULL, prob_lo, p) : __shfl_sync(FULL, prob_hi, p - 32);
        const float p1 = p < 32 ? __shfl_sync(FULL, prob_lo, p + 1) : __shfl_sync(FULL, prob_hi, p - 31);
        const float2 P0 = dup2(p0), P1 = dup2(p1);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          float2 r;
          r = fma2(P0, lo2(x[i]), lo2(am0[i])); am0[i].x = r.x; am0[i].y = r.y;
          r = fma2(P0, hi2(x[i]), hi2(am0[i])); am0[i].z = r.x; am0[i].w = r.y;
          r = fma2(P1, lo2(x[i]), lo2(am1[i])); am1[i].x = r.x; am1[i].y = r.y;
          r = fma2(P1, hi2(x[i]), hi2(am1[i])); am1[i].z = r.x; am1[i].w = r.y;
        }
#pragma unroll
        for (int i = 0; i < GA_P_ITERS; ++i) {
          if (i < 2 || third) {
            const float2 te = reinterpret_cast<const float2 *>(s_te + it * GA_TE_LD)[lane + 32 * i];
            at0[i] = fma2(P0, te, at0[i]);
            at1[i] = fma2(P1, te, at1[i]);
          }
        }
      };
      for (int it = 0; it < n_valid; it += 2) {
        const bool more = todo != 0;
        if (more) {
          load_slot(__ffs(todo) - 1, xb);
          todo &= todo - 1;
        }
        pass2_slot(it, xa);
        if (!more) break;
        if (todo) {
          load_slot(__ffs(todo) - 1, xa);
          todo &= todo - 1;
        }
        pass2_slot(it + 1, xb);
      }
      // write the row: [head 0: gathered 344 | time 172][head 1: ...]
      float *out = ctx + (size_t)row * QT;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        if (i < 2 || third) {
          reinterpret_cast<float4 *>(out)[lane + 32 * i] = am0[i];
          reinterpret_cast<float4 *>(out + KEY)[lane + 32 * i] = am1[i];
          reinterpret_cast<float2 *>(out + 2 * D)[lane + 32 * i] = at0[i];
          reinterpret_cast<float2 *>(out + KEY + 2 * D)[lane + 32 * i] = at1[i];
        }
      }
      if (lane == 0) valid_out[row] = 1;
      prof_rows += 1;
      prof_slots += (unsigned long long)n_valid;
      __syncwarp();   // the parked values of this row are dead before the next row overwrites them
    }
    row = next;
    my_nbr = nx_nbr;
    my_eid = nx_eid;
    my_dt = nx_dt;
  }
  if (lane == 0) {
    // the last warp to run out of tickets leaves the counters at zero for the next launch
    const int total = (int)(gridDim.x * (blockDim.x >> 5));
    if (atomicAdd(&ticket[1], 1) == total - 1) {
      atomicExch(&ticket[0], 0);
      atomicExch(&ticket[1], 0);
    }
    if (prof != nullptr && prof_rows) {
      atomicAdd(&prof[0], prof_rows);     // rows that gathered
      atomicAdd(&prof[1], prof_slots);    // gathered neighbour slots
    }
  }
}

// `ticket`: two zeroed device words that the launch leaves at zero; launches that may overlap on the GPU
// need words of their own
int launch_attn_gather(const float *d_qt, const float *d_nbr_table, const float *d_edge_table,
                       const float *d_time_w, const int32_t *d_nbr, const int32_t *d_eid, const float *d_delta,
                       int k, int n_rows_cap, const int32_t *d_n_rows, int rows_hint, const int32_t *d_order,
                       float *d_ctx, uint8_t *d_valid, int32_t *d_ticket, cudaStream_t stream) {
  ORCA_CHECK_ARG(d_qt && d_nbr_table && d_edge_table && d_time_w && d_nbr && d_eid && d_delta && d_ctx &&
                 d_valid && d_ticket);
  ORCA_CHECK_ARG(k >= 1 && k <= ORCA_MAX_K && n_rows_cap >= 0);
  ORCA_CHECK_ARG(((uintptr_t)d_qt % 16 == 0) && ((uintptr_t)d_nbr_table % 16 == 0) &&
                 ((uintptr_t)d_edge_table % 16 == 0));
  if (n_rows_cap == 0) return ORCA_OK;
  Ctx *c = cur();
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_attn_gather: no context for the current device");
  // two blocks per SM share its shared memory (1 KB per block is the system's): as many warps per block as
  // fit into half of it
  const int warps = std::max(1, std::min(GA_WARPS, (GA_SMEM_LIMIT / 2 - 1024) / (ga_warp_floats(k) * (int)sizeof(float))));
  const size_t smem = (size_t)warps * ga_warp_floats(k) * sizeof(float);
  static thread_local int configured_device = -1;
  if (configured_device != c->device) {
    ORCA_CUDA(cudaFuncSetAttribute(attn_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   GA_SMEM_LIMIT / 2));
    configured_device = c->device;
  }
  GatherProfile &pf = c->prof;
  if (pf.on) {
    if (pf.used + 2 > pf.ev.size()) {
      cudaEvent_t a, b;
      ORCA_CUDA(cudaEventCreate(&a));
      ORCA_CUDA(cudaEventCreate(&b));
      pf.ev.push_back(a);
      pf.ev.push_back(b);
    }
    ORCA_CUDA(cudaEventRecord(pf.ev[pf.used], stream));
  }
  // one resident wave at most; fewer blocks when the caller expects fewer rows than the capacity
  const int rows = rows_hint > 0 ? std::min(rows_hint, n_rows_cap) : n_rows_cap;
  const int grid = std::min(ceil_div(rows, warps), c->sm_count * 2);
  // (the profiling events would sit between this kernel and its neighbours: plain launch then)
  if (pf.on)
    attn_gather_kernel<<<grid, warps * 32, smem, stream>>>(d_qt, d_nbr_table, d_edge_table, d_time_w, d_nbr, d_eid,
                                                           d_delta, k, n_rows_cap, d_n_rows, d_order, d_ctx, d_valid,
                                                           d_ticket, pf.d_counters);
  else
    ORCA_CUDA(launch_dep(attn_gather_kernel, grid, warps * 32, smem, stream, d_qt, d_nbr_table, d_edge_table,
                         d_time_w, d_nbr, d_eid, d_delta, (int)k, (int)n_rows_cap, d_n_rows, d_order, d_ctx, d_valid, d_ticket,
                         (unsigned long long *)nullptr));
  if (pf.on) {
    ORCA_CUDA(cudaEventRecord(pf.ev[pf.used + 1], stream));
    pf.used += 2;
  }
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

// rows of two neighbour tables (the two attention layers of a batch) in the order the gather kernel should
// take them: heaviest first
int launch_row_order(const int32_t *d_nbr_a, int n_cap_a, const int32_t *d_n_a, int32_t *d_order_a,
                     const int32_t *d_nbr_b, int n_cap_b, const int32_t *d_n_b, int32_t *d_order_b, int k,
                     cudaStream_t stream) {
  ORCA_CHECK_ARG(d_nbr_a && d_order_a && d_nbr_b && d_order_b && k >= 1 && k <= ORCA_MAX_K && n_cap_a >= 0 &&
                 n_cap_b >= 0);
  ORCA_CUDA(launch_dep(row_order_kernel, 2, 1024, 0, stream, d_nbr_a, (int)n_cap_a, d_n_a, d_order_a, d_nbr_b,
                       (int)n_cap_b, d_n_b, d_order_b, (int)k));
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace orca

using namespace orca;

extern "C" int orca_attn_gather(const float *d_qt, const float *d_nbr_table, const float *d_edge_table,
                                const float *d_time_w, const int32_t *d_nbr, const int32_t *d_eid,
                                const float *d_delta, int32_t k, int32_t n_rows_cap,
                                const int32_t *d_n_rows, float *d_ctx, uint8_t *d_valid,
                                int32_t *d_status, void *stream) {
  (void)d_status;
  Ctx *c = cur();
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_attn_gather: no context for the current device");
  return launch_attn_gather(d_qt, d_nbr_table, d_edge_table, d_time_w, d_nbr, d_eid, d_delta, k, n_rows_cap,
                            d_n_rows, 0, nullptr, d_ctx, d_valid, c->d_words + CTX_TICKET_MAIN, (cudaStream_t)stream);
}
