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
//           processed), and columns l, l+32, ... of the time-encoding part, which is computed
//           (cos of delta * w) and parked in shared memory.  The lane's partial dot products with
//           the two query heads are parked too; no cross-lane work happens inside the slot loop.
//   softmax the 2 * slots partial-sum rows are reduced by 2 * slots lanes at once, the two heads'
//           softmax runs across lanes;
//   pass 2  the gathered pieces are loaded again (they sit in L1/L2 now), the time encodings come back
//           from shared memory, and the weighted key sum is accumulated in registers.
// Keeping the reductions and the exponentials out of the slot loops matters: with one row per warp
// the kernel is bound by the length of each warp's dependent instruction chain, not by bandwidth.
// (The 688-byte rows are not moved by cp.async.bulk: an SM retires only about one small bulk copy
// per ~130 cycles, which capped an earlier version at 1.5 TB/s whatever else it did.)
//
// Rows are handed out by ticket (one atomic per row on a counter the launch leaves at zero again), not
// by a fixed stride: rows differ tenfold in cost (0 to k valid slots) and a launch holds only two to
// four rows per resident warp, so a static split ends with most warps idle behind the unlucky ones.
// A warp draws its next ticket and loads that row's slot indices before it works on the current row,
// and -- between the two passes -- asks for the next row's neighbour and edge-feature rows to be
// brought into L2 (prefetch.global.L2, one 32-byte sector per lane): the gathers are random 688-byte
// reads over gigabytes, each a DRAM access behind a TLB miss, and without the prefetch a row's five
// double-buffered load rounds each pay that latency in full.
// The multiply-adds are the packed two-wide form (fma.rn.f32x2 of this architecture): half the issue
// slots for the dot products and the weighted sums.
// No block-level synchronisation; a block is eight independent warps.
constexpr int GA_MEM_F4 = 2 * D / 4;            // 86 sixteen-byte pieces of [neighbour | edge feature]
constexpr int GA_ROW_F4 = D / 4;                // 43 pieces per table row
constexpr int GA_T_ITERS = (D + 31) / 32;       // 6 time columns per lane (the last one partial)
constexpr int GA_TE_LD = 172;                   // floats per parked time encoding
constexpr int GA_PART_LD = 33;                  // 32 partial sums + 1 pad (conflict-free column reads)
constexpr int GA_ROW_SECTORS = 22;              // 32-byte sectors a 688-byte row can touch, minus none: a row
                                                // that starts 16 bytes into a sector ends 16 bytes into its 22nd
__host__ __device__ constexpr int ga_warp_floats(int k) { return k * GA_TE_LD + 2 * k * GA_PART_LD; }

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 lo2(const float4 &v) { return make_float2(v.x, v.y); }
__device__ __forceinline__ float2 hi2(const float4 &v) { return make_float2(v.z, v.w); }
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Time encodings of one slot for this lane's columns lane, lane+32, ...: the first NL column groups
// hold large arguments (fixed-point reduction), the others small ones (fp32 reduction).  w decreases
// with the column, so "large" groups are always a prefix; NL is uniform over the warp and the body is
// branch free, which lets the six cosines of a lane overlap.
template <int NL>
__device__ __forceinline__ void time_terms(float dt, const float (&wt)[6], float (&te)[6]) {
#pragma unroll
  for (int i = 0; i < 6; ++i) {
    const float x = dt * wt[i];
    te[i] = i < NL ? cos_fixed(x) : cos_small(x);
  }
}

__global__ void __launch_bounds__(GA_THREADS, 2)
attn_gather_kernel(const float *__restrict__ qt, const float *__restrict__ nbr_table,
                   const float *__restrict__ edge_table, const float *__restrict__ time_w,
                   const int32_t *__restrict__ nbr, const int32_t *__restrict__ eid,
                   const float *__restrict__ delta, int k, int n_cap, const int32_t *__restrict__ d_n,
                   float *__restrict__ ctx, uint8_t *__restrict__ valid_out, int32_t *__restrict__ ticket,
                   unsigned long long *__restrict__ prof) {
  extern __shared__ __align__(128) float smem[];
  constexpr unsigned FULL = 0xffffffffu;
  dep_trigger();
  dep_wait();
  const int n = rows_of(n_cap, d_n);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float *s_te = smem + warp * ga_warp_floats(k);  // [k][172]
  float *s_part = s_te + k * GA_TE_LD;            // [2k][33]
  // this lane's time-encoding frequencies
  float wt[GA_T_ITERS];
#pragma unroll
  for (int i = 0; i < GA_T_ITERS; ++i) wt[i] = (lane + 32 * i < D) ? __ldg(time_w + lane + 32 * i) : 0.f;
  const bool third = lane + 64 < GA_MEM_F4;       // lanes 0..21 own a third 16-byte piece
  const bool tail_col = lane + 32 * (GA_T_ITERS - 1) < D;   // lanes 0..11 own a sixth time column
  unsigned long long prof_rows = 0, prof_slots = 0;

  auto draw = [&]() -> int {
    int r = 0;
    if (lane == 0) r = atomicAdd(&ticket[0], 1);
    return __shfl_sync(FULL, r, 0);
  };
  int row = draw();
  int my_nbr = 0, my_eid = 0;
  float my_dt = 0.f;
  if (row < n && lane < k) {
    const size_t o = (size_t)row * k + lane;
    my_nbr = nbr[o];
    my_eid = eid[o];
    my_dt = delta[o];
  }
  while (row < n) {
    // the next row of this warp: the ticket is requested now and read (with that row's slot indices) once
    // the first loads of the current row are under way
    int tkt = 0;
    if (lane == 0) tkt = atomicAdd(&ticket[0], 1);
    int next = 0, nx_nbr = 0, nx_eid = 0;
    float nx_dt = 0.f;
    auto fetch_next = [&]() {
      next = __shfl_sync(FULL, tkt, 0);
      if (next < n && lane < k) {
        const size_t o = (size_t)next * k + lane;
        nx_nbr = nbr[o];
        nx_eid = eid[o];
        nx_dt = delta[o];
      }
    };
    // asks for the table rows of the next row's valid slots to be brought into L2
    auto prefetch_next = [&]() {
      unsigned nm = __ballot_sync(FULL, nx_nbr != 0);
      while (nm) {
        const int j = __ffs(nm) - 1;
        nm &= nm - 1;
        const int nb = __shfl_sync(FULL, nx_nbr, j), ei = __shfl_sync(FULL, nx_eid, j);
        const char *nrow = reinterpret_cast<const char *>(nbr_table + (size_t)nb * D);
        const char *erow = reinterpret_cast<const char *>(edge_table + (size_t)ei * D);
        prefetch_l2(lane < GA_ROW_SECTORS ? nrow + 32 * lane : erow + 32 * (lane - GA_ROW_SECTORS));
        if (lane < 2 * GA_ROW_SECTORS - 32) prefetch_l2(erow + 32 * (lane + 32 - GA_ROW_SECTORS));
      }
    };
    const unsigned vmask = __ballot_sync(FULL, my_nbr != 0);
    if (vmask == 0) {
      // every slot is padding: the layer ignores the attention term for this row
      if (lane == 0) valid_out[row] = 0;
      fetch_next();
      prefetch_next();
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
      // which column groups of this lane's slot need the fixed-point cosine (see time_terms)
      int my_nl = 0;
      {
        const float adt = fabsf(my_dt);
#pragma unroll
        for (int i = 0; i < GA_T_ITERS; ++i) my_nl += adt * __ldg(time_w + 32 * i) >= 32768.f ? 1 : 0;
        if (!(adt * __ldg(time_w) < 1073741824.f)) my_nl = -1;   // beyond the fixed-point range (or not finite)
      }
      // the lane's pieces of the two query heads (head h starts at h * 528 in the projected query);
      // the time part is kept as (head 0, head 1) pairs for the two-wide multiply-adds
      const float *qrow = qt + (size_t)row * QT_LD;
      float4 qa[3], qb[3];
      float2 qtt[GA_T_ITERS];
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int f = (i < 2 || third) ? lane + 32 * i : 0;
        qa[i] = __ldg(reinterpret_cast<const float4 *>(qrow) + f);
        qb[i] = __ldg(reinterpret_cast<const float4 *>(qrow + QT_HEAD) + f);
      }
#pragma unroll
      for (int i = 0; i < GA_T_ITERS; ++i) {
        const bool in = i < GA_T_ITERS - 1 || tail_col;
        const int c = in ? lane + 32 * i : 0;
        const float a = __ldg(qrow + 2 * D + c), b = __ldg(qrow + QT_HEAD + 2 * D + c);
        qtt[i] = in ? make_float2(a, b) : make_float2(0.f, 0.f);   // a column past the end contributes nothing
      }
      fetch_next();

      // ---- pass 1: time encodings and partial logits, slot by slot
      auto pass1_slot = [&](int it, int j, const float4(&x)[3]) {
        const float dt = __shfl_sync(FULL, my_dt, j);
        const int nl = __shfl_sync(FULL, my_nl, j);
        float te[GA_T_ITERS];
        switch (nl) {
          case 0: time_terms<0>(dt, wt, te); break;
          case 1: time_terms<1>(dt, wt, te); break;
          case 2: time_terms<2>(dt, wt, te); break;
          case 3: time_terms<3>(dt, wt, te); break;
          default:
#pragma unroll
            for (int i = 0; i < GA_T_ITERS; ++i) te[i] = cos_any(dt * wt[i]);
        }
        float2 st = make_float2(0.f, 0.f);             // (head 0, head 1) over the time columns
#pragma unroll
        for (int i = 0; i < GA_T_ITERS; ++i) {
          if (i < GA_T_ITERS - 1 || tail_col) s_te[it * GA_TE_LD + lane + 32 * i] = te[i];
          st = fma2(make_float2(te[i], te[i]), qtt[i], st);
        }
        float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);   // head 0 / head 1, two partial sums each
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          if (i < 2 || third) {
            a0 = fma2(lo2(x[i]), lo2(qa[i]), a0);
            a0 = fma2(hi2(x[i]), hi2(qa[i]), a0);
            a1 = fma2(lo2(x[i]), lo2(qb[i]), a1);
            a1 = fma2(hi2(x[i]), hi2(qb[i]), a1);
          }
        }
        s_part[(2 * it) * GA_PART_LD + lane] = a0.x + a0.y + st.x;
        s_part[(2 * it + 1) * GA_PART_LD + lane] = a1.x + a1.y + st.y;
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
      // pass 2's first slot goes out before the softmax, the next row's prefetches behind it
      todo = vmask;
      load_slot(__ffs(todo) - 1, xa);
      todo &= todo - 1;
      prefetch_next();

      // ---- softmax: lane p reduces partial row p = 2 * slot + head; heads live on even / odd lanes
      // (k <= 16 keeps all 2k rows on the 32 lanes; for larger k a lane takes rows p and p + 32)
      float prob_lo = 0.f, prob_hi = 0.f;
      {
        float lg_lo = -INFINITY, lg_hi = -INFINITY;
        if (lane < 2 * n_valid) {
          float a = 0.f;
#pragma unroll 8
          for (int t = 0; t < 32; ++t) a += s_part[lane * GA_PART_LD + t];
          lg_lo = a;
        }
        if (lane + 32 < 2 * n_valid) {
          float a = 0.f;
#pragma unroll 8
          for (int t = 0; t < 32; ++t) a += s_part[(lane + 32) * GA_PART_LD + t];
          lg_hi = a;
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

      // ---- pass 2: weighted key sum
      float4 am0[3], am1[3];                         // gathered part, heads 0 / 1
      float2 at[GA_T_ITERS];                         // time part, (head 0, head 1)
#pragma unroll
      for (int i = 0; i < 3; ++i) am0[i] = am1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < GA_T_ITERS; ++i) at[i] = make_float2(0.f, 0.f);
      auto pass2_slot = [&](int it, const float4(&x)[3]) {
        const int p = 2 * it;
        const float p0 = p < 32 ? __shfl_sync(FULL, prob_lo, p) : __shfl_sync(FULL, prob_hi, p - 32);
        const float p1 = p < 32 ? __shfl_sync(FULL, prob_lo, p + 1) : __shfl_sync(FULL, prob_hi, p - 31);
        const float2 P0 = make_float2(p0, p0), P1 = make_float2(p1, p1), P01 = make_float2(p0, p1);
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          float2 r;
          r = fma2(P0, lo2(x[i]), lo2(am0[i])); am0[i].x = r.x; am0[i].y = r.y;
          r = fma2(P0, hi2(x[i]), hi2(am0[i])); am0[i].z = r.x; am0[i].w = r.y;
          r = fma2(P1, lo2(x[i]), lo2(am1[i])); am1[i].x = r.x; am1[i].y = r.y;
          r = fma2(P1, hi2(x[i]), hi2(am1[i])); am1[i].z = r.x; am1[i].w = r.y;
        }
#pragma unroll
        for (int i = 0; i < GA_T_ITERS; ++i) {
          if (i < GA_T_ITERS - 1 || tail_col) {
            const float te = s_te[it * GA_TE_LD + lane + 32 * i];
            at[i] = fma2(P01, make_float2(te, te), at[i]);
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
        }
      }
#pragma unroll
      for (int i = 0; i < GA_T_ITERS; ++i) {
        if (i < GA_T_ITERS - 1 || tail_col) {
          out[2 * D + lane + 32 * i] = at[i].x;
          out[KEY + 2 * D + lane + 32 * i] = at[i].y;
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
                       int k, int n_rows_cap, const int32_t *d_n_rows, int rows_hint, float *d_ctx,
                       uint8_t *d_valid, int32_t *d_ticket, cudaStream_t stream) {
  ORCA_CHECK_ARG(d_qt && d_nbr_table && d_edge_table && d_time_w && d_nbr && d_eid && d_delta && d_ctx &&
                 d_valid && d_ticket);
  ORCA_CHECK_ARG(k >= 1 && k <= ORCA_MAX_K && n_rows_cap >= 0);
  ORCA_CHECK_ARG(((uintptr_t)d_qt % 16 == 0) && ((uintptr_t)d_nbr_table % 16 == 0) &&
                 ((uintptr_t)d_edge_table % 16 == 0));
  if (n_rows_cap == 0) return ORCA_OK;
  Ctx *c = cur();
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_attn_gather: no context for the current device");
  // two blocks per SM share its shared memory: as many warps per block as fit into half of it
  const int warps = std::max(1, std::min(GA_WARPS, GA_SMEM_LIMIT / 2 / (ga_warp_floats(k) * (int)sizeof(float))));
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
                                                           d_delta, k, n_rows_cap, d_n_rows, d_ctx, d_valid, d_ticket,
                                                           pf.d_counters);
  else
    ORCA_CUDA(launch_dep(attn_gather_kernel, grid, warps * 32, smem, stream, d_qt, d_nbr_table, d_edge_table,
                         d_time_w, d_nbr, d_eid, d_delta, (int)k, (int)n_rows_cap, d_n_rows, d_ctx, d_valid, d_ticket,
                         (unsigned long long *)nullptr));
  if (pf.on) {
    ORCA_CUDA(cudaEventRecord(pf.ev[pf.used + 1], stream));
    pf.used += 2;
  }
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
                            d_n_rows, 0, d_ctx, d_valid, c->d_words + CTX_TICKET_MAIN, (cudaStream_t)stream);
}
