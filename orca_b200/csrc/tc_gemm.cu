// Dense projections on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
//   C[M, n_tiles*176] = A[M, K] . W[K, N]  (+ fused epilogue), fp32 in / fp32 out
//
// Precision: a single reduced-precision pass (TF32 or bf16) costs 2e-3 or more on the link scores
// (the path is specified to 1e-3).  Each fp32 operand is therefore split into a bf16 head and a bf16
// tail, x ~ hi + lo (16 significant bits), and three MMAs accumulate hi*hi + lo*hi + hi*lo in fp32 in
// tensor memory; emulating exactly this arithmetic over whole eval runs gives 3e-5 on the scores.
// The tensor core truncates when it adds into the fp32 accumulator, so the error grows with the
// number of accumulation steps at full magnitude: the two cross terms (2^-8 smaller) get an
// accumulator of their own and are added once, in the epilogue.  The weight heads/tails are split
// once on the host; the activation heads/tails are split by the producer warps on their way into
// shared memory.
//
// Tile: 128 rows x 176 columns, K consumed 64 elements per stage (4 MMA steps of K = 16, 12 MMAs),
// two stages; a CTA walks the row blocks blockIdx.y, blockIdx.y + gridDim.y, ... of its column tile.
// Every hop over an mbarrier costs ~250-300 cycles and a thread that arrives on one stalls until its
// outstanding global loads have landed, so stages are large and the A side is produced by two warp
// groups that alternate stages: while one group waits for its loads, the other converts and the tensor
// core works on the stage before.  Measured per k-block: ~0.7 us, set by the bytes a stage pulls into
// the SM (32 KB of fp32 rows + 44 KB of packed weights at ~55 B/clk).
// Warp roles (320 threads):
//   warps 0-3, 6-9  producer groups 0 / 1: group g fills stage g for every k-block kb = g (mod 2).
//              A lane owns one tile row's table index (index array, up to two tables concatenated
//              along K); inside a stage 8 lanes cover the 256 contiguous bytes a row contributes, 4
//              rows per load instruction (row indices exchanged by shuffle), each lane splits its 8
//              floats and stores one 16-byte chunk of the head and of the tail image in the no-swizzle
//              K-major core-matrix layout the MMA reads.
//   warp 4     streams the packed weight stage (one 44 KB bulk copy per stage).
//   warp 5     allocates tensor memory and issues the MMAs (one thread), releasing each stage with
//              tcgen05.commit.
// Epilogue: the producer warps move the accumulators (thread = row) into a row-major tile in the idle
// stage ring; all warps then write whole rows with coalesced stores (bias / ReLU / LayerNorm + push /
// GRU gates applied on the way).
//
// The merger of an attention layer (EPI_MERGER) chains a second product behind the first without leaving
// the SM: the first epilogue applies bias + ReLU to the 128 x 176 accumulator tile, splits it into bf16 head /
// tail and stores it in shared memory as the A image of (hidden . W2), whose three weight k-blocks are
// fetched while the first product still runs (k-block 0) and right after it (k-blocks 1, 2); the second
// product reuses the accumulator columns and ends in the LayerNorm epilogue.
//
// Every wait on an mbarrier is bounded; a wait that gives up records ORCA_E_TIMEOUT and the kernel
// runs to its end (tensor memory is always released).
#include <algorithm>
#include <cuda_bf16.h>

#include "common.cuh"
#include "context.cuh"
#include "tc_gemm.cuh"

namespace orca {
namespace tc {

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait (`limit` SM clocks, about a second by default); records the failure if the barrier never
// flipped.  `alive` makes the failure sticky: a thread that gave up once does not wait again, so a
// broken pipeline drains in one limit instead of one time-out per stage.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int32_t *status, int where, bool &alive,
                                          long long limit) {
  if (!alive) return;
  if (mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > limit) {
      report(status, ORCA_E_TIMEOUT, where);
      alive = false;
      return;
    }
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// shared-memory matrix descriptor, no swizzle, K-major: 8 rows x 16 bytes form one contiguous
// 128-byte core matrix; `lbo` = bytes between the two 16-byte K chunks of one MMA, `sbo` = bytes
// between consecutive 8-row groups
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  return d;
}

// D[tmem] (+)= A[smem] . B[smem]^T, 128 x 176 x 16, bf16 inputs, fp32 accumulate
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 consecutive accumulator columns of this thread's lane (= tile row)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// main accumulator + cross-term accumulator: both loads in flight, one wait
__device__ __forceinline__ void tmem_ld16_sum(uint32_t taddr, float (&v)[16]) {
  uint32_t a[16], b[16];
  tmem_ld16_nowait(taddr, a);
  tmem_ld16_nowait(taddr + TMEM_SMALL, b);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(a[i]) + __uint_as_float(b[i]);
}

__device__ __forceinline__ float4 ld_shared_f4(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void st_shared_f4(uint32_t saddr, float4 v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// x ~ head + tail, both bf16 (round to nearest even), for 8 consecutive K elements: one 16-byte chunk
// of the head image and one of the tail image.  Packed conversions (two floats per instruction).
__device__ __forceinline__ uint32_t pack_split(float x0, float x1, uint32_t &lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
  const uint32_t hb = *reinterpret_cast<const uint32_t *>(&h);
  const float r0 = x0 - __uint_as_float(hb << 16);
  const float r1 = x1 - __uint_as_float(hb & 0xffff0000u);
  const __nv_bfloat162 l = __floats2bfloat162_rn(r0, r1);
  lo = *reinterpret_cast<const uint32_t *>(&l);
  return hb;
}
__device__ __forceinline__ void split_chunk(const float4 a, const float4 b, uint4 &hi, uint4 &lo) {
  hi.x = pack_split(a.x, a.y, lo.x);
  hi.y = pack_split(a.z, a.w, lo.y);
  hi.z = pack_split(b.x, b.y, lo.z);
  hi.w = pack_split(b.z, b.w, lo.w);
}

struct Smem {
  uint32_t base;  // shared-window address of the (1024-byte aligned) stage ring
  __device__ uint32_t a_hi(int s) const { return base + s * STAGE_BYTES; }
  __device__ uint32_t a_lo(int s) const { return base + s * STAGE_BYTES + A_BYTES; }
  __device__ uint32_t b_hi(int s) const { return base + s * STAGE_BYTES + 2 * A_BYTES; }
  __device__ uint32_t b_lo(int s) const { return base + s * STAGE_BYTES + 2 * A_BYTES + B_BYTES; }
};

__device__ __forceinline__ const float *src_row(const RowSrc &s, int m) {
  const int r = s.idx ? s.idx[m] : (s.mod > 0 ? m % s.mod : m) + s.add;
  return s.p + (size_t)r * s.width;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __align__(16) float g_zero16[4] = {0.f, 0.f, 0.f, 0.f};

// Pass 2 of the epilogue (all ten warps): one warp per row of the tile that pass 1 left in shared
// memory, lanes along the columns (two 16-byte pieces per lane); four rows are in flight per warp so
// that their load / shuffle / store chains overlap.  meta_a / meta_b: lane i of warp w holds the
// per-row inputs of row w + 10*i (validity, push winner and id, GRU node).
template <int EPI>
constexpr int tile_bn() { return BN; }

template <int EPI>
__device__ __forceinline__ void tile_output(const Args &g, const float *tile, const float *s_bias, const float *s_v1,
                                            const float *s_v2, const float *s_dot, int m0, int m_rows, int nt,
                                            int warp, int lane, int meta_a, int meta_b) {
  if (EPI == EPI_SCORE) {
    const int tid = warp * 32 + lane;
    if (tid < m_rows) g.out[m0 + tid] = 1.f / (1.f + expf(-(s_dot[tid] + s_dot[BM + tid] + g.b2)));
    return;
  }
  constexpr int RB = 4;   // (2 measured the same, 8 spills)
  constexpr int BNv = tile_bn<EPI>();
  const int c0 = nt * BNv;
  const int j0 = lane, j1 = lane + 32;
  const int nj = (EPI == EPI_BIAS || EPI == EPI_GRU) ? BNv / 4 : D / 4;
  const bool has0 = j0 < nj;      // (only a 96-column tile leaves lanes without a first piece)
  const bool has1 = j1 < nj;
  const float4 f4z = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 bA = *reinterpret_cast<const float4 *>(&s_bias[4 * j0]);
  const float4 bB = has1 ? *reinterpret_cast<const float4 *>(&s_bias[4 * j1]) : f4z;
  const float4 vA = *reinterpret_cast<const float4 *>(&s_v1[4 * j0]);
  const float4 vB = has1 ? *reinterpret_cast<const float4 *>(&s_v1[4 * j1]) : f4z;
  const float4 lA = *reinterpret_cast<const float4 *>(&s_v2[4 * j0]);
  const float4 lB = has1 ? *reinterpret_cast<const float4 *>(&s_v2[4 * j1]) : f4z;
  auto add4 = [](float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); };
  const int uA = nt * (BNv / 4) + j0, uB = nt * (BNv / 4) + j1;   // GRU units of this lane
  const uint32_t tile_saddr = smem_addr(tile);
  for (int it0 = 0; warp + (THREADS / 32) * it0 < m_rows; it0 += RB) {
    float4 a[RB], b[RB];
    float hA[RB], hB[RB];
    int ma[RB], mb[RB], m[RB];
    bool ok[RB];
#pragma unroll
    for (int k = 0; k < RB; ++k) {
      const int r = warp + (THREADS / 32) * (it0 + k);
      ok[k] = r < m_rows;
      m[k] = m0 + r;
      ma[k] = __shfl_sync(0xffffffffu, meta_a, (it0 + k) & 31);
      mb[k] = __shfl_sync(0xffffffffu, meta_b, (it0 + k) & 31);
      const int rr = ok[k] ? r : 0;
      const uint32_t ra = tile_saddr + (uint32_t)(rr * TILE_LD + 4 * j0) * 4u;
      a[k] = add4(ld_shared_f4(ra), bA);
      b[k] = has1 ? add4(ld_shared_f4(ra + 512u), bB) : f4z;
      hA[k] = hB[k] = 0.f;
      if (EPI == EPI_GRU && ok[k]) {
        const float *hrow = g.memory + (size_t)mb[k] * D;
        if (uA < D) hA[k] = hrow[uA];
        if (has1 && uB < D) hB[k] = hrow[uB];
      }
    }
    if (EPI == EPI_BIAS) {
#pragma unroll
      for (int k = 0; k < RB; ++k)
        if (ok[k]) {
          float *o = g.out + (size_t)m[k] * g.out_ld + c0;
          *reinterpret_cast<float4 *>(o + 4 * j0) = a[k];
          if (has1) *reinterpret_cast<float4 *>(o + 4 * j1) = b[k];
        }
    } else if (EPI == EPI_LAYERNORM) {
      // both moments in one sweep (the row is O(1) after the merger, so E[y^2] - mean^2 loses nothing
      // that matters at the 1e-5 epsilon)
      float sum[RB], sumsq[RB];
#pragma unroll
      for (int k = 0; k < RB; ++k) {
        sum[k] = (a[k].x + a[k].y) + (a[k].z + a[k].w) + (b[k].x + b[k].y) + (b[k].z + b[k].w);
        sumsq[k] = a[k].x * a[k].x + a[k].y * a[k].y + a[k].z * a[k].z + a[k].w * a[k].w + b[k].x * b[k].x +
                   b[k].y * b[k].y + b[k].z * b[k].z + b[k].w * b[k].w;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int k = 0; k < RB; ++k) {
          sum[k] += __shfl_xor_sync(0xffffffffu, sum[k], o);
          sumsq[k] += __shfl_xor_sync(0xffffffffu, sumsq[k], o);
        }
      }
#pragma unroll
      for (int k = 0; k < RB; ++k)
        if (ok[k]) {
          const float mean = sum[k] * (1.f / D);
          const float sq = fmaxf(sumsq[k] - sum[k] * mean, 0.f);
          const float inv = 1.f / sqrtf(sq * (1.f / D) + 1e-5f);
          const float4 ya = make_float4((a[k].x - mean) * inv * vA.x + lA.x, (a[k].y - mean) * inv * vA.y + lA.y,
                                        (a[k].z - mean) * inv * vA.z + lA.z, (a[k].w - mean) * inv * vA.w + lA.w);
          const float4 yb = make_float4((b[k].x - mean) * inv * vB.x + lB.x, (b[k].y - mean) * inv * vB.y + lB.y,
                                        (b[k].z - mean) * inv * vB.z + lB.z, (b[k].w - mean) * inv * vB.w + lB.w);
          float *o = g.out + (size_t)m[k] * D;
          *reinterpret_cast<float4 *>(o + 4 * j0) = ya;
          if (has1) *reinterpret_cast<float4 *>(o + 4 * j1) = yb;
          if (g.push_table != nullptr && ma[k] != 0) {
            float *prow = g.push_table + (size_t)mb[k] * D;
            *reinterpret_cast<float4 *>(prow + 4 * j0) = ya;
            if (has1) *reinterpret_cast<float4 *>(prow + 4 * j1) = yb;
          }
          // multi-GPU exchange: the row also goes to every rank's exchange buffer (peer stores)
          for (int q = 0; q < g.peer.world; ++q) {
            float *prow = g.peer.rows[q] + g.peer.off + (size_t)m[k] * D;
            *reinterpret_cast<float4 *>(prow + 4 * j0) = ya;
            if (has1) *reinterpret_cast<float4 *>(prow + 4 * j1) = yb;
          }
        }
    } else {  // EPI_GRU: four gate columns per unit, unit = nt * 44 + j
#pragma unroll
      for (int k = 0; k < RB; ++k)
        if (ok[k]) {
          // (row of the whole list; with the multi-GPU split the row also goes to every rank's buffer)
          const size_t orow = (size_t)(g.row_stride > 1 ? m[k] * g.row_stride + g.row_off : m[k]) * D;
          if (uA < D) {
            const float rg = 1.f / (1.f + expf(-a[k].x)), z = 1.f / (1.f + expf(-a[k].y));
            const float h = (1.f - z) * tanhf(a[k].z + rg * a[k].w) + z * hA[k];
            if (g.peer.world == 0) g.out[orow + uA] = h;
            for (int q = 0; q < g.peer.world; ++q) g.peer.rows[q][g.peer.off + orow + uA] = h;
          }
          if (has1 && uB < D) {
            const float rg = 1.f / (1.f + expf(-b[k].x)), z = 1.f / (1.f + expf(-b[k].y));
            const float h = (1.f - z) * tanhf(b[k].z + rg * b[k].w) + z * hB[k];
            if (g.peer.world == 0) g.out[orow + uB] = h;
            for (int q = 0; q < g.peer.world; ++q) g.peer.rows[q][g.peer.off + orow + uB] = h;
          }
        }
    }
  }
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1) tc_gemm_kernel(Args g) {
  extern __shared__ unsigned char raw[];
  const int nt = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool producer = warp < 4 || warp >= 6;
  const int grp = warp >= 6 ? 1 : 0;
  const int pw = grp ? warp - 6 : warp;   // producer warp within its group: tile rows pw*32 .. pw*32+31
  const int rsub = lane >> 3, f = lane & 7;
  const int w0 = g.a0.width, w1 = g.a1.width, Kd = g.Kd;
  constexpr int BNv = tile_bn<EPI>();
  constexpr bool kMerger = EPI == EPI_MERGER;
  constexpr uint32_t BvLBO = BNv * 16, BvBYTES = CHUNKS * BvLBO;   // weight images of this tile width
  const int rstride = g.row_stride > 1 ? g.row_stride : 1;
  const int nkb = g.n_kblocks;

  dep_trigger();
  int M = 0;   // live rows (known after the wait below)
  // Per-tile loads that head a dependency chain (issued right after the dependency wait below, together
  // with the load of the live row count): the table row of tile row (pw*32 + lane) for the producers,
  // and the per-row inputs of the output pass (warp w writes rows w, w+10, ...; lane i holds what row
  // w + 10*i needs).  For the CTA's first tile they are issued before the live row count is known (rows
  // up to m_cap: the arrays are sized for it) and discarded afterwards if the row is not live.
  int ri0 = -1, ri1 = -1, meta_a = 0, meta_b = 0;
  float row_on = 0.f;   // merger: validity of the accumulator row this thread moves in the first epilogue
  auto prefetch_rows = [&](int m0, int limit) {
    ri0 = ri1 = -1;
    meta_a = meta_b = 0;
    if (kMerger && producer) {
      const int m = m0 + (warp & 3) * 32 + lane;
      row_on = (m < limit && (g.row_valid == nullptr || g.row_valid[m] != 0)) ? 1.f : 0.f;
    }
    if (producer) {
      const int m = m0 + pw * 32 + lane;
      if (m < limit) {
        // (row_stride > 1: this launch covers every row_stride-th row of the index lists, from row_off)
        const int mi = rstride > 1 ? min(m * rstride + g.row_off, g.idx_limit - 1) : m;
        ri0 = g.a0.idx ? g.a0.idx[mi] : (g.a0.mod > 0 ? m % g.a0.mod : m) + g.a0.add;
        if (w1) ri1 = g.a1.idx ? g.a1.idx[mi] : (g.a1.mod > 0 ? m % g.a1.mod : m) + g.a1.add;
        // an invalid row reads zeros for its first zero_cols columns: with zero_cols == a0.width (the
        // only use) that is the whole first source
        if (g.row_valid != nullptr && g.zero_cols > 0 && g.row_valid[m] == 0) ri0 = -1;
      }
    }
    const int r = warp + (THREADS / 32) * lane;
    const int m = m0 + r;
    if (r < BM && m < limit) {
      if (kMerger && g.push_table != nullptr) {
        meta_b = g.push_ids[m];
        if (g.push_win != nullptr) meta_a = g.push_win[m];
      }
      if (EPI == EPI_GRU) meta_b = g.nodes[rstride > 1 ? min(m * rstride + g.row_off, g.idx_limit - 1) : m];
    }
  };

  const uint32_t raw_addr = smem_addr(raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  const Smem sm{base};
  const uint32_t bar_base = base + (kMerger ? MERGER_RING_BYTES : STAGES * STAGE_BYTES);
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 64u + 8u * s; };
  const uint32_t accbar = bar_base + 128u;
  const uint32_t slot = bar_base + 136u;
  // merger only: k-block 0 of the second weights has landed / k-blocks 1 and 2 have landed / the hidden
  // tile is in shared memory as an A image
  const uint32_t w2bar0 = bar_base + 144u, w2bar1 = bar_base + 152u, a2bar = bar_base + 160u;
  volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(raw + (slot - raw_addr));

  // Producer lane layout inside a stage: 8 lanes cover the 256 contiguous bytes a row contributes
  // (two 16-byte loads each = one 8-element chunk), 4 rows per load instruction, 8 instructions for
  // the warp's 32 rows.  The table row of each of them comes from the lane that owns it by shuffle.
  const float4 *zero = reinterpret_cast<const float4 *>(g_zero16);
  float4 x[16];
  auto load_stage = [&](int kb) {
    const int col = kb * BK + f * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r0 = __shfl_sync(0xffffffffu, ri0, 4 * i + rsub);
      const int r1 = __shfl_sync(0xffffffffu, ri1, 4 * i + rsub);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = col + 4 * h;
        const bool in0 = c < w0;
        const int r = in0 ? r0 : r1;
        const float *bp = in0 ? g.a0.p + (size_t)r * w0 + c : g.a1.p + (size_t)r * w1 + (c - w0);
        x[2 * i + h] = *((c >= Kd || r < 0) ? zero : reinterpret_cast<const float4 *>(bp));
      }
    }
  };
  auto fix_rows = [&](int m0) {   // after the live count is known
    if (producer && m0 + pw * 32 + lane >= M) ri0 = ri1 = -1;
  };
  // (called after the tile's first stage has been requested: the lookup is two dependent loads and its
  // result is only needed by the output pass)
  auto push_winners = [&](int m0) {
    if (kMerger && g.push_table != nullptr && g.push_win == nullptr) {
      // winners by record; only for live rows: the id of a row past the live count is not a valid index
      const int r = warp + (THREADS / 32) * lane;
      const int m = m0 + r;
      if (r < BM && m < M)
        meta_a = (m >= g.push_all_from || g.push_last_pos[meta_b] == (unsigned long long)(g.push_base + m)) ? 1 : 0;
    }
  };
  // ---- set-up that reads nothing an earlier kernel wrote: barriers, tensor memory, epilogue vectors
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 4 + 1);  // one elected lane per producer warp of the group + the weight loader
      mbar_init(empty(s), 1);     // one tcgen05.commit
    }
    mbar_init(accbar, 1);
    if (kMerger) {
      mbar_init(w2bar0, 1);
      mbar_init(w2bar1, 1);
      mbar_init(a2bar, 8);   // one elected lane per producer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // epilogue vectors of this column tile, staged once (a global load per accumulator chunk would put
  // an L2 round trip into every step of the epilogue)
  __shared__ __align__(16) float s_bias[BN], s_v1[BN], s_v2[BN];
  __shared__ __align__(16) float s_out[kMerger ? 3 : 1][kMerger ? BN : 4];   // merger: bias, weight, shift of the LayerNorm
  if (warp == 4 || warp == 5) {
    const int lim = (EPI == EPI_BIAS || EPI == EPI_GRU) ? BNv : D - nt * BNv;   // columns of this tile that exist
    for (int i = tid - 128; i < BN; i += 64) {
      const bool in = i < lim && i < BNv;
      s_bias[i] = in ? g.bias[nt * BNv + i] : 0.f;
      const float *v1 = kMerger ? g.bias2 : EPI == EPI_SCORE ? g.w2 : nullptr;
      s_v1[i] = (v1 != nullptr && in) ? v1[nt * BNv + i] : 0.f;
      s_v2[i] = 0.f;
      if (kMerger) {
        s_out[0][i] = in ? g.bias_out[i] : 0.f;
        s_out[1][i] = in ? g.ln_w[i] : 0.f;
        s_out[2][i] = in ? g.ln_b[i] : 0.f;
      }
    }
  }
  // ---- everything below may read what the previous kernels of the stream produced
  dep_wait();
  prefetch_rows(blockIdx.y * BM, g.m_cap);
  M = rows_of(g.m_cap, g.d_m);
  if (rstride > 1) {   // d_m counts the rows of the whole list: this launch's share of them
    const int all = g.d_m != nullptr ? *g.d_m : g.idx_limit;
    M = min(g.m_cap, all > g.row_off ? (all - g.row_off + rstride - 1) / rstride : 0);
  }
  fix_rows(blockIdx.y * BM);
  if ((int)blockIdx.y * BM < M && producer && grp < nkb) load_stage(grp);   // in flight across the barrier
  push_winners(blockIdx.y * BM);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  bool alive = true;
  float *tile = reinterpret_cast<float *>(raw + (base - raw_addr));
  __shared__ float s_dot[2][BM];   // scorer: partial dot products of the two column halves
  // uses of stage s per tile: its k-blocks are s, s+2, ...; the barrier phase of a use is its running index
  const int uses0 = (nkb + 1) / 2, uses1 = nkb / 2;

  // A CTA walks the row blocks blockIdx.y, blockIdx.y + gridDim.y, ...: barriers, tensor memory and the
  // epilogue vectors are set up once
  for (int t = 0, mblk = blockIdx.y; mblk * BM < M; ++t, mblk += gridDim.y) {
    const int m0 = mblk * BM;
    if (t > 0) {
      prefetch_rows(m0, M);
      fix_rows(m0);
      if (producer && grp < nkb) load_stage(grp);
      push_winners(m0);
    }
    if (producer) {
      // ---------------------------------------------------------------- producer groups
      const int s = grp;
      const int u0 = t * (grp ? uses1 : uses0);
      const uint32_t st_off = (uint32_t)f * A_LBO + (uint32_t)(pw * 32 + rsub) * 16u;
      for (int kb = grp; kb < nkb; kb += 2) {
        mbar_wait(empty(s), ((u0 + (kb >> 1)) & 1) ^ 1, g.status, 100 + s, alive, g.wait_limit);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 hi, lo;
          split_chunk(x[2 * i], x[2 * i + 1], hi, lo);
          st_shared_v4(sm.a_hi(s) + st_off + i * 64u, hi);
          st_shared_v4(sm.a_lo(s) + st_off + i * 64u, lo);
        }
        fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0) mbar_arrive(full(s));
        // a thread that arrives stalls until its outstanding loads have landed, so the next stage's
        // loads go out after the arrival
        if (kb + 2 < nkb) load_stage(kb + 2);
      }
    } else if (warp == 4) {
      // ---------------------------------------------------------------- weight stages
      if (lane == 0) {
        const char *wsrc = reinterpret_cast<const char *>(g.w_packed) +
                           (size_t)nt * g.n_kblocks * (2 * BvBYTES);
        // second weights of the merger: k-block 0 once per CTA (its place lies past the stage ring), k-blocks
        // 1 and 2 into the ring as soon as the first product has finished reading it
        const char *w2 = reinterpret_cast<const char *>(g.w2_packed);
        if (kMerger && t == 0) {
          mbar_expect_tx(w2bar0, 2 * B_BYTES);
          bulk_g2s(base + W2_KB0, w2, 2 * B_BYTES, w2bar0);
        }
        for (int kb = 0; kb < nkb; ++kb) {
          const int s = kb & 1;
          const int u = t * (s ? uses1 : uses0) + (kb >> 1);
          mbar_wait(empty(s), (u & 1) ^ 1, g.status, 200 + s, alive, g.wait_limit);
          mbar_expect_tx(full(s), 2 * BvBYTES);
          bulk_g2s(sm.b_hi(s), wsrc + (size_t)kb * (2 * BvBYTES), 2 * BvBYTES, full(s));
        }
        if (kMerger) {
          mbar_wait(accbar, 0, g.status, 210, alive, g.wait_limit);
          constexpr uint32_t kTail = W2_TAIL_CHUNKS * B_LBO;
          mbar_expect_tx(w2bar1, 2 * B_BYTES + 2 * kTail);
          bulk_g2s(base + W2_KB1, w2 + 2 * B_BYTES, 2 * B_BYTES, w2bar1);
          bulk_g2s(base + W2_KB2, w2 + 4 * B_BYTES, kTail, w2bar1);
          bulk_g2s(base + W2_KB2 + kTail, w2 + 5 * B_BYTES, kTail, w2bar1);
        }
      }
      __syncwarp();
    } else {
      // ---------------------------------------------------------------- MMA issue
      if (lane == 0) {
        // fp32 accumulate, bf16 x bf16, both K-major, N = 176 (96), M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNv >> 3) << 17) |
                                   ((uint32_t)(BM >> 4) << 24);
        for (int kb = 0; kb < nkb; ++kb) {
          const int s = kb & 1;
          const int u = t * (s ? uses1 : uses0) + (kb >> 1);
          mbar_wait(full(s), u & 1, g.status, 300 + s, alive, g.wait_limit);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {
            const uint64_t ah = make_desc(sm.a_hi(s) + ks * 2 * A_LBO, A_LBO, A_SBO);
            const uint64_t al = make_desc(sm.a_lo(s) + ks * 2 * A_LBO, A_LBO, A_SBO);
            // (the tail image follows the head image of the stage copy directly)
            const uint64_t bh = make_desc(sm.b_hi(s) + ks * 2 * BvLBO, BvLBO, B_SBO);
            const uint64_t bl = make_desc(sm.b_hi(s) + BvBYTES + ks * 2 * BvLBO, BvLBO, B_SBO);
            const uint32_t first = (kb > 0 || ks > 0) ? 1u : 0u;
            mma_bf16(tmem, ah, bh, idesc, first);
            mma_bf16(tmem + TMEM_SMALL, al, bh, idesc, first);
            mma_bf16(tmem + TMEM_SMALL, ah, bl, idesc, 1u);
          }
          mma_commit(empty(s));  // the stage may be refilled once these MMAs have read it
        }
        mma_commit(accbar);
        if (kMerger) {
          // second product: hidden tile (A image written by the first epilogue) x second weights, into the
          // same accumulator columns (the first epilogue has read them when a2bar completes)
          mbar_wait(a2bar, t & 1, g.status, 310, alive, g.wait_limit);
          mbar_wait(w2bar0, 0, g.status, 311, alive, g.wait_limit);
          tc_fence_after();
          for (int ks = 0; ks < A2_CHUNKS / 2; ++ks) {
            if (ks == BK / 16) {
              mbar_wait(w2bar1, t & 1, g.status, 312, alive, g.wait_limit);
              tc_fence_after();
            }
            const int kb = ks / (BK / 16), kk = ks % (BK / 16);
            const uint32_t wb = base + (kb == 0 ? W2_KB0 : kb == 1 ? W2_KB1 : W2_KB2) + kk * 2 * B_LBO;
            const uint32_t wtail = kb == 2 ? W2_TAIL_CHUNKS * B_LBO : B_BYTES;
            const uint64_t ah = make_desc(base + ks * 2 * A_LBO, A_LBO, A_SBO);
            const uint64_t al = make_desc(base + A2_BYTES + ks * 2 * A_LBO, A_LBO, A_SBO);
            const uint64_t bh = make_desc(wb, B_LBO, B_SBO);
            const uint64_t bl = make_desc(wb + wtail, B_LBO, B_SBO);
            const uint32_t first = ks > 0 ? 1u : 0u;
            mma_bf16(tmem, ah, bh, idesc, first);
            mma_bf16(tmem + TMEM_SMALL, al, bh, idesc, first);
            mma_bf16(tmem + TMEM_SMALL, ah, bl, idesc, 1u);
          }
          mma_commit(accbar);
        }
      }
      __syncwarp();
    }

    // ------------------------------------------------------------------ epilogue
    // Pass 1 (the eight producer warps): thread = tile row = accumulator lane; a warp may only read the
    // lane quarter (warp % 4), so warps 0-3 take accumulator columns 0..95 and warps 6-9 columns
    // 96..175 of their quarter.  Values (both accumulators summed) go to a row-major tile in the now
    // idle stage ring, so that pass 2 can write whole rows with coalesced stores.
    const int m_rows = min(BM, M - m0);
    if (producer) {
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
      if (kMerger) {
        // first epilogue: hidden = relu(acc + bias + valid * bias2), split into bf16 head / tail and stored
        // as the A image of the second product (thread = row: chunk c of the row is 16 bytes at c * A_LBO)
        mbar_wait(accbar, 0, g.status, 401, alive, g.wait_limit);
        tc_fence_after();
        constexpr int kHalf = (BN / 16 + 1) / 2;
        const uint32_t arow = base + (uint32_t)row * 16u;
        for (int ch = grp ? kHalf : 0; ch < (grp ? BN / 16 : kHalf); ++ch) {
          float v[16];
          tmem_ld16_sum(trow + ch * 16, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i] + s_bias[ch * 16 + i] + row_on * s_v1[ch * 16 + i], 0.f);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4 hi, lo;
            split_chunk(make_float4(v[8 * h], v[8 * h + 1], v[8 * h + 2], v[8 * h + 3]),
                        make_float4(v[8 * h + 4], v[8 * h + 5], v[8 * h + 6], v[8 * h + 7]), hi, lo);
            st_shared_v4(arow + (uint32_t)(2 * ch + h) * A_LBO, hi);
            st_shared_v4(arow + A2_BYTES + (uint32_t)(2 * ch + h) * A_LBO, lo);
          }
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a2bar);
      }
      mbar_wait(accbar, kMerger ? 1 : (t & 1), g.status, 400, alive, g.wait_limit);
      tc_fence_after();
      const uint32_t trow_sa = base + (uint32_t)(row * TILE_LD) * 4u;   // the tile starts at the stage ring
      float dot = 0.f;
      constexpr int kSplit = (BNv / 16 + 1) / 2;   // accumulator chunks of 16 columns: first half / second half
      const int ch0 = grp ? kSplit : 0, ch1 = grp ? BNv / 16 : kSplit;
      for (int ch = ch0; ch < ch1; ++ch) {
        float v[16];
        tmem_ld16_sum(trow + ch * 16, v);
        if (EPI == EPI_SCORE) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int c = ch * 16 + i;
            if (c < D) dot += fmaxf(v[i] + s_bias[c], 0.f) * s_v1[c];
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_shared_f4(trow_sa + (uint32_t)(ch * 16 + q * 4) * 4u,
                         make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]));
        }
      }
      if (EPI == EPI_SCORE) s_dot[grp][row] = dot;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if constexpr (kMerger)
      tile_output<EPI_LAYERNORM>(g, tile, s_out[0], s_out[1], s_out[2], &s_dot[0][0], m0, m_rows, nt, warp, lane,
                                 meta_a, meta_b);
    else
      tile_output<EPI>(g, tile, s_bias, s_v1, s_v2, &s_dot[0][0], m0, m_rows, nt, warp, lane, meta_a, meta_b);
    // the tile lives in the stage ring: the next row block's bulk copies and stores may only land
    // once every warp has read it
    fence_async_smem();
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
  if ((EPI == EPI_GRU || kMerger) && g.peer.world > 0) {
    // every CTA (with or without rows) checks out; the last one posts the batch's sequence number to all
    // ranks, after every CTA's peer stores have been fenced system-wide
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
      const int n_cta = (int)(gridDim.x * gridDim.y * gridDim.z);
      if (atomicAdd(g.peer.counter, 1) == n_cta - 1) {
        *g.peer.counter = 0;
        __threadfence_system();
        for (int q = 0; q < g.peer.world; ++q)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(g.peer.flags[q] + g.peer.rank), "r"(g.peer.seq)
                       : "memory");
      }
    }
  }
}

int launch(int epilogue, const Args &a, int n_tiles, cudaStream_t stream) {
  if (a.m_cap <= 0) return ORCA_OK;
  Ctx *c = cur();
  if (c == nullptr) return set_error(ORCA_E_CUDA, "tc::launch: no context for the current device");
  static thread_local int configured_device = -1;
  if (configured_device != c->device) {
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_GRU>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_SCORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_MERGER>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   MERGER_SMEM_BYTES));
    configured_device = c->device;
  }
  Args b = a;
  b.status = c->status_word;
  b.wait_limit = c->wait_limit;
  // one wave: a CTA walks several row blocks when there are more tiles than SMs; CTAs past the live row
  // count (m_cap is a capacity) leave at once
  dim3 grid(n_tiles, std::min(ceil_div(a.m_cap, BM), std::max(1, c->sm_count / n_tiles)), 1);
  switch (epilogue) {
    case EPI_BIAS: ORCA_CUDA(launch_dep(tc_gemm_kernel<EPI_BIAS>, grid, THREADS, SMEM_BYTES, stream, b)); break;
    case EPI_GRU: ORCA_CUDA(launch_dep(tc_gemm_kernel<EPI_GRU>, grid, THREADS, SMEM_BYTES, stream, b)); break;
    case EPI_SCORE: ORCA_CUDA(launch_dep(tc_gemm_kernel<EPI_SCORE>, grid, THREADS, SMEM_BYTES, stream, b)); break;
    case EPI_MERGER:
      ORCA_CUDA(launch_dep(tc_gemm_kernel<EPI_MERGER>, grid, THREADS, MERGER_SMEM_BYTES, stream, b));
      break;
    default: return set_error(ORCA_E_BADARG, "tc::launch: unknown epilogue %d", epilogue);
  }
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace tc
}  // namespace orca
