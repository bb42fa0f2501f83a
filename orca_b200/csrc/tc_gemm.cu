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
// Tile: 128 rows x 176 columns per CTA, K consumed 64 elements per stage (4 MMA steps of K = 16,
// 12 MMAs), two stages.  Every hop over an mbarrier costs ~250-300 cycles and a thread that arrives
// on one stalls until its outstanding global loads have landed, so stages are large and the A side
// is produced by two warp groups that alternate stages: while one group waits for its loads, the
// other converts and the tensor core works on the stage before.
// Warp roles (320 threads):
//   warps 0-3, 6-9  producer groups 0 / 1: group g fills stage g for every k-block kb = g (mod 2).
//              A lane loads 16-byte pieces of the gathered rows (16 lanes cover the 256 contiguous
//              bytes a row contributes to the stage; table rows picked by an index array, up to two
//              tables concatenated along K), splits them and stores head and tail in the no-swizzle
//              K-major core-matrix layout the MMA reads.  Group 0 later runs the epilogue (warp w
//              owns accumulator lanes 32w..32w+31 = tile rows).
//   warp 4     streams the packed weight stage (one 44 KB bulk copy per stage).
//   warp 5     allocates tensor memory and issues the MMAs (one thread), releasing each stage with
//              tcgen05.commit.
//
// Every wait on an mbarrier is bounded; a wait that gives up records ORCA_E_TIMEOUT and the kernel
// runs to its end (tensor memory is always released).
#include <algorithm>
#include <cuda_bf16.h>

#include "common.cuh"
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
// bounded wait (about a second of SM clocks); records the failure if the barrier never flipped.
// `alive` makes the failure sticky: a thread that gave up once does not wait again, so a broken
// pipeline drains in about a second instead of one time-out per stage.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int32_t *status, int where, bool &alive) {
  if (!alive) return;
  if (mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > 2000000000ll) {
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

// x ~ head + tail, both bf16 (round to nearest even); returns the two pairs packed for an 8-byte store
__device__ __forceinline__ void split_bf16(const float4 x, uint2 &hi, uint2 &lo) {
  const __nv_bfloat16 h0 = __float2bfloat16_rn(x.x), h1 = __float2bfloat16_rn(x.y), h2 = __float2bfloat16_rn(x.z),
                      h3 = __float2bfloat16_rn(x.w);
  const __nv_bfloat16 l0 = __float2bfloat16_rn(x.x - __bfloat162float(h0)),
                      l1 = __float2bfloat16_rn(x.y - __bfloat162float(h1)),
                      l2 = __float2bfloat16_rn(x.z - __bfloat162float(h2)),
                      l3 = __float2bfloat16_rn(x.w - __bfloat162float(h3));
  hi.x = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
  hi.y = (uint32_t)__bfloat16_as_ushort(h2) | ((uint32_t)__bfloat16_as_ushort(h3) << 16);
  lo.x = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
  lo.y = (uint32_t)__bfloat16_as_ushort(l2) | ((uint32_t)__bfloat16_as_ushort(l3) << 16);
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

__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}

__device__ __align__(16) float g_zero16[4] = {0.f, 0.f, 0.f, 0.f};

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1) tc_gemm_kernel(Args g) {
  extern __shared__ unsigned char raw[];
  const int M = rows_of(g.m_cap, g.d_m);
  const int m0 = blockIdx.y * BM;
  if (m0 >= M) return;  // nothing allocated yet
  const int nt = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const uint32_t raw_addr = smem_addr(raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  const Smem sm{base};
  const uint32_t bar_base = base + STAGES * STAGE_BYTES;
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 64u + 8u * s; };
  const uint32_t accbar = bar_base + 128u;
  const uint32_t slot = bar_base + 136u;
  volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(raw + (slot - raw_addr));

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 4 + 1);  // one elected lane per producer warp of the group + the weight loader
      mbar_init(empty(s), 1);     // one tcgen05.commit
    }
    mbar_init(accbar, 1);
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
  if (tid >= 192) {   // warps 6-9
    const int lim = (EPI == EPI_BIAS || EPI == EPI_GRU) ? BN : D;
    for (int i = tid - 192; i < BN; i += 128) {
      const bool in = i < lim;
      s_bias[i] = in ? g.bias[nt * BN + i] : 0.f;
      const float *v1 = EPI == EPI_HIDDEN ? g.bias2 : EPI == EPI_LAYERNORM ? g.ln_w : EPI == EPI_SCORE ? g.w2 : nullptr;
      s_v1[i] = (v1 != nullptr && in) ? v1[i] : 0.f;
      s_v2[i] = (EPI == EPI_LAYERNORM && in) ? g.ln_b[i] : 0.f;
    }
  }
  // per-row source pointers of the tile, resolved once (index arrays, validity)
  __shared__ const float *s_p0[BM];
  __shared__ const float *s_p1[BM];
  if (tid < BM) {
    const int m = m0 + tid;
    const float *q0 = g_zero16, *q1 = g_zero16;
    if (m < M) {
      q0 = src_row(g.a0, m);
      if (g.a1.width) q1 = src_row(g.a1, m);
      // an invalid row reads zeros for its first zero_cols columns: with zero_cols == a0.width (the
      // only use) that is the whole first source
      if (g.row_valid != nullptr && g.row_valid[m] == 0 && g.zero_cols > 0) q0 = nullptr;
    } else {
      q0 = nullptr;
      q1 = nullptr;
    }
    s_p0[tid] = q0;
    s_p1[tid] = q1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  const int nkb = g.n_kblocks;
  bool alive = true;

  if (warp < 4 || warp >= 6) {
    // ------------------------------------------------------------------ producer groups
    const int grp = warp >= 6 ? 1 : 0;
    const int pw = grp ? warp - 6 : warp;  // warp within the group: rows pw*32 .. pw*32+31
    const int half = lane >> 4;            // which of the two rows of a load instruction
    const int f = lane & 15;               // 16-byte piece of the row's 256-byte stage segment
    const uint32_t piece_off = (uint32_t)(f >> 1) * A_LBO + (uint32_t)(f & 1) * 8u;
    for (int kb = grp; kb < nkb; kb += 2) {
      const int s = grp;
      const int col = kb * BK + f * 4;
      // issue the 16 loads of this lane (rows pw*32 + 2i + half), addresses selected up front so
      // that nothing consumes a loaded register before all loads are in flight
      float4 x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int r = pw * 32 + 2 * i + half;
        const float *rowp = nullptr;
        int c = col;
        if (col < g.a0.width) rowp = s_p0[r];
        else if (col < g.Kd) { rowp = s_p1[r]; c = col - g.a0.width; }
        const float4 *src = rowp ? reinterpret_cast<const float4 *>(rowp + c)
                                 : reinterpret_cast<const float4 *>(g_zero16);
        x[i] = *src;
      }
      mbar_wait(empty(s), ((kb >> 1) & 1) ^ 1, g.status, 100 + s, alive);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int r = pw * 32 + 2 * i + half;
        uint2 hi, lo;
        split_bf16(x[i], hi, lo);
        const uint32_t off = piece_off + (uint32_t)(r >> 3) * A_SBO + (uint32_t)(r & 7) * 16u;
        st_shared_v2(sm.a_hi(s) + off, hi);
        st_shared_v2(sm.a_lo(s) + off, lo);
      }
      fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async-proxy reads
      __syncwarp();
      if (lane == 0) mbar_arrive(full(s));
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ weight stages
    if (lane == 0) {
      const char *wsrc = reinterpret_cast<const char *>(g.w_packed) + (size_t)nt * nkb * (2 * B_BYTES);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb & 1;
        mbar_wait(empty(s), ((kb >> 1) & 1) ^ 1, g.status, 200 + s, alive);
        mbar_expect_tx(full(s), 2 * B_BYTES);
        bulk_g2s(sm.b_hi(s), wsrc + (size_t)kb * (2 * B_BYTES), 2 * B_BYTES, full(s));
      }
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // fp32 accumulate, bf16 x bf16, both K-major, N = 176, M = 128
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)(BM >> 4) << 24);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb & 1;
        mbar_wait(full(s), (kb >> 1) & 1, g.status, 300 + s, alive);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
          const uint64_t ah = make_desc(sm.a_hi(s) + ks * 2 * A_LBO, A_LBO, A_SBO);
          const uint64_t al = make_desc(sm.a_lo(s) + ks * 2 * A_LBO, A_LBO, A_SBO);
          const uint64_t bh = make_desc(sm.b_hi(s) + ks * 2 * B_LBO, B_LBO, B_SBO);
          const uint64_t bl = make_desc(sm.b_lo(s) + ks * 2 * B_LBO, B_LBO, B_SBO);
          const uint32_t first = (kb > 0 || ks > 0) ? 1u : 0u;
          mma_bf16(tmem, ah, bh, idesc, first);
          mma_bf16(tmem + TMEM_SMALL, al, bh, idesc, first);
          mma_bf16(tmem + TMEM_SMALL, ah, bl, idesc, 1u);
        }
        mma_commit(empty(s));  // the stage may be refilled once these MMAs have read it
      }
      mma_commit(accbar);
    }
  }

  if (warp < 4) {
    // ------------------------------------------------------------------ epilogue: thread = tile row
    mbar_wait(accbar, 0, g.status, 400, alive);
    tc_fence_after();
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16);
    const int m = m0 + tid;
    const bool live = m < M;
    const int c0 = nt * BN;
    float v[16];
    if (EPI == EPI_BIAS) {
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
        if (live) {
          float *o = g.out + (size_t)m * g.out_ld + c0 + ch * 16;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 b = *reinterpret_cast<const float4 *>(&s_bias[ch * 16 + q * 4]);
            *reinterpret_cast<float4 *>(o + q * 4) =
                make_float4(v[q * 4] + b.x, v[q * 4 + 1] + b.y, v[q * 4 + 2] + b.z, v[q * 4 + 3] + b.w);
          }
        }
      }
    } else if (EPI == EPI_HIDDEN) {
      const float rvf = (live && (g.row_valid == nullptr || g.row_valid[m] != 0)) ? 1.f : 0.f;
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
        if (live) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int c = ch * 16 + q * 4;
            if (c < D) {
              const float4 b = *reinterpret_cast<const float4 *>(&s_bias[c]);
              const float4 b2 = *reinterpret_cast<const float4 *>(&s_v1[c]);
              *reinterpret_cast<float4 *>(g.out + (size_t)m * D + c) =
                  make_float4(fmaxf(v[q * 4] + b.x + rvf * b2.x, 0.f), fmaxf(v[q * 4 + 1] + b.y + rvf * b2.y, 0.f),
                              fmaxf(v[q * 4 + 2] + b.z + rvf * b2.z, 0.f), fmaxf(v[q * 4 + 3] + b.w + rvf * b2.w, 0.f));
            }
          }
        }
      }
    } else if (EPI == EPI_LAYERNORM) {
      // one pass over the accumulator for both moments (the row is O(1) after the merger, so
      // E[y^2] - mean^2 loses nothing that matters at the 1e-5 epsilon)
      float sum = 0.f, sumsq = 0.f;
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (ch * 16 + i < D) {
            const float y = v[i] + s_bias[ch * 16 + i];
            sum += y;
            sumsq = fmaf(y, y, sumsq);
          }
      }
      const float mean = sum * (1.f / D);
      const float sq = fmaxf(sumsq - sum * mean, 0.f);
      const float inv = 1.f / sqrtf(sq * (1.f / D) + 1e-5f);
      const bool push = live && g.push_table != nullptr && g.push_win[m] != 0;
      float *prow = push ? g.push_table + (size_t)g.push_ids[m] * D : nullptr;
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
        if (live) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int c = ch * 16 + q * 4;
            if (c < D) {
              const float4 b = *reinterpret_cast<const float4 *>(&s_bias[c]);
              const float4 w = *reinterpret_cast<const float4 *>(&s_v1[c]);
              const float4 lb = *reinterpret_cast<const float4 *>(&s_v2[c]);
              const float4 o = make_float4((v[q * 4] + b.x - mean) * inv * w.x + lb.x,
                                           (v[q * 4 + 1] + b.y - mean) * inv * w.y + lb.y,
                                           (v[q * 4 + 2] + b.z - mean) * inv * w.z + lb.z,
                                           (v[q * 4 + 3] + b.w - mean) * inv * w.w + lb.w);
              *reinterpret_cast<float4 *>(g.out + (size_t)m * D + c) = o;
              if (push) *reinterpret_cast<float4 *>(prow + c) = o;
            }
          }
        }
      }
    } else if (EPI == EPI_GRU) {
      const float *hrow = live ? g.memory + (size_t)g.nodes[m] * D : nullptr;
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
        if (live) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int u = nt * (BN / 4) + ch * 4 + q;  // GRU unit of these four gate columns
            if (u < D) {
              const float4 b = *reinterpret_cast<const float4 *>(&s_bias[ch * 16 + q * 4]);
              const float r = 1.f / (1.f + expf(-(v[q * 4] + b.x)));
              const float z = 1.f / (1.f + expf(-(v[q * 4 + 1] + b.y)));
              const float nn = tanhf((v[q * 4 + 2] + b.z) + r * (v[q * 4 + 3] + b.w));
              g.out[(size_t)m * D + u] = (1.f - z) * nn + z * hrow[u];
            }
          }
        }
      }
    } else {  // EPI_SCORE
      float part = 0.f;
      for (int ch = 0; ch < BN / 16; ++ch) {
        tmem_ld16_sum(trow + ch * 16, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int c = ch * 16 + i;
          if (c < D) part += fmaxf(v[i] + s_bias[c], 0.f) * s_v1[c];
        }
      }
      if (live) g.out[m] = 1.f / (1.f + expf(-(part + g.b2)));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

int launch(int epilogue, const Args &a, int n_tiles, cudaStream_t stream) {
  if (a.m_cap <= 0) return ORCA_OK;
  static thread_local int configured_device = -1;
  int dev = 0;
  ORCA_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_HIDDEN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_LAYERNORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_GRU>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    ORCA_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<EPI_SCORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured_device = dev;
  }
  dim3 grid(n_tiles, ceil_div(a.m_cap, BM));
  switch (epilogue) {
    case EPI_BIAS: tc_gemm_kernel<EPI_BIAS><<<grid, THREADS, SMEM_BYTES, stream>>>(a); break;
    case EPI_HIDDEN: tc_gemm_kernel<EPI_HIDDEN><<<grid, THREADS, SMEM_BYTES, stream>>>(a); break;
    case EPI_LAYERNORM: tc_gemm_kernel<EPI_LAYERNORM><<<grid, THREADS, SMEM_BYTES, stream>>>(a); break;
    case EPI_GRU: tc_gemm_kernel<EPI_GRU><<<grid, THREADS, SMEM_BYTES, stream>>>(a); break;
    case EPI_SCORE: tc_gemm_kernel<EPI_SCORE><<<grid, THREADS, SMEM_BYTES, stream>>>(a); break;
    default: return set_error(ORCA_E_BADARG, "tc::launch: unknown epilogue %d", epilogue);
  }
  ORCA_COUNT_LAUNCH();
  ORCA_LAUNCH_CHECK();
  return ORCA_OK;
}

}  // namespace tc
}  // namespace orca
