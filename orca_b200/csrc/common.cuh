// Shared helpers of the orca_b200 kernels: error reporting, launch checks, small device utilities.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/orca_b200.h"

namespace orca {

constexpr int D = ORCA_DIM;          // 172 floats = 688 bytes = 43 x 16 bytes
constexpr int H = ORCA_HEADS;        // 2
constexpr int KEY = ORCA_KEY_DIM;    // 516
constexpr int QT = ORCA_QT_DIM;      // 1032
constexpr int QT_LD = ORCA_QT_LD;    // 1056: head h of a projected query starts at h * 528
constexpr int QT_HEAD = QT_LD / H;   // 528
constexpr int MSG = ORCA_MSG_DIM;    // 688
constexpr int ROW_BYTES = D * 4;     // 688

// status word layout (int32[4]): [0] first error code, [1] rows at layer 1, [2] unique positives,
// [3] detail of the error (row / id)
int set_error(int code, const char *fmt, ...);

#define ORCA_CHECK_ARG(cond)                                                        \
  do {                                                                              \
    if (!(cond)) return orca::set_error(ORCA_E_BADARG, "%s: bad argument: %s", __func__, #cond); \
  } while (0)

#define ORCA_CUDA(call)                                                             \
  do {                                                                              \
    cudaError_t e_ = (call);                                                        \
    if (e_ != cudaSuccess)                                                          \
      return orca::set_error(ORCA_E_CUDA, "%s: %s failed: %s", __func__, #call,     \
                             cudaGetErrorString(e_));                               \
  } while (0)

#define ORCA_LAUNCH_CHECK()                                                         \
  do {                                                                              \
    cudaError_t e_ = cudaGetLastError();                                            \
    if (e_ != cudaSuccess)                                                          \
      return orca::set_error(ORCA_E_CUDA, "%s: kernel launch failed: %s", __func__, \
                             cudaGetErrorString(e_));                               \
  } while (0)

// number of kernels launched by this thread since the counter was last reset
int &launch_counter();
#define ORCA_COUNT_LAUNCH() (++orca::launch_counter())

// Programmatic dependent launch: a kernel launched through launch_dep() may begin (block scheduling,
// set-up that touches nothing an earlier kernel wrote) while its predecessor in the stream is still
// draining.  EVERY such kernel calls dep_wait() before its first access to memory another kernel
// produced -- and before returning, even when it has nothing to do, so that completion stays
// transitive along the stream -- and dep_trigger() as early as it likes.  Both are no-ops in a kernel
// that was launched the plain way.
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool dependent_launch_enabled();   // switch of the context in effect (context.cuh)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (dependent_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ int rows_of(int cap, const int32_t *d_n) {
  if (d_n == nullptr) return cap;
  int n = *d_n;
  return n < cap ? n : cap;
}

__device__ __forceinline__ void report(int32_t *status, int code, int detail) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) status[3] = detail;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// cos(x) for an fp32 argument of any magnitude, accurate to about 1e-6 absolute.
// The arguments here are delta * w with delta up to 3e8 seconds and w down from 1, so many of them are
// far outside the range where cosf() stays on its fast path, and its slow path (Payne-Hanek) costs a
// hundred instructions; double-precision reduction is no way out either (the fp64 and conversion
// pipes of this GPU made a warp-wide cosine cost ~160 cycles).  fp32 and integer pipes only:
//   |x| < 2^15   Cody-Waite: k = rint(x / 2pi) (< 2^13), r = x - k*C1 - k*C2 - k*C3 with 2pi split so that
//                k*C1 and k*C2 are exact (C1 8 bits, C2 11 bits); reduction error 1e-7;
//   |x| < 2^30   fixed point: x = m * 2^e with a 24-bit m; the fraction of x / 2pi is the low part of
//                m * F (F = 2^64 / 2pi) shifted by e, of which the top 32 bits are kept (96-bit product
//                from two 32 x 32 multiplies); cos is even, so |fraction| (24 bits) goes back to a
//                float through the 2^23 exponent trick; reduction error 4e-7;
//   else         cosf().
// The hardware cosine approximation is applied to the reduced argument in [-pi, pi] (2^-21 absolute).
// |x| < 2^15, branch free
__device__ __forceinline__ float cos_small(float x) {
  const float ax = fabsf(x);
  const float k = rintf(ax * 0.15915494309189535f);
  float r = fmaf(-k, 6.28125f, ax);
  r = fmaf(-k, 0.0019350051879882812f, r);
  r = fmaf(-k, 3.019916050561733e-07f, r);
  return __cosf(r);
}
// 2^-8 <= |x| < 2^30, branch free
__device__ __forceinline__ float cos_fixed(float x) {
  const uint32_t bits = __float_as_uint(fabsf(x));
  const int e = (int)(bits >> 23) - 150;           // |x| = m * 2^e, e in [-31, 6]
  const uint32_t m = (bits & 0x7fffffu) | 0x800000u;
  const unsigned long long a = (unsigned long long)m * 0x9391054aull;   // m * low word of F
  const unsigned long long mid = (a >> 32) + (unsigned long long)m * 0x28be60dbull;
  const uint32_t w0 = (uint32_t)a, w1 = (uint32_t)mid, w2 = (uint32_t)(mid >> 32);
  // top 32 bits of frac(m * F * 2^e / 2^64)
  const uint32_t top = e >= 0 ? __funnelshift_l(w0, w1, e) : __funnelshift_r(w1, w2, -e);
  const int t = (int)top;                          // turns in [-1/2, 1/2) scaled by 2^32
  const uint32_t u = min((uint32_t)(t < 0 ? -t : t) >> 8, 0x7fffffu);
  const float f = __uint_as_float(0x4b000000u | u) - 8388608.f;   // (float)u, exact
  return __cosf(f * 3.7450702829239286e-07f);      // 2pi / 2^24
}
__device__ __forceinline__ float cos_any(float x) {
  const float ax = fabsf(x);
  if (ax < 32768.f) return cos_small(x);
  if (ax < 1073741824.f) return cos_fixed(x);
  return cosf(x);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace orca
