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

// cos(x) for an fp32 argument of any magnitude up to 1e9, accurate to about 5e-7 absolute.
// The arguments here are delta * w with delta up to 3e8 seconds and w down from 1, so most of them
// are far outside the range where cosf() stays on its fast path, and its slow path (Payne-Hanek)
// costs a hundred instructions.  Here the argument is reduced in double precision --
// r = x - round(x / 2pi) * 2pi with 2pi in two doubles, exact enough for |x| < 1e9 -- and the
// hardware cosine approximation is applied to r in [-pi, pi], where its absolute error is 2^-21.
__device__ __forceinline__ float cos_any(float x) {
  if (!(fabsf(x) < 1.0e9f)) return cosf(x);
  const double xd = (double)x;
  const double k = rint(xd * 0.15915494309189533577);          // 1 / 2pi
  double r = fma(-k, 6.28318530717958623200e+00, xd);          // 2pi, high part
  r = fma(-k, 2.44929359829470641435e-16, r);                  // 2pi, low part
  return __cosf((float)r);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace orca
