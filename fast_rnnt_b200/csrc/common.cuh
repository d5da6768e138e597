// Shared host/device helpers of libfrnnt_sm100.so.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "frnnt.h"

namespace frnnt {

// ---- host: error reporting --------------------------------------------------
void set_error(const char *fmt, ...);

#define FRNNT_REQUIRE(cond, code, ...)      \
  do {                                      \
    if (!(cond)) {                          \
      ::frnnt::set_error(__VA_ARGS__);      \
      return (code);                        \
    }                                       \
  } while (0)

#define FRNNT_CUDA(call)                                                        \
  do {                                                                          \
    cudaError_t err__ = (call);                                                 \
    if (err__ != cudaSuccess) {                                                 \
      ::frnnt::set_error("%s failed: %s", #call, cudaGetErrorString(err__));    \
      return FRNNT_ECUDA;                                                       \
    }                                                                           \
  } while (0)

// every kernel launch goes through this macro so that callers can ask how many
// kernels the library has launched (frnnt_launch_count)
void count_launch();
#define FRNNT_KERNEL(...) (::frnnt::count_launch(), __VA_ARGS__)

// multiprocessors of the current device (queried once per device; 148 on a B200);
// a fallback of 148 if the query fails, since grid sizes are only a tuning matter
int sm_count();

inline int check_dtype(int dtype) { return dtype == FRNNT_F32 || dtype == FRNNT_F64; }
inline size_t dtype_size(int dtype) { return dtype == FRNNT_F64 ? 8 : 4; }

// ---- device: inputs that may be 16-bit (FRNNT_F16 / FRNNT_BF16), read as float32 ------------
__device__ __forceinline__ float in_f32(float x) { return x; }
__device__ __forceinline__ float in_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float in_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
// four consecutive values starting at element 4 * v of a row (16- resp. 8-byte aligned)
__device__ __forceinline__ float4 in_load4(const float *row, int v) {
  return reinterpret_cast<const float4 *>(row)[v];
}
__device__ __forceinline__ float4 in_load4(const __half *row, int v) {
  const uint2 q = reinterpret_cast<const uint2 *>(row)[v];
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&q.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&q.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 in_load4(const __nv_bfloat16 *row, int v) {
  const uint2 q = reinterpret_cast<const uint2 *>(row)[v];
  // a bfloat16 is the upper half of a float32
  return make_float4(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xffff0000u),
                     __uint_as_float(q.y << 16), __uint_as_float(q.y & 0xffff0000u));
}
inline bool is_half_input(int dtype) { return dtype == FRNNT_F16 || dtype == FRNNT_BF16; }

// row / d and row % d for a row index that is 64 bits wide for safety but nearly always fits
// 32: the 32-bit division is an order of magnitude fewer instructions than the 64-bit one
__device__ __forceinline__ long long div_rows(long long row, int d) {
  return (unsigned long long)row <= 0xffffffffull ? (long long)((unsigned)row / (unsigned)d) : row / d;
}
__device__ __forceinline__ int mod_rows(long long row, int d) {
  return (unsigned long long)row <= 0xffffffffull ? (int)((unsigned)row % (unsigned)d) : (int)(row % d);
}

// ---- device: math in the reference's operation order ------------------------
template <typename real> __device__ __forceinline__ real neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double neg_inf<double>() { return -(double)INFINITY; }

__device__ __forceinline__ float exp_r(float x) { return expf(x); }
__device__ __forceinline__ double exp_r(double x) { return exp(x); }
// exp for sums of many terms (softmax denominators): one FMUL + MUFU.EX2, relative
// error ~2^-21, far below the 1e-5 tolerance of the log-sum; double stays exact.
__device__ __forceinline__ float exp_sum(float x) { return __expf(x); }
__device__ __forceinline__ double exp_sum(double x) { return exp(x); }
__device__ __forceinline__ float log1p_r(float x) { return log1pf(x); }
__device__ __forceinline__ double log1p_r(double x) { return log1p(x); }
__device__ __forceinline__ float log_r(float x) { return logf(x); }
__device__ __forceinline__ double log_r(double x) { return log(x); }

// log(exp(x) + exp(y)) with the guards of the reference's LogAdd
// (fast_rnnt/csrc/mutual_information.h:36-65): when the difference is not
// finite (an operand is -inf) the larger operand is returned unchanged.
template <typename real>
__device__ __forceinline__ real log_add(real x, real y) {
  // same arithmetic as the reference (larger + log1p(exp(smaller - larger))), written
  // without divergent branches: the guard is a select on the finished result
  const real hi = x < y ? y : x;
  const real diff = x < y ? x - y : y - x;
  const real r = hi + log1p_r(exp_r(diff));
  return (diff - diff != 0) ? hi : r;
}

template <typename T>
__device__ __forceinline__ T warp_max(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace frnnt
