// Prune-range selection and the pruning gather.
//
// Replaces, in the reference's python (fast_rnnt/python/fast_rnnt/rnnt_loss.py):
//   get_rnnt_prune_ranges :726-777 with _adjust_pruning_lower_bound :617-632 and
//                          _monotonic_lower_bound :578-581 (about 15 ATen kernels)
//   do_rnnt_pruning       :810-818 (an element-wise gather driven by an
//                          expanded int64 index) and its autograd scatter-add.
//
// prune_ranges: one CTA per utterance.  Each thread owns frames t, t+256, ...:
//   it walks the S+2-R window positions, adding the R occupancies py_grad[s+k][t]
//   in the order k = 0..R-1 in the input precision (the float result decides
//   an argmax whose top-2 margin is often one ulp, so the order is part of the
//   contract), subtracts px_grad[s-1][t] and keeps the first maximum.  The two
//   reverse running minima of the monotone fix-up are block scans over the T
//   frame values kept in shared memory; everything after the argmax is integer.
//
// prune_gather: a row copy lm[b][ranges[b][t][k]][:] -> out[b][t][k][:] with
//   16-byte accesses; its backward sums, for every (b, s), the gradient rows
//   whose range entry equals s, in frame order (deterministic, no atomics).
#include "common.cuh"

namespace frnnt {

constexpr int kPruneThreads = 256;

// in place: arr[t] = min(arr[t..n-1]); every thread owns a contiguous chunk
__device__ void block_suffix_min(int *arr, int n, int *part) {
  const int tid = threadIdx.x;
  const int per = (n + kPruneThreads - 1) / kPruneThreads;
  const int lo = tid * per, hi = min(n, lo + per);
  int run = INT_MAX;
  for (int t = hi - 1; t >= lo; --t) {
    run = min(run, arr[t]);
    arr[t] = run;
  }
  part[tid] = run;
  __syncthreads();
  int carry = INT_MAX;
  for (int j = tid + 1; j < kPruneThreads; ++j) carry = min(carry, part[j]);
  for (int t = lo; t < hi; ++t) arr[t] = min(arr[t], carry);
  __syncthreads();
}

template <typename real>
__global__ void __launch_bounds__(kPruneThreads)
prune_ranges_kernel(const real *__restrict__ px_grad, const real *__restrict__ py_grad,
                    const int64_t *__restrict__ boundary, int64_t *__restrict__ ranges, int S,
                    int T, int T1, int R) {
  extern __shared__ int sm[];
  int *arr = sm;        // [T]
  int *part = sm + T;   // [kPruneThreads]
  const int b = blockIdx.x;
  const int S1 = S + 1;
  const int n_win = S1 - R + 1;
  const real *GX = px_grad + (size_t)b * S * T1;
  const real *GY = py_grad + (size_t)b * S1 * T;
  const long long Sb = boundary[4 * b + 2], Tb = boundary[4 * b + 3];
  long long pad = Sb - R + 1;
  if (pad < 0) pad = 0;
  if (pad > n_win - 1) pad = n_win - 1;  // keeps ranges inside [0, S] for malformed rows

  for (int t = threadIdx.x; t < T; t += kPruneThreads) {
    int best_s = 0;
    if ((long long)t < Tb - 1) {
      real best = 0;
      for (int s = 0; s < n_win; ++s) {
        real acc = GY[(size_t)s * T + t];
        for (int k = 1; k < R; ++k) acc = acc + GY[(size_t)(s + k) * T + t];
        const real score = acc - (s == 0 ? (real)0 : GX[(size_t)(s - 1) * T1 + t]);
        if (s == 0 || score > best) {
          best = score;
          best_s = s;
        }
      }
    } else {
      best_s = (int)pad;
    }
    arr[t] = best_s;
  }
  __syncthreads();

  // _adjust_pruning_lower_bound with window 2 (modified shapes) or R (regular)
  const int step = (T1 == T ? 2 : R) - 1;
  block_suffix_min(arr, T, part);
  for (int t = threadIdx.x; t < T; t += kPruneThreads) arr[t] = step * t - arr[t];
  __syncthreads();
  block_suffix_min(arr, T, part);
  for (int t = threadIdx.x; t < T; t += kPruneThreads) arr[t] = step * t - max(arr[t], 0);
  __syncthreads();

  int64_t *out = ranges + (size_t)b * T * R;
  for (int idx = threadIdx.x; idx < T * R; idx += kPruneThreads)
    out[idx] = (int64_t)arr[idx / R] + (idx % R);
}

// out[b][t][k][:] = lm[b][ranges[b][t][k]][:]
template <typename vec>
__global__ void prune_gather_kernel(const vec *__restrict__ lm, const int64_t *__restrict__ ranges,
                                    vec *__restrict__ out, long long rows, int TR, int S1,
                                    int dvec) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const long long b = row / TR;
    long long s = ranges[row];
    s = s < 0 ? 0 : (s >= S1 ? S1 - 1 : s);  // never read outside lm
    const vec *src = lm + ((size_t)b * S1 + s) * dvec;
    vec *dst = out + (size_t)row * dvec;
    for (int v = lane; v < dvec; v += 32) dst[v] = src[v];
  }
}

// lm_grad[b][s][:] = sum over (t,k) with ranges[b][t][k] == s of g[b][t][k][:]
template <typename real>
__global__ void __launch_bounds__(128)
prune_gather_backward_kernel(const real *__restrict__ g, const int64_t *__restrict__ ranges,
                             real *__restrict__ lm_grad, int TR, int S1, int D) {
  constexpr int kEntries = 2048;
  __shared__ int sm_s[kEntries];
  const int b = blockIdx.y, s = blockIdx.x;
  const int64_t *rg = ranges + (size_t)b * TR;
  const real *G = g + (size_t)b * TR * D;
  real *out = lm_grad + ((size_t)b * S1 + s) * D;
  for (int d0 = 0; d0 < D; d0 += 4 * 128) {
    real acc[4] = {0, 0, 0, 0};
    for (int base = 0; base < TR; base += kEntries) {
      const int n = min(kEntries, TR - base);
      __syncthreads();
      for (int e = threadIdx.x; e < n; e += 128) sm_s[e] = (int)rg[base + e];
      __syncthreads();
      for (int e = 0; e < n; ++e) {
        if (sm_s[e] == s) {
          const real *row = G + (size_t)(base + e) * D;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int d = d0 + j * 128 + threadIdx.x;
            if (d < D) acc[j] += row[d];
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = d0 + j * 128 + threadIdx.x;
      if (d < D) out[d] = acc[j];
    }
  }
}

}  // namespace frnnt

using namespace frnnt;

extern "C" int frnnt_prune_ranges(int dtype, const void *px_grad, const void *py_grad,
                                  const int64_t *boundary, int64_t *ranges, int B, int S, int T,
                                  int T1, int s_range, void *stream) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(B >= 0 && S >= 1 && T >= 1, FRNNT_EINVAL, "bad sizes B=%d S=%d T=%d", B, S, T);
  FRNNT_REQUIRE(T1 == T || T1 == T + 1, FRNNT_EINVAL, "px_grad must have T or T+1 columns");
  FRNNT_REQUIRE(s_range >= 1 && s_range <= S + 1, FRNNT_EINVAL,
                "s_range=%d outside [1, S+1=%d] (adjust it on the host first)", s_range, S + 1);
  FRNNT_REQUIRE(px_grad && py_grad && boundary && ranges, FRNNT_EINVAL, "NULL argument");
  const size_t smem = (size_t)(T + kPruneThreads) * sizeof(int);
  FRNNT_REQUIRE(smem <= 200 * 1024, FRNNT_EUNSUPPORTED, "T=%d too long for one CTA's scan", T);
  if (B == 0) return FRNNT_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FRNNT_F32) {
    auto kern = prune_ranges_kernel<float>;
    if (smem > 48 * 1024)
      FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FRNNT_KERNEL(kern<<<B, kPruneThreads, smem, st>>>((const float *)px_grad, (const float *)py_grad, boundary,
                                         ranges, S, T, T1, s_range));
  } else {
    auto kern = prune_ranges_kernel<double>;
    if (smem > 48 * 1024)
      FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FRNNT_KERNEL(kern<<<B, kPruneThreads, smem, st>>>((const double *)px_grad, (const double *)py_grad,
                                         boundary, ranges, S, T, T1, s_range));
  }
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_prune_gather(int dtype, const void *lm, const int64_t *ranges, void *out,
                                  int B, int S1, int T, int R, int D, void *stream) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(B >= 0 && S1 >= 1 && T >= 0 && R >= 1 && D >= 1, FRNNT_EINVAL, "bad sizes");
  const long long rows = (long long)B * T * R;
  if (rows == 0) return FRNNT_OK;
  FRNNT_REQUIRE(lm && ranges && out, FRNNT_EINVAL, "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t row_bytes = (size_t)D * dtype_size(dtype);
  long long want = (rows + 7) / 8;
  const int grid = (int)(want < 148LL * 32 ? want : 148LL * 32);
  if (row_bytes % 16 == 0 && (uintptr_t)lm % 16 == 0 && (uintptr_t)out % 16 == 0) {
    FRNNT_KERNEL(prune_gather_kernel<float4><<<grid, 256, 0, st>>>((const float4 *)lm, ranges, (float4 *)out,
                                                     rows, T * R, S1, (int)(row_bytes / 16)));
  } else if (dtype == FRNNT_F32) {
    FRNNT_KERNEL(prune_gather_kernel<float><<<grid, 256, 0, st>>>((const float *)lm, ranges, (float *)out, rows,
                                                    T * R, S1, D));
  } else {
    FRNNT_KERNEL(prune_gather_kernel<double><<<grid, 256, 0, st>>>((const double *)lm, ranges, (double *)out,
                                                     rows, T * R, S1, D));
  }
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_prune_gather_backward(int dtype, const void *out_grad, const int64_t *ranges,
                                           void *lm_grad, int B, int S1, int T, int R, int D,
                                           void *stream) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(B >= 0 && S1 >= 1 && T >= 0 && R >= 1 && D >= 1, FRNNT_EINVAL, "bad sizes");
  FRNNT_REQUIRE(B <= 65535, FRNNT_EUNSUPPORTED, "B too large for the grid");
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(lm_grad && (ranges || T == 0) && (out_grad || T == 0), FRNNT_EINVAL,
                "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)S1, (unsigned)B);
  if (dtype == FRNNT_F32)
    FRNNT_KERNEL(prune_gather_backward_kernel<float><<<grid, 128, 0, st>>>((const float *)out_grad, ranges,
                                                             (float *)lm_grad, T * R, S1, D));
  else
    FRNNT_KERNEL(prune_gather_backward_kernel<double><<<grid, 128, 0, st>>>((const double *)out_grad, ranges,
                                                              (double *)lm_grad, T * R, S1, D));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}
