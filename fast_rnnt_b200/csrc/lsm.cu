// Log-softmax over the vocabulary fused with the symbol / blank gather, for the
// pruned joiner output [B][T][R][C] and the unpruned one [B][T][S+1][C].
//
// Replaces, in the reference's python (fast_rnnt/python/fast_rnnt/rnnt_loss.py):
//   get_rnnt_logprobs_pruned :940-1017  (logsumexp, two gathers, -inf padding,
//                                        roll by ranges[:, :, 0], permutes)
//   get_rnnt_logprobs_joint  :418-442   (same without pruning)
// and the autograd graph behind them.
//
// Stage 1 (HBM bound, the only pass over the logits): one group of threads per
//   row of C logits keeps the row in registers, reduces max and sum(exp) and
//   emits three numbers per row: lse, logit[symbol]-lse, logit[blank]-lse.
// Stage 2 (small): the [B][T][R] bands are placed into the lattices
//   px [B][S][T1] and py [B][S+1][T] at row (ranges[b][t][0] + k) mod (S+1),
//   -inf elsewhere, with the -inf column at t = T (regular), the -inf at
//   t = t_end (regular + boundary) and px += py[s+1] (constrained).
// Backward (HBM bound, one read of the logits and one write of their gradient):
//   g[row][c] = -(gx+gy) * exp(logit - lse) + gx*[c == symbol] + gy*[c == blank]
//   with gx, gy picked out of the lattice gradients by the inverse placement.
#include "common.cuh"
#include "lsm_band.cuh"

namespace frnnt {

template <typename real, int VW> struct VecT;
template <> struct VecT<float, 4> { using type = float4; };
template <> struct VecT<float, 1> { using type = float; };
template <> struct VecT<double, 2> { using type = double2; };
template <> struct VecT<double, 1> { using type = double; };

template <typename real> __device__ __forceinline__ real elem(const float4 &v, int i) {
  return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}
template <typename real> __device__ __forceinline__ real elem(const double2 &v, int i) {
  return i == 0 ? v.x : v.y;
}
template <typename real> __device__ __forceinline__ real elem(const float &v, int) { return v; }
template <typename real> __device__ __forceinline__ real elem(const double &v, int) { return v; }

__device__ __forceinline__ void set_elem(float4 &v, int i, float x) {
  if (i == 0) v.x = x; else if (i == 1) v.y = x; else if (i == 2) v.z = x; else v.w = x;
}
__device__ __forceinline__ void set_elem(double2 &v, int i, double x) {
  if (i == 0) v.x = x; else v.y = x;
}
__device__ __forceinline__ void set_elem(float &v, int, float x) { v = x; }
__device__ __forceinline__ void set_elem(double &v, int, double x) { v = x; }

constexpr int kRowCta = 256;  // threads per CTA of the row kernels
constexpr int kRowCache = 8;  // vectors a thread keeps in registers

template <typename real, int GROUP>
__device__ __forceinline__ real group_reduce(real v, bool is_max, real *scratch, int gid, int lane_in_group) {
  // reduce inside each warp, then across the GROUP/32 warps of the group
  v = is_max ? warp_max(v) : warp_sum(v);
  if (GROUP > 32) {
    constexpr int WPG = GROUP / 32;
    __syncthreads();
    if ((lane_in_group & 31) == 0) scratch[gid * WPG + lane_in_group / 32] = v;
    __syncthreads();
    real r = scratch[gid * WPG];
#pragma unroll
    for (int w = 1; w < WPG; ++w) {
      const real o = scratch[gid * WPG + w];
      r = is_max ? max(r, o) : r + o;
    }
    v = r;
  }
  return v;
}

// Stage 1.  rows = B*T*R, one GROUP of threads per row.
// CACHE: vectors a thread keeps of its row (4 when the row fits: fewer registers,
// more rows in flight per SM)
template <typename real, int VW, int GROUP, int CACHE>
__global__ void __launch_bounds__(kRowCta, CACHE == 4 ? 5 : 4)
lsm_rows_forward_kernel(const real *__restrict__ logits, const int64_t *__restrict__ symbols,
                        const int64_t *__restrict__ ranges, real *__restrict__ lse,
                        real *__restrict__ pxb, real *__restrict__ pyb, long long rows, int T,
                        int R, int S, int C, int blank) {
  using vec = typename VecT<real, VW>::type;
  constexpr int GPC = kRowCta / GROUP;  // groups (rows) per CTA
  __shared__ real scratch[kRowCta / 32];
  const int gid = threadIdx.x / GROUP, lig = threadIdx.x % GROUP;
  const int nvec = C / VW;
  const bool cached = nvec <= GROUP * CACHE;
  const real ninf = neg_inf<real>();

  for (long long row0 = (long long)blockIdx.x * GPC; row0 < rows; row0 += (long long)gridDim.x * GPC) {
    const long long row = row0 + gid;
    const bool valid = row < rows;
    const vec *src = reinterpret_cast<const vec *>(logits + (valid ? row : 0) * (long long)C);
    vec reg[CACHE];
    real m = ninf;
    if (cached) {
#pragma unroll
      for (int j = 0; j < CACHE; ++j) {
        const int v = lig + j * GROUP;
        if (valid && v < nvec) {
          reg[j] = src[v];
#pragma unroll
          for (int e = 0; e < VW; ++e) m = max(m, elem<real>(reg[j], e));
        }
      }
    } else if (valid) {
      for (int v = lig; v < nvec; v += GROUP) {
        const vec x = src[v];
#pragma unroll
        for (int e = 0; e < VW; ++e) m = max(m, elem<real>(x, e));
      }
    }
    m = group_reduce<real, GROUP>(m, true, scratch, gid, lig);
    // torch.logsumexp: an infinite maximum is replaced by 0 before subtracting
    const real m0 = (m - m != 0) ? (real)0 : m;
    real sum = 0;
    if (cached) {
#pragma unroll
      for (int j = 0; j < CACHE; ++j) {
        const int v = lig + j * GROUP;
        if (valid && v < nvec) {
#pragma unroll
          for (int e = 0; e < VW; ++e) sum += exp_sum(elem<real>(reg[j], e) - m0);
        }
      }
    } else if (valid) {
      for (int v = lig; v < nvec; v += GROUP) {
        const vec x = src[v];
#pragma unroll
        for (int e = 0; e < VW; ++e) sum += exp_sum(elem<real>(x, e) - m0);
      }
    }
    sum = group_reduce<real, GROUP>(sum, false, scratch, gid, lig);
    if (valid && lig == 0) {
      const real l = log_r(sum) + m0;
      const long long bt = div_rows(row, R);
      const int k = mod_rows(row, R);
      const int b = (int)div_rows(bt, T);
      const int y = band_symbol(symbols, ranges, b, (size_t)row, k, S, blank, C);
      const real *x = logits + row * (long long)C;
      lse[row] = l;
      pxb[row] = x[y] - l;
      pyb[row] = x[blank] - l;
    }
  }
}

// Backward: one warp per row, streaming.
template <typename real, int VW>
__global__ void __launch_bounds__(kRowCta)
lsm_rows_backward_kernel(const real *__restrict__ logits, const int64_t *__restrict__ symbols,
                         const int64_t *__restrict__ ranges, const int64_t *__restrict__ boundary,
                         const real *__restrict__ lse, const real *__restrict__ g_px,
                         const real *__restrict__ g_py, real *__restrict__ g_logits,
                         long long rows, int T, int R, int S, int C, int blank, int rnnt_type) {
  using vec = typename VecT<real, VW>::type;
  const int lane = threadIdx.x & 31;
  const int S1 = S + 1;
  const int T1 = (rnnt_type == FRNNT_REGULAR) ? T + 1 : T;
  const int nvec = C / VW;
  const long long warp0 = ((long long)blockIdx.x * kRowCta + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * kRowCta) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const long long bt = div_rows(row, R);
    const int k = mod_rows(row, R);
    const int b = (int)div_rows(bt, T), t = mod_rows(bt, T);
    const int s = band_row(ranges, (size_t)bt, R, k, S1);
    real gx = 0, gy = 0;
    {
      gy = g_py[((size_t)b * S1 + s) * T + t];
      const bool masked = rnnt_type == FRNNT_REGULAR && boundary != nullptr &&
                          (long long)t == (long long)boundary[4 * b + 3];
      if (s < S && !masked) gx = g_px[((size_t)b * S + s) * T1 + t];
      if (rnnt_type == FRNNT_CONSTRAINED && s >= 1) gy += g_px[((size_t)b * S + s - 1) * T1 + t];
    }
    const int y = band_symbol(symbols, ranges, b, (size_t)row, k, S, blank, C);
    const real l = lse[row];
    const real neg = -(gx + gy);
    const vec *src = reinterpret_cast<const vec *>(logits + row * (long long)C);
    vec *dst = reinterpret_cast<vec *>(g_logits + row * (long long)C);
    for (int v = lane; v < nvec; v += 32) {
      const vec x = src[v];
      vec o;
#pragma unroll
      for (int e = 0; e < VW; ++e) {
        const int c = v * VW + e;
        real g = neg * exp_sum(elem<real>(x, e) - l);
        if (c == y) g += gx;
        if (c == blank) g += gy;
        set_elem(o, e, g);
      }
      dst[v] = o;
    }
  }
}

template <typename real>
static int lsm_forward_impl(const void *logits, const int64_t *symbols, const int64_t *ranges,
                            const int64_t *boundary, void *lse, void *pxb, void *pyb, void *px,
                            void *py, int B, int T, int R, int S, int C, int blank, int rnnt_type,
                            double delay_penalty, cudaStream_t st) {
  constexpr int VWMAX = sizeof(real) == 4 ? 4 : 2;
  const long long rows = (long long)B * T * R;
  const bool vec_ok = (C % VWMAX == 0) && ((uintptr_t)logits % 16 == 0);
  const int nvec = vec_ok ? C / VWMAX : C;
  int group = 32;
  while (group < 256 && nvec > group * kRowCache) group *= 2;
  const bool small_cache = nvec <= group * 4;
  const int gpc = kRowCta / group;
  long long want = (rows + gpc - 1) / gpc;
  const int grid = (int)(want < (long long)sm_count() * 64 ? (want > 0 ? want : 1) : (long long)sm_count() * 64);
#define LSM_FWD1(VW, G, CA)                                                                    \
  FRNNT_KERNEL(lsm_rows_forward_kernel<real, VW, G, CA><<<grid, kRowCta, 0, st>>>(                            \
      (const real *)logits, symbols, ranges, (real *)lse, (real *)pxb, (real *)pyb, rows, T, R, \
      S, C, blank))
#define LSM_FWD(VW, G)                  \
  do {                                  \
    if (small_cache) {                  \
      LSM_FWD1(VW, G, 4);               \
    } else {                            \
      LSM_FWD1(VW, G, kRowCache);       \
    }                                   \
  } while (0)
  if (rows > 0) {
    if (vec_ok) {
      if (group == 32) LSM_FWD(VWMAX, 32);
      else if (group == 64) LSM_FWD(VWMAX, 64);
      else if (group == 128) LSM_FWD(VWMAX, 128);
      else LSM_FWD(VWMAX, 256);
    } else {
      if (group == 32) LSM_FWD(1, 32);
      else if (group == 64) LSM_FWD(1, 64);
      else if (group == 128) LSM_FWD(1, 128);
      else LSM_FWD(1, 256);
    }
    FRNNT_CUDA(cudaGetLastError());
  }
#undef LSM_FWD
#undef LSM_FWD1
  if (px != nullptr && py != nullptr && B > 0) {
    dim3 grid2((unsigned)((T + 1 + 127) / 128), (unsigned)(S + 1), (unsigned)B);
    FRNNT_KERNEL(band_to_lattice_kernel<real><<<grid2, 128, 0, st>>>((const real *)pxb, (const real *)pyb,
                                                       ranges, boundary, (real *)px, (real *)py,
                                                       S, T, R, rnnt_type, delay_penalty));
    FRNNT_CUDA(cudaGetLastError());
  }
  return FRNNT_OK;
}

template <typename real>
static int lsm_backward_impl(const void *logits, const int64_t *symbols, const int64_t *ranges,
                             const int64_t *boundary, const void *lse, const void *g_px,
                             const void *g_py, void *g_logits, int B, int T, int R, int S, int C,
                             int blank, int rnnt_type, cudaStream_t st) {
  constexpr int VWMAX = sizeof(real) == 4 ? 4 : 2;
  const long long rows = (long long)B * T * R;
  if (rows == 0) return FRNNT_OK;
  const bool vec_ok = (C % VWMAX == 0) && ((uintptr_t)logits % 16 == 0) &&
                      ((uintptr_t)g_logits % 16 == 0);
  long long want = (rows + 7) / 8;
  const int grid = (int)(want < (long long)sm_count() * 64 ? want : (long long)sm_count() * 64);
  if (vec_ok)
    FRNNT_KERNEL(lsm_rows_backward_kernel<real, VWMAX><<<grid, kRowCta, 0, st>>>(
        (const real *)logits, symbols, ranges, boundary, (const real *)lse, (const real *)g_px,
        (const real *)g_py, (real *)g_logits, rows, T, R, S, C, blank, rnnt_type));
  else
    FRNNT_KERNEL(lsm_rows_backward_kernel<real, 1><<<grid, kRowCta, 0, st>>>(
        (const real *)logits, symbols, ranges, boundary, (const real *)lse, (const real *)g_px,
        (const real *)g_py, (real *)g_logits, rows, T, R, S, C, blank, rnnt_type));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

static int lsm_check(int dtype, int B, int T, int R, int S, int C, int blank, int rnnt_type) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(B >= 0 && T >= 0 && R >= 1 && S >= 0 && C >= 1, FRNNT_EINVAL,
                "bad sizes B=%d T=%d R=%d S=%d C=%d", B, T, R, S, C);
  FRNNT_REQUIRE(R <= S + 1, FRNNT_EINVAL, "band width R=%d exceeds S+1=%d", R, S + 1);
  FRNNT_REQUIRE(blank >= 0 && blank < C, FRNNT_EINVAL, "blank=%d outside [0,%d)", blank, C);
  FRNNT_REQUIRE(rnnt_type >= 0 && rnnt_type <= 2, FRNNT_EINVAL, "bad rnnt_type %d", rnnt_type);
  FRNNT_REQUIRE(S + 1 <= 65535 && B <= 65535, FRNNT_EUNSUPPORTED, "S or B too large for the grid");
  return FRNNT_OK;
}

}  // namespace frnnt

using namespace frnnt;

extern "C" int frnnt_lsm_gather_forward(int dtype, const void *logits, const int64_t *symbols,
                                        const int64_t *ranges, const int64_t *boundary,
                                        void *lse, void *px_band, void *py_band, void *px,
                                        void *py, int B, int T, int R, int S, int C, int blank,
                                        int rnnt_type, double delay_penalty, void *stream) {
  int rc = lsm_check(dtype, B, T, R, S, C, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0 || T == 0) return FRNNT_OK;
  FRNNT_REQUIRE(logits && lse && px_band && py_band && (symbols || S == 0), FRNNT_EINVAL,
                "NULL argument");
  FRNNT_REQUIRE(ranges != nullptr || R == S + 1, FRNNT_EINVAL,
                "without ranges the band must cover all S+1 rows");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FRNNT_F32)
    return lsm_forward_impl<float>(logits, symbols, ranges, boundary, lse, px_band, py_band, px,
                                   py, B, T, R, S, C, blank, rnnt_type, delay_penalty, st);
  return lsm_forward_impl<double>(logits, symbols, ranges, boundary, lse, px_band, py_band, px, py,
                                  B, T, R, S, C, blank, rnnt_type, delay_penalty, st);
}

extern "C" int frnnt_lsm_gather_backward(int dtype, const void *logits, const int64_t *symbols,
                                         const int64_t *ranges, const int64_t *boundary,
                                         const void *lse, const void *px_grad,
                                         const void *py_grad, void *logits_grad, int B, int T,
                                         int R, int S, int C, int blank, int rnnt_type,
                                         void *stream) {
  int rc = lsm_check(dtype, B, T, R, S, C, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0 || T == 0) return FRNNT_OK;
  FRNNT_REQUIRE(logits && lse && py_grad && logits_grad && (px_grad || S == 0) &&
                    (symbols || S == 0),
                FRNNT_EINVAL, "NULL argument");
  FRNNT_REQUIRE(ranges != nullptr || R == S + 1, FRNNT_EINVAL,
                "without ranges the band must cover all S+1 rows");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == FRNNT_F32)
    return lsm_backward_impl<float>(logits, symbols, ranges, boundary, lse, px_grad, py_grad,
                                    logits_grad, B, T, R, S, C, blank, rnnt_type, st);
  return lsm_backward_impl<double>(logits, symbols, ranges, boundary, lse, px_grad, py_grad,
                                   logits_grad, B, T, R, S, C, blank, rnnt_type, st);
}
