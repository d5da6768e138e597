// Shared by the log-softmax kernels (lsm.cu) and the fused joiner (joiner_pairs.cu):
// where a band entry (b, t, k) of the pruned / unpruned joiner output sits in the
// lattices, which symbol it scores, and the kernel that places the bands
// [B][T][R] into px [B][S][T1] and py [B][S+1][T]
// (reference: fast_rnnt/python/fast_rnnt/rnnt_loss.py:942-1022 and :418-447).
#pragma once
#include "common.cuh"

namespace frnnt {

// Lattice row of band entry k at frame (b, t).
__device__ __forceinline__ int band_row(const int64_t *ranges, size_t bt, int R, int k, int S1) {
  if (ranges == nullptr) return k;
  long long s = (long long)ranges[bt * R] + k;
  s %= S1;
  if (s < 0) s += S1;
  return (int)s;
}

// Symbol whose log-prob goes to px for band entry (b, t, k).
__device__ __forceinline__ int band_symbol(const int64_t *symbols, const int64_t *ranges, int b,
                                           size_t row, int k, int S, int blank, int C) {
  long long r = ranges ? (long long)ranges[row] : k;
  long long y = (r >= 0 && r < S) ? (long long)symbols[(size_t)b * S + r] : blank;
  if (y < 0 || y >= C) y = blank;  // never index outside the row
  return (int)y;
}

// Delay penalty of the reference's loss functions (rnnt_loss.py:309-324 and its three copies):
// px[b][s][t] += delay_penalty * ((T_b - 1) / 2 - t), with the roundings torch makes there --
// with a boundary tensor the offset (an integer tensor divided by 2) and hence the whole
// penalty are float32 whatever px's type is; without one they have px's type; the product is
// rounded before it is added.  Zero when delay_penalty is not positive.
template <typename real>
__device__ __forceinline__ real delay_penalty_at(const int64_t *boundary, int b, int T, int t, double dp) {
  if (!(dp > 0.0)) return (real)0;
  if (boundary != nullptr) {
    const float off = (float)(boundary[4 * b + 3] - 1) / 2.0f;
    return (real)__fmul_rn(off - (float)t, (float)dp);
  }
  if (sizeof(real) == 4) return (real)__fmul_rn((float)(T - 1) / 2.0f - (float)t, (float)dp);
  return (real)__dmul_rn((double)(T - 1) / 2.0 - (double)t, dp);
}
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }

// bands -> lattices: row (ranges[b][t][0] + k) mod (S+1), -inf elsewhere, the -inf column
// at t = T (regular), the -inf at t = t_end (regular + boundary), px += py[s+1] (constrained),
// the delay penalty on px
template <typename real>
__global__ void band_to_lattice_kernel(const real *__restrict__ pxb, const real *__restrict__ pyb,
                                       const int64_t *__restrict__ ranges,
                                       const int64_t *__restrict__ boundary, real *__restrict__ px,
                                       real *__restrict__ py, int S, int T, int R, int rnnt_type,
                                       double delay_penalty = 0.0) {
  const int b = blockIdx.z, s = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int S1 = S + 1;
  const int T1 = (rnnt_type == FRNNT_REGULAR) ? T + 1 : T;
  if (t > T) return;
  const real ninf = neg_inf<real>();
  real vy = ninf, vx = ninf, vy_next = ninf;
  if (t < T) {
    const size_t bt = (size_t)b * T + t;
    long long shift = ranges ? (long long)ranges[bt * R] : 0;
    shift %= S1;
    if (shift < 0) shift += S1;
    int k = s - (int)shift;
    if (k < 0) k += S1;
    if (k < R) {
      vy = pyb[bt * R + k];
      vx = pxb[bt * R + k];
    }
    if (rnnt_type == FRNNT_CONSTRAINED && s < S) {
      int k1 = s + 1 - (int)shift;
      if (k1 < 0) k1 += S1;
      if (k1 >= S1) k1 -= S1;
      if (k1 < R) vy_next = pyb[bt * R + k1];
    }
    py[((size_t)b * S1 + s) * T + t] = vy;
  }
  if (s < S && t < T1) {
    if (rnnt_type == FRNNT_REGULAR) {
      if (t == T) vx = ninf;
      if (boundary != nullptr && (long long)t == (long long)boundary[4 * b + 3]) vx = ninf;
    } else if (rnnt_type == FRNNT_CONSTRAINED) {
      vx = vx + vy_next;
    }
    if (delay_penalty > 0.0) vx = add_rn(vx, delay_penalty_at<real>(boundary, b, T, t, delay_penalty));
    px[((size_t)b * S + s) * T1 + t] = vx;
  }
}

}  // namespace frnnt
