// "Simple" (factorised joiner) log-prob lattices and their gradient:
// get_rnnt_logprobs and get_rnnt_logprobs_smoothed of the reference
// (fast_rnnt/python/fast_rnnt/rnnt_loss.py:160-227 and :1246-1369), which the
// reference composes from ~20-40 ATen kernels plus autograd.
//
//   N[b,s,t]  = log( sum_c e^{lm[b,s,c]-lmmax[b,s]} e^{am[b,t,c]-ammax[b,t]} + tiny ) + lmmax + ammax
//   px[b,s,t] = am[b,t,y_bs] + lm[b,s,y_bs] - N[b,s,t]      (t < T; -inf at t = T and t = t_end)
//   py[b,s,t] = am[b,t,blank] + lm[b,s,blank] - N[b,s,t]
//   smoothed:  x*(1-l-a) + x_lmonly*l + x_amonly*a with the lm-only softmax
//              normalizer, the batch-wide unigram and the am-only normalizer.
//
// Forward  = row statistics (max, sum exp) -> [unigram, am-only normalizer] ->
//            batched contraction with the exp() applied while the operand tiles
//            are staged and log()+max in the epilogue -> lattice assembly.
// Backward = analytic: with W = -(g_px + g_py)/(M + tiny) the two contractions
//            dlm = L .* (W A), dam = A .* (W^T L) plus the one-hot gather terms
//            and the lm-only / am-only / unigram terms.  The row maxima are
//            treated as constants: N does not depend on them analytically.
//
// This file holds the fp32/fp64 SIMT version of the contraction (FMA pipes,
// shared-memory tiles); it is the general path for both dtypes.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "lsm_band.cuh"
#include "simple_pairs.cuh"

namespace frnnt {

template <typename real> __device__ __forceinline__ real tiny_v();
template <> __device__ __forceinline__ float tiny_v<float>() { return 1.17549435e-38f; }
template <> __device__ __forceinline__ double tiny_v<double>() { return 2.2250738585072014e-308; }

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

// ---- buffers -----------------------------------------------------------------
// "saved": what the forward keeps for the backward.
struct SavedLayout {
  size_t norm, lmmax, lmsum, ammax, amonly, uni, loguni, total;
  SavedLayout(size_t es, int B, int S, int T, int C) {
    size_t o = 0;
    norm = o;   o += align_up(es * (size_t)B * (S + 1) * T);
    lmmax = o;  o += align_up(es * (size_t)B * (S + 1));
    lmsum = o;  o += align_up(es * (size_t)B * (S + 1));
    ammax = o;  o += align_up(es * (size_t)B * T);
    amonly = o; o += align_up(es * (size_t)B * T);
    uni = o;    o += align_up(es * (size_t)C);
    loguni = o; o += align_up(es * (size_t)C);
    total = o;
  }
};

constexpr int kColChunkRows = 32;  // rows folded by one CTA of the column-sum kernels

// row pitch of the gradient-weight matrix (16-byte aligned rows for the tensor-core path)
static inline int rw_pitch(int T) { return (T + 3) & ~3; }

// "scratch": temporaries of one call.
struct ScratchLayout {
  size_t rw, sgx, sgy, cgx, cgy, gl, h, partial, dp, rowdot, total;
  int nchunk;
  ScratchLayout(size_t es, int B, int S, int T, int C) {
    size_t o = 0;
    const size_t rows_max = (size_t)B * (T > S + 1 ? T : S + 1);
    nchunk = (int)((rows_max + kColChunkRows - 1) / kColChunkRows);
    rw = o;      o += align_up(es * (size_t)B * (S + 1) * rw_pitch(T));  // gradient weights, rows padded to 4
    sgx = o;     o += align_up(es * (size_t)B * (S + 1));      // sum_t gx, sum_t gy
    sgy = o;     o += align_up(es * (size_t)B * (S + 1));
    cgx = o;     o += align_up(es * (size_t)B * T);            // sum_s gx, sum_s gy
    cgy = o;     o += align_up(es * (size_t)B * T);
    gl = o;      o += align_up(es * (size_t)B * (S + 1));      // weight of the lm-only softmax
    h = o;       o += align_up(es * (size_t)B * T);            // weight of the am-only normalizer
    partial = o; o += align_up(es * (size_t)nchunk * C);       // column-sum partials
    dp = o;      o += align_up(es * (size_t)C);                // d loss / d unigram-softmax mean
    rowdot = o;  o += align_up(es * (size_t)B * (S + 1));
    total = o;
  }
};

// ---- row statistics ------------------------------------------------------------
// one warp per row: max and sum(exp(x - max))
template <typename real>
__global__ void row_stats_kernel(const real *__restrict__ x, real *__restrict__ rmax,
                                 real *__restrict__ rsum, long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const real *src = x + row * (long long)C;
    real m = neg_inf<real>();
    for (int c = lane; c < C; c += 32) m = max(m, src[c]);
    m = warp_max(m);
    real s = 0;
    for (int c = lane; c < C; c += 32) s += exp_r(src[c] - m);
    s = warp_sum(s);
    if (lane == 0) {
      rmax[row] = m;
      rsum[row] = s;
    }
  }
}

// one warp per row: the maximum alone (all that is needed of the am rows), 16-byte loads
// when the rows allow them
template <typename real>
__global__ void row_max_kernel(const real *__restrict__ x, real *__restrict__ rmax, long long rows,
                               int C, int vec_ok) {
  constexpr int VW = 16 / sizeof(real);
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const real *src = x + row * (long long)C;
    real m = neg_inf<real>();
    if (vec_ok) {
      const float4 *v4 = reinterpret_cast<const float4 *>(src);
      for (int c = lane; c < C / VW; c += 32) {
        const float4 q = v4[c];
        const real *e = reinterpret_cast<const real *>(&q);
#pragma unroll
        for (int i = 0; i < VW; ++i) m = max(m, e[i]);
      }
    } else {
      for (int c = lane; c < C; c += 32) m = max(m, src[c]);
    }
    m = warp_max(m);
    if (lane == 0) rmax[row] = m;
  }
}

// partial[chunk][c] = sum over the chunk's rows of f(row, c); one thread per column
//   MODE 0: softmax(lm row)[c]                      (unigram)
//   MODE 1: h[row] * e^{am[row,c]-ammax[row]} / Z[row]   (d unigram via the am-only normalizer)
template <typename real, int MODE>
__global__ void column_partial_kernel(const real *__restrict__ x, const real *__restrict__ rmax,
                                      const real *__restrict__ aux, const real *__restrict__ h,
                                      real *__restrict__ partial, long long rows, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long r0 = (long long)blockIdx.y * kColChunkRows;
  const long long r1 = min(rows, r0 + kColChunkRows);
  real acc = 0;
  for (long long r = r0; r < r1; ++r) {
    const real e = exp_r(x[r * C + c] - rmax[r]);
    if (MODE == 0) {
      acc += e / aux[r];  // aux = sum exp
    } else {
      // aux = am-only normalizer (log Z + ammax)  ->  1/Z = e^{ammax - aux}
      acc += h[r] * e * exp_r(rmax[r] - aux[r]);
    }
  }
  partial[(size_t)blockIdx.y * C + c] = acc;
}

template <typename real>
__global__ void unigram_final_kernel(const real *__restrict__ partial, int nchunk, long long rows,
                                     int C, real *__restrict__ uni, real *__restrict__ loguni) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  real acc = 0;
  for (int j = 0; j < nchunk; ++j) acc += partial[(size_t)j * C + c];
  const real u = acc / (real)rows + tiny_v<real>();
  uni[c] = u;
  loguni[c] = log_r(u);
}

// one warp per am row: log(sum_c e^{am-ammax} u[c]) + ammax
template <typename real>
__global__ void am_only_norm_kernel(const real *__restrict__ am, const real *__restrict__ ammax,
                                    const real *__restrict__ uni, real *__restrict__ amonly,
                                    long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const real *src = am + row * (long long)C;
    const real m = ammax[row];
    real z = 0;
    for (int c = lane; c < C; c += 32) z += exp_r(src[c] - m) * uni[c];
    z = warp_sum(z);
    if (lane == 0) amonly[row] = log_r(z) + m;
  }
}

// ---- the contraction (SIMT) ---------------------------------------------------------
// C[m][n] = sum_k X(m,k) * Y(n,k); the problem policy supplies the (transformed)
// operands, says which index is contiguous in memory, and consumes the result.
template <typename real, int BM, int BN, int BK, int TM, int TN, typename Prob>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) contraction_kernel(Prob prob) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int PAD = 4;
  __shared__ real Xs[BK][BM + PAD];
  __shared__ real Ys[BK][BN + PAD];
  prob.set_batch(blockIdx.z);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  real acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0;

  const int K = prob.K();
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll 4
    for (int idx = tid; idx < BM * BK; idx += NT) {
      const int k = Prob::X_K_CONTIG ? idx % BK : idx / BM;
      const int m = Prob::X_K_CONTIG ? idx / BK : idx % BM;
      Xs[k][m] = prob.x(m0 + m, k0 + k);
    }
#pragma unroll 4
    for (int idx = tid; idx < BN * BK; idx += NT) {
      const int k = Prob::Y_K_CONTIG ? idx % BK : idx / BN;
      const int n = Prob::Y_K_CONTIG ? idx / BK : idx % BN;
      Ys[k][n] = prob.y(n0 + n, k0 + k);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      real a[TM], bq[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = Xs[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) bq[j] = Ys[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] += a[i] * bq[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) prob.store(m0 + ty * TM + i, n0 + tx * TN + j, acc[i][j]);
}

// N[s][t] = log(sum_c L[s][c] A[t][c] + tiny) + lmmax[s] + ammax[t]
template <typename real>
struct NormProb {
  static constexpr bool X_K_CONTIG = true, Y_K_CONTIG = true;
  const real *lm, *am, *lmmax, *ammax;
  real *norm;
  int S1, T, C;
  __device__ void set_batch(int b) {
    lm += (size_t)b * S1 * C;
    am += (size_t)b * T * C;
    lmmax += (size_t)b * S1;
    ammax += (size_t)b * T;
    norm += (size_t)b * S1 * T;
  }
  __device__ int K() const { return C; }
  __device__ real x(int s, int c) const {
    return (s < S1 && c < C) ? exp_r(lm[(size_t)s * C + c] - lmmax[s]) : (real)0;
  }
  __device__ real y(int t, int c) const {
    return (t < T && c < C) ? exp_r(am[(size_t)t * C + c] - ammax[t]) : (real)0;
  }
  __device__ void store(int s, int t, real acc) const {
    if (s < S1 && t < T) norm[(size_t)s * T + t] = log_r(acc + tiny_v<real>()) + lmmax[s] + ammax[t];
  }
};

// dlm[s][c] = -L[s][c] * sum_t Rw[s][t] A[t][c]  - gl[s] P[s][c] + P[s][c] (dP[c] - rowdot[s])
template <typename real>
struct LmGradProb {
  static constexpr bool X_K_CONTIG = true, Y_K_CONTIG = false;
  const real *rw, *am, *ammax, *lm, *lmmax, *lmsum, *gl, *dp, *rowdot;
  real *lm_grad;
  int S1, T, C, Tp;
  __device__ void set_batch(int b) {
    rw += (size_t)b * S1 * Tp;
    am += (size_t)b * T * C;
    ammax += (size_t)b * T;
    lm += (size_t)b * S1 * C;
    lmmax += (size_t)b * S1;
    lmsum += (size_t)b * S1;
    if (gl) gl += (size_t)b * S1;
    if (rowdot) rowdot += (size_t)b * S1;
    lm_grad += (size_t)b * S1 * C;
  }
  __device__ int K() const { return T; }
  __device__ real x(int s, int t) const { return (s < S1 && t < T) ? rw[(size_t)s * Tp + t] : (real)0; }
  __device__ real y(int c, int t) const {
    return (c < C && t < T) ? exp_r(am[(size_t)t * C + c] - ammax[t]) : (real)0;
  }
  __device__ void store(int s, int c, real acc) const {
    if (s >= S1 || c >= C) return;
    const real L = exp_r(lm[(size_t)s * C + c] - lmmax[s]);
    real v = -(L * acc);
    if (gl != nullptr) {
      const real P = L / lmsum[s];
      v -= gl[s] * P;
      if (dp != nullptr) v += P * (dp[c] - rowdot[s]);
    }
    lm_grad[(size_t)s * C + c] = v;
  }
};

// dam[t][c] = -A[t][c] * sum_s Rw[s][t] L[s][c]  - h[t] A[t][c] u[c] / Z[t]
template <typename real>
struct AmGradProb {
  static constexpr bool X_K_CONTIG = false, Y_K_CONTIG = false;
  const real *rw, *lm, *lmmax, *am, *ammax, *h, *uni, *amonly;
  real *am_grad;
  int S1, T, C, Tp;
  __device__ void set_batch(int b) {
    rw += (size_t)b * S1 * Tp;
    lm += (size_t)b * S1 * C;
    lmmax += (size_t)b * S1;
    am += (size_t)b * T * C;
    ammax += (size_t)b * T;
    if (h) {
      h += (size_t)b * T;
      amonly += (size_t)b * T;
    }
    am_grad += (size_t)b * T * C;
  }
  __device__ int K() const { return S1; }
  __device__ real x(int t, int s) const { return (t < T && s < S1) ? rw[(size_t)s * Tp + t] : (real)0; }
  __device__ real y(int c, int s) const {
    return (c < C && s < S1) ? exp_r(lm[(size_t)s * C + c] - lmmax[s]) : (real)0;
  }
  __device__ void store(int t, int c, real acc) const {
    if (t >= T || c >= C) return;
    const real A = exp_r(am[(size_t)t * C + c] - ammax[t]);
    real v = -(A * acc);
    if (h != nullptr) v -= h[t] * A * uni[c] * exp_r(ammax[t] - amonly[t]);
    am_grad[(size_t)t * C + c] = v;
  }
};

template <typename real> struct TileCfg;
template <> struct TileCfg<float> { static constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8; };
template <> struct TileCfg<double> { static constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4; };

template <typename real, typename Prob>
static int launch_contraction(const Prob &prob, int M, int N, int B, cudaStream_t st) {
  using Cfg = TileCfg<real>;
  dim3 grid((unsigned)((N + Cfg::BN - 1) / Cfg::BN), (unsigned)((M + Cfg::BM - 1) / Cfg::BM),
            (unsigned)B);
  FRNNT_KERNEL(contraction_kernel<real, Cfg::BM, Cfg::BN, Cfg::BK, Cfg::TM, Cfg::TN, Prob>
               <<<grid, (Cfg::BM / Cfg::TM) * (Cfg::BN / Cfg::TN), 0, st>>>(prob));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

// ---- lattice assembly -------------------------------------------------------------
struct SmoothCfg {
  int smoothed;
  // the am-only branch is left out: am_only_scale == 0.  The reference multiplies the
  // branch by 1e-20 in that case (rnnt_loss.py:1346-1351), which changes an fp32 / fp64
  // px or py only if that value is exactly 0; its three extra passes (unigram, am-only
  // normalizer) are not worth that
  int am_only_off;
  double both, ls, as;  // 1-l-a, lm-only scale, am-only scale (zero lm scale replaced by 1e-20)
  double delay_penalty = 0.0;  // added to px by the lattice-writing kernels when positive
};

template <typename real>
__global__ void assemble_kernel(const real *__restrict__ lm, const real *__restrict__ am,
                                const int64_t *__restrict__ symbols,
                                const int64_t *__restrict__ boundary, const real *__restrict__ norm,
                                const real *__restrict__ lmmax, const real *__restrict__ lmsum,
                                const real *__restrict__ amonly, const real *__restrict__ loguni,
                                real *__restrict__ px, real *__restrict__ py, int S, int T, int C,
                                int blank, int rnnt_type, SmoothCfg cfg) {
  const int b = blockIdx.z, s = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int S1 = S + 1;
  const int T1 = (rnnt_type == FRNNT_REGULAR) ? T + 1 : T;
  if (t > T) return;
  const real ninf = neg_inf<real>();
  const real both = (real)cfg.both, ls = (real)cfg.ls, as = (real)cfg.as;
  const real *lmrow = lm + ((size_t)b * S1 + s) * C;
  real lm_only_norm = 0;
  if (cfg.smoothed) lm_only_norm = log_r(lmsum[(size_t)b * S1 + s]) + lmmax[(size_t)b * S1 + s];

  // py at (s, t) and, for the constrained type, at (s+1, t)
  auto py_at = [&](int ss) -> real {
    const real *amrow = am + ((size_t)b * T + t) * C;
    const real *lr = lm + ((size_t)b * S1 + ss) * C;
    const real py_am = amrow[blank], py_lm = lr[blank];
    real v = py_am + py_lm - norm[((size_t)b * S1 + ss) * T + t];
    if (cfg.smoothed) {
      const real lnorm = log_r(lmsum[(size_t)b * S1 + ss]) + lmmax[(size_t)b * S1 + ss];
      const real v_lm = py_lm - lnorm;
      v = v * both + v_lm * ls;
      if (!cfg.am_only_off) v += (py_am + loguni[blank] - amonly[(size_t)b * T + t]) * as;
    }
    return v;
  };

  if (t < T) py[((size_t)b * S1 + s) * T + t] = py_at(s);

  if (s < S && t < T1) {
    int y = (int)symbols[(size_t)b * S + s];
    if (y < 0 || y >= C) y = blank;
    const real px_lm = lmrow[y];
    real px_am = ninf, v;
    if (t < T) {
      px_am = am[((size_t)b * T + t) * C + y];
      v = px_am + px_lm - norm[((size_t)b * S1 + s) * T + t];
    } else {
      v = px_am + px_lm;  // the -inf column of the regular type
    }
    if (cfg.smoothed) {
      const real v_lm = px_lm - lm_only_norm;
      v = v * both + v_lm * ls;
      if (!cfg.am_only_off) {
        real v_am = px_am + loguni[y];
        if (t < T) v_am -= amonly[(size_t)b * T + t];
        v += v_am * as;
      }
    }
    if (rnnt_type == FRNNT_REGULAR) {
      if (boundary != nullptr && (long long)t == (long long)boundary[4 * b + 3]) v = ninf;
    } else if (rnnt_type == FRNNT_CONSTRAINED) {
      v += py_at(s + 1);
    }
    if (cfg.delay_penalty > 0.0) v = add_rn(v, delay_penalty_at<real>(boundary, b, T, t, cfg.delay_penalty));
    px[((size_t)b * S + s) * T1 + t] = v;
  }
}

// ---- backward helpers -------------------------------------------------------------
// Gradients that actually reach the un-masked lattice entries:
//   gx: px_grad with the t = t_end column of the regular type dropped
//   gy: py_grad, plus px_grad[s-1] for the constrained type (px += py[s+1])
template <typename real>
struct EffGrads {
  const real *g_px, *g_py;
  const int64_t *boundary;
  int S, T, T1, rnnt_type;
  __device__ real gx(int b, int s, int t) const {
    if (s >= S || t >= T1) return 0;
    if (rnnt_type == FRNNT_REGULAR && boundary != nullptr &&
        (long long)t == (long long)boundary[4 * b + 3])
      return 0;
    return g_px[((size_t)b * S + s) * T1 + t];
  }
  __device__ real gy(int b, int s, int t) const {
    if (t >= T) return 0;
    real v = g_py[((size_t)b * (S + 1) + s) * T + t];
    if (rnnt_type == FRNNT_CONSTRAINED && s >= 1) v += g_px[((size_t)b * S + s - 1) * T1 + t];
    return v;
  }
};

// Rw[b,s,t] = both * (gx + gy) / (M + tiny),   1/(M+tiny) = e^{lmmax + ammax - N}
template <typename real>
__global__ void grad_weight_kernel(EffGrads<real> eg, const real *__restrict__ norm,
                                   const real *__restrict__ lmmax, const real *__restrict__ ammax,
                                   real *__restrict__ rw, real both, int Tp) {
  const int b = blockIdx.z, s = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= Tp) return;
  const size_t o = ((size_t)b * (eg.S + 1) + s) * Tp + t;
  if (t >= eg.T) {  // row padding
    rw[o] = 0;
    return;
  }
  const size_t i = ((size_t)b * (eg.S + 1) + s) * eg.T + t;
  const real w = both * (eg.gx(b, s, t) + eg.gy(b, s, t));
  const real inv = exp_r(lmmax[(size_t)b * (eg.S + 1) + s] + ammax[(size_t)b * eg.T + t] - norm[i]);
  rw[o] = (w == 0) ? (real)0 : w * inv;
}

// The two kernels above and below in one pass, for the tensor-core path: one CTA per lattice
// row (b, s) writes the row of Rw, the row sums of gx (all T1 columns) and gy, and the
// row's largest |Rw| (which sets the scale of the fp16 planes Rw is split into).
template <typename real>
__global__ void __launch_bounds__(128)
grad_weight_rows_kernel(EffGrads<real> eg, const real *__restrict__ norm, const real *__restrict__ lmmax,
                        const real *__restrict__ ammax, real *__restrict__ rw, real *__restrict__ sgx,
                        real *__restrict__ sgy, float *__restrict__ rowmax, real both, int Tp) {
  __shared__ real red[3][4];
  const int row = blockIdx.x, b = row / (eg.S + 1), s = row % (eg.S + 1);
  const real lmx = lmmax[row];
  real ax = 0, ay = 0, mx = 0;
  const int n = max(Tp, eg.T1);
  for (int t = threadIdx.x; t < n; t += blockDim.x) {
    const real gx = eg.gx(b, s, t), gy = eg.gy(b, s, t);
    ax += gx;
    ay += gy;
    if (t < Tp) {
      real v = 0;
      if (t < eg.T) {
        const real w = both * (gx + gy);
        const real inv = exp_r(lmx + ammax[(size_t)b * eg.T + t] - norm[(size_t)row * eg.T + t]);
        v = (w == 0) ? (real)0 : w * inv;
      }
      rw[(size_t)row * Tp + t] = v;
      mx = max(mx, v < 0 ? -v : v);
    }
  }
  ax = warp_sum(ax);
  ay = warp_sum(ay);
  mx = warp_max(mx);
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) red[0][w] = ax, red[1][w] = ay, red[2][w] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    sgx[row] = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
    sgy[row] = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
    rowmax[row] = (float)max(max(red[2][0], red[2][1]), max(red[2][2], red[2][3]));
  }
}

// one warp per (b, s): sums over t of gx (all T1 columns) and gy
template <typename real>
__global__ void grad_row_sums_kernel(EffGrads<real> eg, real *__restrict__ sgx,
                                     real *__restrict__ sgy, int B) {
  const int lane = threadIdx.x & 31;
  const int row = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (row >= B * (eg.S + 1)) return;
  const int b = row / (eg.S + 1), s = row % (eg.S + 1);
  real ax = 0, ay = 0;
  for (int t = lane; t < eg.T1; t += 32) {
    ax += eg.gx(b, s, t);
    ay += eg.gy(b, s, t);
  }
  ax = warp_sum(ax);
  ay = warp_sum(ay);
  if (lane == 0) {
    sgx[row] = ax;
    sgy[row] = ay;
  }
}

// sums over s for 32 frames per CTA: lane <-> frame, the 8 warps take every 8th row
// each (contiguous 128-byte loads, all of a warp's rows independent), then the eight
// partial sums are added in warp order
constexpr int kColSumWarps = 8;
template <typename real>
__global__ void __launch_bounds__(32 * kColSumWarps)
grad_col_sums_kernel(EffGrads<real> eg, real *__restrict__ cgx, real *__restrict__ cgy, int B) {
  __shared__ real px_part[kColSumWarps][32], py_part[kColSumWarps][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int b = blockIdx.y, t = blockIdx.x * 32 + lane;
  real ax = 0, ay = 0;
  if (t < eg.T) {
#pragma unroll 4
    for (int s = w; s <= eg.S; s += kColSumWarps) {
      ax += eg.gx(b, s, t);
      ay += eg.gy(b, s, t);
    }
  }
  px_part[w][lane] = ax;
  py_part[w][lane] = ay;
  __syncthreads();
  if (w == 0 && t < eg.T) {
    ax = px_part[0][lane];
    ay = py_part[0][lane];
    for (int q = 1; q < kColSumWarps; ++q) {
      ax += px_part[q][lane];
      ay += py_part[q][lane];
    }
    cgx[(size_t)b * eg.T + t] = ax;
    cgy[(size_t)b * eg.T + t] = ay;
  }
}

// v[i] = alpha * (a[i] + b[i])
template <typename real>
__global__ void scaled_sum_kernel(const real *a, const real *b, real *v, real alpha, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) v[i] = alpha * (a[i] + b[i]);
}

// one-hot terms of lm_grad: symbol column gets cx*sgx, blank column gets cx*sgy
template <typename real>
__global__ void lm_onehot_kernel(const int64_t *__restrict__ symbols, const real *__restrict__ sgx,
                                 const real *__restrict__ sgy, real *__restrict__ lm_grad, int B,
                                 int S, int C, int blank, real coef) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= B * (S + 1)) return;
  const int b = row / (S + 1), s = row % (S + 1);
  real *g = lm_grad + (size_t)row * C;
  if (s < S) {
    int y = (int)symbols[(size_t)b * S + s];
    if (y < 0 || y >= C) y = blank;
    g[y] += coef * sgx[row];
  }
  g[blank] += coef * sgy[row];
}

// one-hot terms of am_grad: for every s the symbol column gets coef*gx[s][t]; blank gets coef*cgy[t]
template <typename real>
__global__ void am_onehot_kernel(EffGrads<real> eg, const int64_t *__restrict__ symbols,
                                 const real *__restrict__ cgy, real *__restrict__ am_grad, int B,
                                 int C, int blank, real coef) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * eg.T) return;
  const int b = idx / eg.T, t = idx % eg.T;
  real *g = am_grad + (size_t)idx * C;
  // fire-and-forget adds: this thread owns row (b, t), and adds issued by one
  // thread to one address are applied in program order, so the sum is deterministic.
  // Eight gradient loads are issued before their adds (the adds would otherwise keep
  // the next load from starting).
  for (int s0 = 0; s0 < eg.S; s0 += 8) {
    real v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = s0 + u < eg.S ? eg.gx(b, s0 + u, t) : (real)0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (s0 + u >= eg.S || v[u] == 0) continue;
      int y = (int)symbols[(size_t)b * eg.S + s0 + u];
      if (y < 0 || y >= C) y = blank;
      atomicAdd(&g[y], coef * v[u]);
    }
  }
  atomicAdd(&g[blank], coef * cgy[idx]);
}

// d loss / d log-unigram[c] = as * ( sum_{b,s: y_bs = c} sgx[b,s]  +  [c = blank] sum_{b,s} sgy[b,s] )
// then dP[c] = (dlogu[c] / u[c] - du[c]) / rows      (du holds +sum h A / Z)
template <typename real>
__global__ void unigram_grad_kernel(const int64_t *__restrict__ symbols,
                                    const real *__restrict__ sgx, const real *__restrict__ sgy,
                                    const real *__restrict__ du_partial, int nchunk,
                                    const real *__restrict__ uni, real *__restrict__ dp, int B,
                                    int S, int C, int blank, real as) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  real acc = 0;
  for (int b = 0; b < B; ++b)
    for (int s = 0; s <= S; ++s) {
      const int row = b * (S + 1) + s;
      if (s < S) {
        int y = (int)symbols[(size_t)b * S + s];
        if (y < 0 || y >= C) y = blank;
        if (y == c) acc += sgx[row];
      }
      if (c == blank) acc += sgy[row];
    }
  real du = 0;
  for (int j = 0; j < nchunk; ++j) du += du_partial[(size_t)j * C + c];
  dp[c] = (as * acc / uni[c] - du) / (real)((long long)B * (S + 1));
}

// one warp per lm row: rowdot = sum_c softmax(lm row)[c] * dP[c]
template <typename real>
__global__ void row_dot_kernel(const real *__restrict__ lm, const real *__restrict__ lmmax,
                               const real *__restrict__ lmsum, const real *__restrict__ dp,
                               real *__restrict__ rowdot, long long rows, int C) {
  const int lane = threadIdx.x & 31;
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const real *src = lm + row * (long long)C;
  const real m = lmmax[row];
  real acc = 0;
  for (int c = lane; c < C; c += 32) acc += exp_r(src[c] - m) * dp[c];
  acc = warp_sum(acc);
  if (lane == 0) rowdot[row] = acc / lmsum[row];
}

// tensor-core (tcgen05, 3xTF32) contraction: float32 with 16-byte aligned rows;
// everything else (float64, odd vocabulary sizes) takes the SIMT path.  The
// environment variable FRNNT_CONTRACTION=simt forces the SIMT path (for tests).
bool norm_umma_supported(const void *lm, const void *am, int S1, int T, int C);
int launch_norm_umma(const float *lm, const float *am, const float *lmmax, const float *ammax,
                     float *norm, int B, int S1, int T, int C, cudaStream_t st);
int launch_simple_grads_umma(const float *lm, const float *am, const float *lmmax,
                             const float *lmsum, const float *ammax, const float *amonly,
                             const float *uni, const float *rw, const float *gl, const float *h,
                             const float *dp, const float *rowdot, float *lm_grad, float *am_grad,
                             int B, int S1, int T, int C, int Tp, cudaStream_t st);

template <typename real>
static bool use_tensor_cores(const void *lm, const void *am, int S1, int T, int C) {
  if (sizeof(real) != 4) return false;
  const char *mode = getenv("FRNNT_CONTRACTION");
  if (mode != nullptr && strcmp(mode, "simt") == 0) return false;
  return norm_umma_supported(lm, am, S1, T, C);
}

// the fp16-pair engine (FRNNT_CONTRACTION=tf32 keeps the 3xTF32 kernels, =simt the FMA pipe)
template <typename real>
static bool use_pairs(const void *lm, const void *am, int S1, int T, int C, int rnnt_type) {
  if (sizeof(real) != 4) return false;
  const char *mode = getenv("FRNNT_CONTRACTION");
  if (mode != nullptr && (strcmp(mode, "simt") == 0 || strcmp(mode, "tf32") == 0)) return false;
  return simple_pairs_supported(lm, am, S1, T, C, rnnt_type);
}

static int simple_check(int dtype, int B, int S, int T, int C, int blank, int rnnt_type) {
  FRNNT_REQUIRE(check_dtype(dtype) || is_half_input(dtype), FRNNT_EINVAL,
                "dtype must be FRNNT_F32, FRNNT_F64, or FRNNT_F16 / FRNNT_BF16 for 16-bit lm and am");
  FRNNT_REQUIRE(B >= 0 && S >= 0 && T >= 0 && C >= 1, FRNNT_EINVAL,
                "bad sizes B=%d S=%d T=%d C=%d", B, S, T, C);
  FRNNT_REQUIRE(blank >= 0 && blank < C, FRNNT_EINVAL, "blank=%d outside [0,%d)", blank, C);
  FRNNT_REQUIRE(rnnt_type >= 0 && rnnt_type <= 2, FRNNT_EINVAL, "bad rnnt_type %d", rnnt_type);
  FRNNT_REQUIRE(B <= 65535 && S + 1 <= 65535, FRNNT_EUNSUPPORTED, "B or S too large for the grid");
  return FRNNT_OK;
}

static SmoothCfg make_cfg(int smoothed, double lm_only_scale, double am_only_scale) {
  SmoothCfg cfg;
  cfg.smoothed = smoothed;
  cfg.both = 1.0 - lm_only_scale - am_only_scale;
  // exact zeros would turn -inf * 0 into nan (rnnt_loss.py:1346-1351)
  cfg.ls = lm_only_scale == 0.0 ? 1.0e-20 : lm_only_scale;
  cfg.am_only_off = smoothed && am_only_scale == 0.0;
  cfg.as = am_only_scale;
  if (!smoothed) {
    cfg.both = 1.0;
    cfg.ls = 0.0;
    cfg.as = 0.0;
  }
  return cfg;
}

static inline int warps_grid(long long rows) {
  long long want = (rows + 7) / 8;
  if (want < 1) want = 1;
  return (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
}

template <typename real>
static int simple_forward_impl(const void *lm_, const void *am_, const int64_t *symbols,
                               const int64_t *boundary, int blank, int rnnt_type, SmoothCfg cfg,
                               void *px, void *py, void *saved, void *scratch, int B, int S, int T,
                               int C, cudaStream_t st, int input_dtype = FRNNT_F32) {
  const real *lm = (const real *)lm_, *am = (const real *)am_;  // not dereferenced for 16-bit inputs
  const int S1 = S + 1;
  SavedLayout sv(sizeof(real), B, S, T, C);
  ScratchLayout sc(sizeof(real), B, S, T, C);
  char *svb = (char *)saved, *scb = (char *)scratch;
  real *norm = (real *)(svb + sv.norm), *lmmax = (real *)(svb + sv.lmmax);
  real *lmsum = (real *)(svb + sv.lmsum), *ammax = (real *)(svb + sv.ammax);
  real *amonly = (real *)(svb + sv.amonly), *uni = (real *)(svb + sv.uni);
  real *loguni = (real *)(svb + sv.loguni), *partial = (real *)(scb + sc.partial);
  const long long lm_rows = (long long)B * S1, am_rows = (long long)B * T;

  const bool pairs = use_pairs<real>(lm, am, S1, T, C, rnnt_type);
  FRNNT_REQUIRE(!is_half_input(input_dtype) || (pairs && (!cfg.smoothed || cfg.am_only_off)), FRNNT_EUNSUPPORTED,
                "16-bit inputs are read by the tensor-core path without the am-only branch only "
                "(frnnt_simple_reads_16bit_inputs)");
  void *pairs_saved = svb + sv.total;
  if (pairs) {
    int rc0 = launch_simple_forward_pairs(lm_, am_, symbols, boundary, blank,
                                          rnnt_type, cfg.smoothed, cfg.am_only_off, (float)cfg.both,
                                          (float)cfg.ls, (float)cfg.as, (float *)px, (float *)py, (float *)norm,
                                          (float *)lmmax, (float *)lmsum, (float *)ammax, (const float *)amonly,
                                          (const float *)loguni, pairs_saved, B, S, T, C, 0, st, cfg.delay_penalty,
                                          input_dtype);
    if (rc0 != FRNNT_OK) return rc0;
  } else {
    FRNNT_KERNEL(row_stats_kernel<real><<<warps_grid(lm_rows), 256, 0, st>>>(lm, lmmax, lmsum, lm_rows, C));
    constexpr int VW = 16 / sizeof(real);
    const int vec_ok = C % VW == 0 && (uintptr_t)am % 16 == 0;
    FRNNT_KERNEL(row_max_kernel<real><<<warps_grid(am_rows), 256, 0, st>>>(am, ammax, am_rows, C, vec_ok));
  }
  FRNNT_CUDA(cudaGetLastError());
  if (cfg.smoothed && !cfg.am_only_off) {
    const int nchunk = (int)((lm_rows + kColChunkRows - 1) / kColChunkRows);
    dim3 g1((unsigned)((C + 127) / 128), (unsigned)nchunk);
    FRNNT_KERNEL(column_partial_kernel<real, 0><<<g1, 128, 0, st>>>(lm, lmmax, lmsum, nullptr, partial, lm_rows, C));
    FRNNT_KERNEL(unigram_final_kernel<real><<<(C + 127) / 128, 128, 0, st>>>(partial, nchunk, lm_rows, C, uni, loguni));
    FRNNT_KERNEL(am_only_norm_kernel<real><<<warps_grid(am_rows), 256, 0, st>>>(am, ammax, uni, amonly, am_rows, C));
    FRNNT_CUDA(cudaGetLastError());
  }
  int rc;
  if (pairs)
    return launch_simple_forward_pairs(lm_, am_, symbols, boundary, blank,
                                       rnnt_type, cfg.smoothed, cfg.am_only_off, (float)cfg.both,
                                       (float)cfg.ls, (float)cfg.as, (float *)px, (float *)py, (float *)norm,
                                       (float *)lmmax, (float *)lmsum, (float *)ammax, (const float *)amonly,
                                       (const float *)loguni, pairs_saved, B, S, T, C, 1, st, cfg.delay_penalty);
  if (use_tensor_cores<real>(lm, am, S1, T, C)) {
    rc = launch_norm_umma((const float *)lm, (const float *)am, (const float *)lmmax,
                          (const float *)ammax, (float *)norm, B, S1, T, C, st);
  } else {
    NormProb<real> prob{lm, am, lmmax, ammax, norm, S1, T, C};
    rc = launch_contraction<real>(prob, S1, T, B, st);
  }
  if (rc != FRNNT_OK) return rc;
  dim3 g2((unsigned)((T + 1 + 127) / 128), (unsigned)S1, (unsigned)B);
  FRNNT_KERNEL(assemble_kernel<real><<<g2, 128, 0, st>>>(lm, am, symbols, boundary, norm, lmmax, lmsum, amonly,
                                            loguni, (real *)px, (real *)py, S, T, C, blank,
                                            rnnt_type, cfg));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

template <typename real>
static int simple_backward_impl(const void *lm_, const void *am_, const int64_t *symbols,
                                const int64_t *boundary, int blank, int rnnt_type, SmoothCfg cfg,
                                int am_only_active, const void *px_grad, const void *py_grad,
                                const void *saved, void *scratch, void *lm_grad_, void *am_grad_,
                                int B, int S, int T, int C, cudaStream_t st) {
  const real *lm = (const real *)lm_, *am = (const real *)am_;
  real *lm_grad = (real *)lm_grad_, *am_grad = (real *)am_grad_;
  const int S1 = S + 1;
  const int T1 = rnnt_type == FRNNT_REGULAR ? T + 1 : T;
  SavedLayout sv(sizeof(real), B, S, T, C);
  ScratchLayout sc(sizeof(real), B, S, T, C);
  const char *svb = (const char *)saved;
  char *scb = (char *)scratch;
  const real *norm = (const real *)(svb + sv.norm), *lmmax = (const real *)(svb + sv.lmmax);
  const real *lmsum = (const real *)(svb + sv.lmsum), *ammax = (const real *)(svb + sv.ammax);
  const real *amonly = (const real *)(svb + sv.amonly), *uni = (const real *)(svb + sv.uni);
  real *rw = (real *)(scb + sc.rw), *sgx = (real *)(scb + sc.sgx), *sgy = (real *)(scb + sc.sgy);
  real *cgx = (real *)(scb + sc.cgx), *cgy = (real *)(scb + sc.cgy);
  real *gl = (real *)(scb + sc.gl), *h = (real *)(scb + sc.h);
  real *partial = (real *)(scb + sc.partial), *dp = (real *)(scb + sc.dp);
  real *rowdot = (real *)(scb + sc.rowdot);
  const long long lm_rows = (long long)B * S1, am_rows = (long long)B * T;
  EffGrads<real> eg{(const real *)px_grad, (const real *)py_grad, boundary, S, T, T1, rnnt_type};

  const int Tp = rw_pitch(T);
  const bool pairs = use_pairs<real>(lm, am, S1, T, C, rnnt_type) && T > 0;
  dim3 g3((unsigned)((Tp + 127) / 128), (unsigned)S1, (unsigned)B);
  if (pairs) {
    // one pass: Rw, the row sums and the row maxima of |Rw| (first floats of the pairs scratch)
    FRNNT_KERNEL(grad_weight_rows_kernel<real><<<(unsigned)lm_rows, 128, 0, st>>>(
        eg, norm, lmmax, ammax, rw, sgx, sgy, (float *)(scb + sc.total + simple_pairs_rowmax_offset(B, S, T, C)),
        (real)cfg.both, Tp));
  } else {
    if (T > 0)
      FRNNT_KERNEL(grad_weight_kernel<real><<<g3, 128, 0, st>>>(eg, norm, lmmax, ammax, rw, (real)cfg.both, Tp));
    FRNNT_KERNEL(grad_row_sums_kernel<real><<<(int)((lm_rows * 32 + 255) / 256), 256, 0, st>>>(eg, sgx, sgy, B));
  }
  if (T > 0)
    FRNNT_KERNEL(grad_col_sums_kernel<real><<<dim3((unsigned)((T + 31) / 32), (unsigned)B), 32 * kColSumWarps, 0,
                                              st>>>(eg, cgx, cgy, B));
  FRNNT_CUDA(cudaGetLastError());

  const real *gl_p = nullptr, *h_p = nullptr, *dp_p = nullptr, *rowdot_p = nullptr;
  if (cfg.smoothed) {
    // gl[b,s] = ls * (sgx + sgy);  h[b,t] = as * (cgx + cgy)
    FRNNT_KERNEL(scaled_sum_kernel<real><<<(int)((lm_rows + 255) / 256), 256, 0, st>>>(sgx, sgy, gl, (real)cfg.ls,
                                                                      lm_rows));
    gl_p = gl;
    if (am_only_active && T > 0) {
      FRNNT_KERNEL(scaled_sum_kernel<real><<<(int)((am_rows + 255) / 256), 256, 0, st>>>(cgx, cgy, h, (real)cfg.as,
                                                                        am_rows));
      h_p = h;
      const int nchunk = (int)((am_rows + kColChunkRows - 1) / kColChunkRows);
      dim3 g1((unsigned)((C + 127) / 128), (unsigned)nchunk);
      FRNNT_KERNEL(column_partial_kernel<real, 1><<<g1, 128, 0, st>>>(am, ammax, amonly, h, partial, am_rows, C));
      FRNNT_KERNEL(unigram_grad_kernel<real><<<(C + 127) / 128, 128, 0, st>>>(symbols, sgx, sgy, partial, nchunk,
                                                            uni, dp, B, S, C, blank, (real)cfg.as));
      FRNNT_KERNEL(row_dot_kernel<real><<<(int)((lm_rows * 32 + 255) / 256), 256, 0, st>>>(lm, lmmax, lmsum, dp,
                                                                         rowdot, lm_rows, C));
      dp_p = dp;
      rowdot_p = rowdot;
    }
    FRNNT_CUDA(cudaGetLastError());
  }

  int rc;
  if (pairs) {
    rc = launch_simple_grads_pairs((const float *)rw, (const float *)lmsum, (const float *)ammax,
                                   (const float *)amonly, (const float *)uni, (const float *)gl_p,
                                   (const float *)h_p, (const float *)dp_p, (const float *)rowdot_p,
                                   (float *)lm_grad, (float *)am_grad, svb + sv.total, scb + sc.total, B, S, T,
                                   C, Tp, st);
    if (rc != FRNNT_OK) return rc;
  } else if (use_tensor_cores<real>(lm, am, S1, T, C)) {
    rc = launch_simple_grads_umma((const float *)lm, (const float *)am, (const float *)lmmax,
                                  (const float *)lmsum, (const float *)ammax, (const float *)amonly,
                                  (const float *)uni, (const float *)rw, (const float *)gl_p,
                                  (const float *)h_p, (const float *)dp_p, (const float *)rowdot_p,
                                  (float *)lm_grad, (float *)am_grad, B, S1, T, C, Tp, st);
    if (rc != FRNNT_OK) return rc;
  } else {
    LmGradProb<real> p1{rw, am, ammax, lm, lmmax, lmsum, gl_p, dp_p, rowdot_p, lm_grad, S1, T, C, Tp};
    rc = launch_contraction<real>(p1, S1, C, B, st);
    if (rc != FRNNT_OK) return rc;
    AmGradProb<real> p2{rw, lm, lmmax, am, ammax, h_p, uni, amonly, am_grad, S1, T, C, Tp};
    rc = launch_contraction<real>(p2, T, C, B, st);
    if (rc != FRNNT_OK) return rc;
  }

  const real coef_lm = (real)cfg.both + (real)cfg.ls;
  const real coef_am = (real)cfg.both + (am_only_active || !cfg.smoothed ? (real)cfg.as : (real)0);
  FRNNT_KERNEL(lm_onehot_kernel<real><<<(int)((lm_rows + 127) / 128), 128, 0, st>>>(symbols, sgx, sgy, lm_grad, B, S, C,
                                                                   blank, coef_lm));
  FRNNT_KERNEL(am_onehot_kernel<real><<<(int)((am_rows + 127) / 128), 128, 0, st>>>(eg, symbols, cgy, am_grad, B, C,
                                                                   blank, coef_am));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

}  // namespace frnnt

using namespace frnnt;

// float32 calls may take the tensor-core path, whose planes and tables follow the regular areas
extern "C" size_t frnnt_simple_saved_bytes(int dtype, int B, int S, int T, int C) {
  if (is_half_input(dtype)) dtype = FRNNT_F32;
  if (!check_dtype(dtype) || B < 0 || S < 0 || T < 0 || C < 0) return 0;
  return SavedLayout(dtype_size(dtype), B, S, T, C).total +
         (dtype == FRNNT_F32 ? SimplePairsLayout(B, S, T, C).saved_bytes : 0);
}

extern "C" size_t frnnt_simple_scratch_bytes(int dtype, int B, int S, int T, int C) {
  if (is_half_input(dtype)) dtype = FRNNT_F32;
  if (!check_dtype(dtype) || B < 0 || S < 0 || T < 0 || C < 0) return 0;
  return ScratchLayout(dtype_size(dtype), B, S, T, C).total +
         (dtype == FRNNT_F32 ? SimplePairsLayout(B, S, T, C).scratch_bytes : 0);
}

extern "C" int frnnt_simple_reads_16bit_inputs(int S, int T, int C, int rnnt_type, int smoothed,
                                               double am_only_scale) {
  if (S < 0 || T < 1 || C < 1) return 0;
  if (smoothed && am_only_scale != 0.0) return 0;
  // 256-byte aligned rows stand in for the caller's tensors (torch's allocations are)
  return use_pairs<float>((const void *)256, (const void *)256, S + 1, T, C, rnnt_type) ? 1 : 0;
}

extern "C" int frnnt_simple_logprobs_forward(int dtype, const void *lm, const void *am,
                                             const int64_t *symbols, const int64_t *boundary,
                                             int blank, int rnnt_type, int smoothed,
                                             double lm_only_scale, double am_only_scale,
                                             double delay_penalty, void *px, void *py, void *saved,
                                             void *scratch, int B, int S, int T, int C, void *stream) {
  int rc = simple_check(dtype, B, S, T, C, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(lm && (am || T == 0) && (symbols || S == 0) && py && (px || S == 0) && saved &&
                    scratch,
                FRNNT_EINVAL, "NULL argument");
  SmoothCfg cfg = make_cfg(smoothed, lm_only_scale, am_only_scale);
  cfg.delay_penalty = delay_penalty > 0.0 ? delay_penalty : 0.0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype != FRNNT_F64)
    return simple_forward_impl<float>(lm, am, symbols, boundary, blank, rnnt_type, cfg, px, py,
                                      saved, scratch, B, S, T, C, st, dtype);
  return simple_forward_impl<double>(lm, am, symbols, boundary, blank, rnnt_type, cfg, px, py,
                                     saved, scratch, B, S, T, C, st);
}

extern "C" int frnnt_simple_logprobs_backward(int dtype, const void *lm, const void *am,
                                              const int64_t *symbols, const int64_t *boundary,
                                              int blank, int rnnt_type, int smoothed,
                                              double lm_only_scale, double am_only_scale,
                                              const void *px_grad, const void *py_grad,
                                              const void *saved, void *scratch, void *lm_grad,
                                              void *am_grad, int B, int S, int T, int C,
                                              void *stream) {
  int rc = simple_check(dtype, B, S, T, C, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(lm && (am || T == 0) && (symbols || S == 0) && py_grad && (px_grad || S == 0) &&
                    saved && scratch && lm_grad && (am_grad || T == 0),
                FRNNT_EINVAL, "NULL argument");
  SmoothCfg cfg = make_cfg(smoothed, lm_only_scale, am_only_scale);
  // With am_only_scale == 0 the reference still scales the am-only branch by 1e-20; its
  // gradient (<= 1e-19 relative) is below the resolution of either dtype and is skipped.
  const int am_only_active = smoothed && am_only_scale != 0.0;
  cudaStream_t st = (cudaStream_t)stream;
  if (is_half_input(dtype)) {
    // lm and am are not read on this path (the forward kept what the backward needs)
    FRNNT_REQUIRE(use_pairs<float>(lm, am, S + 1, T, C, rnnt_type) && T > 0 && !am_only_active,
                  FRNNT_EUNSUPPORTED, "16-bit inputs: see frnnt_simple_reads_16bit_inputs");
  }
  if (dtype != FRNNT_F64)
    return simple_backward_impl<float>(lm, am, symbols, boundary, blank, rnnt_type, cfg,
                                       am_only_active, px_grad, py_grad, saved, scratch, lm_grad,
                                       am_grad, B, S, T, C, st);
  return simple_backward_impl<double>(lm, am, symbols, boundary, blank, rnnt_type, cfg,
                                      am_only_active, px_grad, py_grad, saved, scratch, lm_grad,
                                      am_grad, B, S, T, C, st);
}
