// Tensor-core (tcgen05 / tensor-memory) version of the normalizer contraction of
// the "simple" RNN-T lattices, float32 with 3xTF32 splitting:
//
//   N[b][s][t] = log( sum_c e^{lm[b][s][c]-lmmax[b][s]} * e^{am[b][t][c]-ammax[b][t]} + tiny )
//                + lmmax[b][s] + ammax[b][t]
//
// replaces torch.matmul(lm_probs, am_probs^T) + log of the reference
// (fast_rnnt/python/fast_rnnt/rnnt_loss.py:176-186, :1266-1272, :1296).
//
// One CTA per (utterance, 128 frames, up to 128 symbol positions).  Per 32-wide
// slice of the vocabulary:
//   * all 8 warps load the raw am / lm slices (16-byte loads, a row's 128 bytes
//     contiguous), apply exp(x - rowmax), split every value into a tf32 "hi"
//     and the fp32 remainder "lo" and store both in the 128-byte-swizzled
//     K-major layout the tensor core reads (the exp() is the prologue of the
//     contraction, so no exponentiated copy of am / lm ever exists in HBM);
//   * one thread issues 4 (K=8 steps) x 3 (hi*hi, hi*lo, lo*hi) tcgen05.mma
//     with the 128 x NP fp32 accumulator in tensor memory, then commits to an
//     mbarrier; the next slice is transformed into the other stage meanwhile.
// The tensor core adds into its accumulator with truncation, and all terms here
// are positive, so a single accumulator over the whole vocabulary would drift
// low by ~K * 2^-24 (2e-5 relative at C = 500).  Slices are therefore grouped
// (64 vocabulary entries per group), each group gets a fresh accumulator, and
// finished groups are folded into a running sum with round-to-nearest fp32
// adds (tcgen05.ld / add / tcgen05.st), one group behind the MMAs.
// Epilogue: tcgen05.ld (thread <-> frame), log(+tiny) + maxima, coalesced stores.
// Every mbarrier wait is bounded; on a timeout the tile is poisoned with NaN.
#include "common.cuh"
#include "umma.cuh"
#include "umma_linear.cuh"

namespace frnnt {

using namespace umma;

constexpr int kUmThreads = 256;
constexpr int kUmBM = 128;     // frames per CTA (the MMA's M)
constexpr int kUmBN = 128;     // symbol positions per CTA at most (the MMA's N)
constexpr int kUmBK = 32;      // vocabulary entries per stage (128 bytes)
constexpr int kUmStages = 2;
constexpr int kUmGroup = 2;    // slices per accumulator group
constexpr int kUmBRows = kUmBN / 32;  // 32-row blocks of the lm operand per thread

__global__ void __launch_bounds__(kUmThreads, 1)
norm_umma_kernel(const float *__restrict__ lm, const float *__restrict__ am,
                 const float *__restrict__ lmmax, const float *__restrict__ ammax,
                 float *__restrict__ norm, int S1, int T, int C) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_mma[kUmStages];  // a stage's MMAs are done
  __shared__ __align__(8) uint64_t bar_grp[2];          // a group's accumulator is complete
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y, t0 = blockIdx.x * kUmBM, s0 = blockIdx.z * kUmBN;
  const int ns = min(kUmBN, S1 - s0);   // symbol positions of this tile
  const int NP = (ns + 15) & ~15;       // the MMA's N
  const uint32_t idesc = idesc_tf32(kUmBM, NP, false, false);
  // tensor memory: two group accumulators and the running sum, 128 columns each
  constexpr uint32_t kCols = 512, kAcc1 = 128, kRun = 256;

  const uint32_t tiles = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  constexpr uint32_t a_bytes = kUmBM * 128, b_bytes = kUmBN * 128;
  constexpr uint32_t stage_bytes = 2 * a_bytes + 2 * b_bytes;
  uint8_t *tiles_ptr = smem_dyn + (tiles - smem_u32(smem_dyn));

  if (tid == 0) {
    for (int s = 0; s < kUmStages; ++s) mbar_init(&bar_mma[s], 1);
    mbar_init(&bar_grp[0], 1);
    mbar_init(&bar_grp[1], 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, kCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  const float *LM = lm + ((size_t)b * S1 + s0) * C;
  const float *AM = am + (size_t)b * T * C;
  const float *LMMAX = lmmax + (size_t)b * S1 + s0;
  const float *AMMAX = ammax + (size_t)b * T;

  // this thread's (row, 16-byte chunk) of every slice: chunk j, rows rb + 32 q
  const int j = tid & 7, rb = tid >> 3;
  float amax_r[4], lmax_r[kUmBRows];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int t = t0 + rb + 32 * q;
    amax_r[q] = t < T ? AMMAX[t] : 0.f;
  }
#pragma unroll
  for (int q = 0; q < kUmBRows; ++q) {
    const int s = rb + 32 * q;
    lmax_r[q] = s < ns ? LMMAX[s] : 0.f;
  }

  const int KB = (C + kUmBK - 1) / kUmBK;
  const int NG = (KB + kUmGroup - 1) / kUmGroup;
  const float4 ninf4 = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
  float4 ra[4], rl[kUmBRows];
  auto load_slice = [&](int kb) {
    const int k = kb * kUmBK + j * 4;
    const bool kv = k < C;  // C % 4 == 0: a chunk is entirely inside or outside
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int t = t0 + rb + 32 * q;
      ra[q] = (kv && t < T) ? *reinterpret_cast<const float4 *>(AM + (size_t)t * C + k) : ninf4;
    }
#pragma unroll
    for (int q = 0; q < kUmBRows; ++q) {
      const int s = rb + 32 * q;
      rl[q] = (kv && s < ns) ? *reinterpret_cast<const float4 *>(LM + (size_t)s * C + k) : ninf4;
    }
  };
  auto exp4 = [](const float4 &v, float m) {
    return make_float4(expf(v.x - m), expf(v.y - m), expf(v.z - m), expf(v.w - m));  // exp(-inf) = 0
  };

  // this warp's part of the accumulator: lanes 32*(warp%4).., half of the 16-column chunks
  const int quarter = warp & 3, half = warp >> 2;
  const int nchunks = NP / 16;
  const int ch_lo = half == 0 ? 0 : (nchunks + 1) / 2;
  const int ch_hi = half == 0 ? (nchunks + 1) / 2 : nchunks;
  const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
  // running sum (+)= accumulator of group g; `first` starts the running sum
  auto fold_group = [&](int g, bool first) {
    const uint32_t acc = tmem_base + lane_base + ((g & 1) ? kAcc1 : 0u);
    const uint32_t run = tmem_base + lane_base + kRun;
    for (int ch = ch_lo; ch < ch_hi; ++ch) {
      float p[16], r[16];
      tmem_ld16(acc + ch * 16, p);
      if (!first) {
        tmem_ld16(run + ch * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) p[i] = r[i] + p[i];
      }
      tmem_st16(run + ch * 16, p);
    }
  };

  load_slice(0);
  int failed = 0;
  for (int kb = 0; kb < KB; ++kb) {
    const int stage = kb % kUmStages;
    const int g = kb / kUmGroup;
    const bool group_start = kb % kUmGroup == 0;
    // the MMAs that read this stage two slices ago must be done
    if (kb >= kUmStages && !mbar_wait(&bar_mma[stage], (uint32_t)((kb / kUmStages - 1) & 1)))
      failed = 1;
    uint8_t *st = tiles_ptr + (size_t)stage * stage_bytes;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = rb + 32 * q;
      float4 hi, lo;
      split_tf32(exp4(ra[q], amax_r[q]), hi, lo);
      const uint32_t o = sw128_offset(r, j);
      *reinterpret_cast<float4 *>(st + o) = hi;
      *reinterpret_cast<float4 *>(st + a_bytes + o) = lo;
    }
#pragma unroll
    for (int q = 0; q < kUmBRows; ++q) {
      const int r = rb + 32 * q;
      if (r < NP) {
        float4 hi, lo;
        split_tf32(exp4(rl[q], lmax_r[q]), hi, lo);
        const uint32_t o = sw128_offset(r, j);
        *reinterpret_cast<float4 *>(st + 2 * a_bytes + o) = hi;
        *reinterpret_cast<float4 *>(st + 2 * a_bytes + b_bytes + o) = lo;
      }
    }
    if (kb + 1 < KB) load_slice(kb + 1);
    // group g is about to reuse the accumulator of group g-2: fold that one away first
    if (group_start && g >= 2 && !failed) {
      if (mbar_wait(&bar_grp[g & 1], (uint32_t)(((g - 2) >> 1) & 1))) {
        tc_fence_after_sync();
        fold_group(g - 2, g == 2);
      } else {
        failed = 1;
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    failed = __syncthreads_or(failed);
    if (failed) break;
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t acc = tmem_base + ((g & 1) ? kAcc1 : 0u);
      const uint32_t sa = tiles + (uint32_t)stage * stage_bytes;
      const uint32_t a_hi = sa, a_lo = sa + a_bytes, b_hi = sa + 2 * a_bytes,
                     b_lo = sa + 2 * a_bytes + b_bytes;
#pragma unroll
      for (int ks = 0; ks < kUmBK / 8; ++ks) {
        const uint32_t ko = ks * 32;  // 8 floats further along the 128-byte rows
        const uint64_t dah = smem_desc_sw128(a_hi + ko, 16, 1024);
        const uint64_t dal = smem_desc_sw128(a_lo + ko, 16, 1024);
        const uint64_t dbh = smem_desc_sw128(b_hi + ko, 16, 1024);
        const uint64_t dbl = smem_desc_sw128(b_lo + ko, 16, 1024);
        mma_tf32(acc, dah, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
        mma_tf32(acc, dah, dbl, idesc, 1u);
        mma_tf32(acc, dal, dbh, idesc, 1u);
      }
      mma_commit(&bar_mma[stage]);
      if (kb % kUmGroup == kUmGroup - 1 || kb == KB - 1) mma_commit(&bar_grp[g & 1]);
    }
  }

  // the last two groups are still in their accumulators: wait for them
  if (!failed) {
    if (NG >= 2 && !mbar_wait(&bar_grp[(NG - 2) & 1], (uint32_t)(((NG - 2) >> 1) & 1))) failed = 1;
    if (!mbar_wait(&bar_grp[(NG - 1) & 1], (uint32_t)(((NG - 1) >> 1) & 1))) failed = 1;
  }
  failed = __syncthreads_or(failed);
  tc_fence_after_sync();

  // epilogue: (running sum + second-to-last group) + last group -> log -> global
  {
    const int t = t0 + 32 * quarter + lane;
    const float am_max = t < T ? AMMAX[t] : 0.f;
    float *NB = norm + ((size_t)b * S1 + s0) * T;
    const uint32_t acc0 = tmem_base + lane_base, acc1 = acc0 + kAcc1, run = acc0 + kRun;
    for (int ch = ch_lo; ch < ch_hi; ++ch) {
      float v[16];
      if (!failed) {
        if (NG >= 3) {
          float p[16];
          tmem_ld16(run + ch * 16, v);
          tmem_ld16(((NG - 2) & 1 ? acc1 : acc0) + ch * 16, p);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += p[i];
          tmem_ld16(((NG - 1) & 1 ? acc1 : acc0) + ch * 16, p);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += p[i];
        } else if (NG == 2) {
          float p[16];
          tmem_ld16(acc0 + ch * 16, v);
          tmem_ld16(acc1 + ch * 16, p);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] += p[i];
        } else {
          tmem_ld16(acc0 + ch * 16, v);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = NAN;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int s = ch * 16 + i;
        if (s < ns && t < T)
          NB[(size_t)s * T + t] = logf(v[i] + 1.17549435e-38f) + LMMAX[s] + am_max;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kCols);
}

bool norm_umma_supported(const void *lm, const void *am, int S1, int T, int C) {
  return C % 4 == 0 && C >= 4 && S1 >= 1 && T >= 1 && (S1 + kUmBN - 1) / kUmBN <= 65535 &&
         (uintptr_t)lm % 16 == 0 && (uintptr_t)am % 16 == 0;
}

int launch_norm_umma(const float *lm, const float *am, const float *lmmax, const float *ammax,
                     float *norm, int B, int S1, int T, int C, cudaStream_t st) {
  const size_t smem = (size_t)kUmStages * (2 * kUmBM * 128 + 2 * kUmBN * 128) + 1024;
  FRNNT_CUDA(cudaFuncSetAttribute(norm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem));
  dim3 grid((unsigned)((T + kUmBM - 1) / kUmBM), (unsigned)B, (unsigned)((S1 + kUmBN - 1) / kUmBN));
  FRNNT_KERNEL(norm_umma_kernel<<<grid, kUmThreads, smem, st>>>(lm, am, lmmax, ammax, norm, S1, T, C));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

// ---- gradient contractions -------------------------------------------------------------
// Both run on the engine in umma_linear.cuh, batched over the utterances (3-D tensor
// maps: rows / columns outside an utterance's matrix arrive as zeros), with the
// exponentiated operand produced in the engine's split pass and the remaining
// factors applied in its epilogue; no exponentiated copy of am / lm exists in HBM.
//
// dlm[s][c] = -L[s][c] * sum_t Rw[s][t] A[t][c]  (+ lm-only / unigram terms)
//   tile: M = s, N = c, K = t
//   A operand = Rw[s][t]:                contiguous along t -> K-major
//   B operand = e^{am[t][c]-ammax[t]}:   contiguous along c -> MN-major, shift = ammax
struct LmGradExt {
  static constexpr bool kBatched = true, kExpB = true, kColSumA = false;
  __device__ float *a_colsum(int, int) const { return nullptr; }
  const float *ammax, *lm, *lmmax, *lmsum, *gl, *dp, *rowdot;
  float *lm_grad;
  int S1, T, C;
  __device__ const float *b_shift(int b) const { return ammax + (size_t)b * T; }
  __device__ const float *pre_row(int b, int s) const { return lm + ((size_t)b * S1 + s) * C; }
  __device__ float *out_row(int b, int s) const { return lm_grad + ((size_t)b * S1 + s) * C; }
  __device__ void finish(int b, int s, int c0, float (&v)[16], const float (&x)[16]) const {
    const size_t row = (size_t)b * S1 + s;
    const float mx = lmmax[row];
    const float inv_sum = gl != nullptr ? 1.f / lmsum[row] : 0.f;
    const float g = gl != nullptr ? gl[row] : 0.f;
    const float rd = (gl != nullptr && dp != nullptr) ? rowdot[row] : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float L = expf(x[i] - mx);
      float r = -(L * v[i]);
      if (gl != nullptr) {
        const float P = L * inv_sum;
        r -= g * P;
        if (dp != nullptr && c0 + i < C) r += P * (dp[c0 + i] - rd);
      }
      v[i] = r;
    }
  }
};

// dam[t][c] = -A[t][c] * sum_s Rw[s][t] L[s][c]  (+ am-only term)
//   tile: M = t, N = c, K = s
//   A operand = Rw[s][t]:                contiguous along t = M -> MN-major
//   B operand = e^{lm[s][c]-lmmax[s]}:   contiguous along c -> MN-major, shift = lmmax
struct AmGradExt {
  static constexpr bool kBatched = true, kExpB = true, kColSumA = false;
  __device__ float *a_colsum(int, int) const { return nullptr; }
  const float *lmmax, *am, *ammax, *h, *uni, *amonly;
  float *am_grad;
  int S1, T, C;
  __device__ const float *b_shift(int b) const { return lmmax + (size_t)b * S1; }
  __device__ const float *pre_row(int b, int t) const { return am + ((size_t)b * T + t) * C; }
  __device__ float *out_row(int b, int t) const { return am_grad + ((size_t)b * T + t) * C; }
  __device__ void finish(int b, int t, int c0, float (&v)[16], const float (&x)[16]) const {
    const size_t row = (size_t)b * T + t;
    const float mx = ammax[row];
    const float w = h != nullptr ? h[row] * expf(mx - amonly[row]) : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float A = expf(x[i] - mx);
      float r = -(A * v[i]);
      if (h != nullptr && c0 + i < C) r -= w * A * uni[c0 + i];
      v[i] = r;
    }
  }
};

int launch_simple_grads_umma(const float *lm, const float *am, const float *lmmax,
                             const float *lmsum, const float *ammax, const float *amonly,
                             const float *uni, const float *rw, const float *gl, const float *h,
                             const float *dp, const float *rowdot, float *lm_grad, float *am_grad,
                             int B, int S1, int T, int C, int Tp, cudaStream_t st) {
  if (B == 0 || C == 0) return FRNNT_OK;
  const int ctiles = (C + kLinTile - 1) / kLinTile;
  CUtensorMap ma, mb;
  int rc;
  {
    rc = make_operand_map(&ma, rw, S1, T, Tp, (long long)S1 * Tp, B, false);
    if (rc == FRNNT_OK) rc = make_operand_map(&mb, am, T, C, C, (long long)T * C, B, true);
    if (rc != FRNNT_OK) return rc;
    const LinShape shape{S1, C, T, ((T + kLinBK - 1) / kLinBK) * kLinBK, (S1 + kLinTile - 1) / kLinTile,
                         ctiles, B};
    const LmGradExt ext{ammax, lm, lmmax, lmsum, gl, dp, rowdot, lm_grad, S1, T, C};
    rc = launch_linear_umma<false, true>(ma, mb, shape, ext, st);
    if (rc != FRNNT_OK) return rc;
  }
  if (T > 0) {
    rc = make_operand_map(&ma, rw, S1, T, Tp, (long long)S1 * Tp, B, true);
    if (rc == FRNNT_OK) rc = make_operand_map(&mb, lm, S1, C, C, (long long)S1 * C, B, true);
    if (rc != FRNNT_OK) return rc;
    const LinShape shape{T, C, S1, ((S1 + kLinBK - 1) / kLinBK) * kLinBK, (T + kLinTile - 1) / kLinTile,
                         ctiles, B};
    const AmGradExt ext{lmmax, am, ammax, h, uni, amonly, am_grad, S1, T, C};
    rc = launch_linear_umma<true, true>(ma, mb, shape, ext, st);
    if (rc != FRNNT_OK) return rc;
  }
  return FRNNT_OK;
}

}  // namespace frnnt
