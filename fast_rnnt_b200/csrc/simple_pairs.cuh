// Interface between simple.cu (drivers, element-wise kernels, float64 / SIMT paths) and
// simple_pairs.cu (the float32 tensor-core path of the simple lattices on the fp16-pair engine).
#pragma once
#include <algorithm>

#include "common.cuh"

namespace frnnt {

// extra state of the tensor-core path: `saved_bytes` follow the regular saved area (kept
// from forward to backward), `scratch_bytes` follow the regular scratch area
struct SimplePairsLayout {
  int Cp, Tq;  // row pitches (halves) of the planes with C resp. T entries per row
  int Sp;      // row pitch (floats) of am_sym [B][T][Sp] = am[b][t][symbols[b][s]]
  size_t lp_hi, lp_lo, ap_hi, ap_lo, lm_blk, lm_sym, lnorm, am_blk, am_sym, saved_bytes;
  size_t rw_hi, rw_lo, parts, inv_scale, scratch_bytes;
  SimplePairsLayout(int B, int S, int T, int C);
};

// offset, inside the pairs scratch, of the per-row maxima of |rw| that the caller fills in
// (B*(S+1) floats) before launch_simple_grads_pairs
size_t simple_pairs_rowmax_offset(int B, int S, int T, int C);

bool simple_pairs_supported(const void *lm, const void *am, int S1, int T, int C, int rnnt_type);

// stage 0: row maxima / sums, exp planes, per-row scalars, the -inf column of px;
// stage 1: normalizer product + lattices (needs amonly / loguni when the am-only branch is on;
// a positive delay_penalty is added to px as the reference's loss functions do)
// lm / am: float32, or 16-bit values when input_dtype is FRNNT_F16 / FRNNT_BF16 (only stage 0 reads them)
int launch_simple_forward_pairs(const void *lm, const void *am, const int64_t *symbols,
                                const int64_t *boundary, int blank, int rnnt_type, int smoothed,
                                int am_only_off, float both, float ls, float as, float *px, float *py,
                                float *norm, float *lmmax, float *lmsum, float *ammax,
                                const float *amonly, const float *loguni, void *pairs_saved, int B, int S,
                                int T, int C, int stage, cudaStream_t st, double delay_penalty = 0.0,
                                int input_dtype = FRNNT_F32);

// lm_grad / am_grad without the one-hot terms, from the gradient weights rw [B][S+1][Tp] and
// the maxima of |rw| per row (see simple_pairs_rowmax_offset)
int launch_simple_grads_pairs(const float *rw, const float *lmsum, const float *ammax, const float *amonly,
                              const float *uni, const float *gl, const float *h, const float *dp,
                              const float *rowdot, float *lm_grad, float *am_grad, const void *pairs_saved,
                              void *pairs_scratch, int B, int S, int T, int C, int Tp, cudaStream_t st);

}  // namespace frnnt
