/*
 * C ABI of libfrnnt_sm100.so -- the pruned RNN-T loss hot path of k2-fsa/fast_rnnt
 * as hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions for every entry point
 *   - returns 0 on success, a negative FRNNT_E* code otherwise; the message of
 *     the last failure on the calling thread is in frnnt_last_error();
 *   - arguments are checked on the host BEFORE anything is launched;
 *   - every pointer is a DEVICE pointer on the current CUDA device unless it is
 *     documented as a host pointer; tensors are contiguous and row-major;
 *   - `dtype` is FRNNT_F32 or FRNNT_F64 (the reference dispatches over float
 *     and double only, fast_rnnt/csrc/mutual_information_cuda.cu:715, :788);
 *     two forwards also read their large inputs as FRNNT_F16 / FRNNT_BF16 (see there);
 *   - three environment variables, read at call time, select an alternative kernel for
 *     the same result: FRNNT_CONTRACTION=tf32|simt, FRNNT_MI=row_per_thread,
 *     FRNNT_PAIR_TILE=128;
 *   - symbols, boundaries and ranges are int64, as in the reference's API;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and
 *     nothing synchronises;
 *   - nothing allocates device memory: outputs and scratch are the caller's
 *     (scratch sizes come from the frnnt_*_bytes / frnnt_*_floats functions next
 *     to each entry point);
 *   - re-entrant.  Global state: the thread-local error string, the launch
 *     counter, a per-device cache of the multiprocessor count, and -- for
 *     frnnt_mi_fwd_bwd_noalloc only -- the built-in scratch region and its cached
 *     per-device address;
 *   - waits inside the kernels are bounded.  A wait that runs out does not fail
 *     the call (nothing synchronises, so the host cannot know): the affected
 *     outputs are poisoned with NaN instead -- ans[b] of the forward recursion,
 *     the first in-box gradient entry (and origin_grad[b]) of the reverse sweep,
 *     the output tile of a tensor-core product.
 *
 * Lattice layouts (identical to the reference's tensors):
 *   px   [B][S][T1]     T1 = T+1 ("regular") or T ("modified"/"constrained")
 *   py   [B][S+1][T]
 *   p    [B][S+1][T+1]
 *   boundary [B][4] = (s_begin, t_begin, s_end, t_end), or NULL for (0,0,S,T)
 */
#ifndef FRNNT_H_
#define FRNNT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FRNNT_F32 0
#define FRNNT_F64 1
/* 16-bit INPUTS (IEEE half, bfloat16), accepted where a function says so: the named inputs
 * are read as 16-bit values and converted (exactly) to float32 on load; lattices, saved
 * state, gradients and every other argument are float32, and the results are those of the
 * FRNNT_F32 call on the converted inputs, bit for bit. */
#define FRNNT_F16 2
#define FRNNT_BF16 3

#define FRNNT_OK 0
#define FRNNT_EINVAL (-1)      /* null pointer, bad dtype, negative size, misalignment */
#define FRNNT_EUNSUPPORTED (-2) /* a size beyond what the kernels are built for */
#define FRNNT_ECUDA (-3)       /* the CUDA runtime refused a launch or an attribute */

#define FRNNT_REGULAR 0
#define FRNNT_MODIFIED 1
#define FRNNT_CONSTRAINED 2

/* Library version (major*10000 + minor*100 + patch). */
int frnnt_version(void);

/* Message of the last failure on this thread ("" if none). */
const char *frnnt_last_error(void);

/* Number of CUDA kernels this library has launched in this process so far
 * (diagnostic; no counterpart in the reference). */
long long frnnt_launch_count(void);

/* Replaces the pybind function with_cuda()
 * (fast_rnnt/python/csrc/mutual_information.cu:69-75): always 1. */
int frnnt_with_cuda(void);

/* ----------------------------------------------------------------------------
 * Mutual-information recursion
 * ------------------------------------------------------------------------- */

/* Bytes of the `lattice` scratch of the functions below: the forward sweep
 * stores there, by anti-diagonal ([B][S+T+1][round_up(S+1,32)]), the exponent of
 * every cell's backward weight, p[s-1][t+o] + px[s-1][t+o] - p[s][t], so that it
 * writes it and the backward sweep reads it fully coalesced; two vectors of
 * S+T+65 values per utterance follow (see frnnt_mi_rows_per_block). */
size_t frnnt_mi_lattice_bytes(int dtype, int B, int S, int T);

/* Lattice rows (S+1) that one launch sweeps: 256 for FRNNT_F32, 128 for
 * FRNNT_F64.  A taller lattice is swept in blocks of that many rows, one launch
 * per block and direction (the reference tiles in 32x32 blocks and launches once
 * per anti-diagonal of tiles, mutual_information_cuda.cu:680-731).  The row above
 * a block and the gradients that cross a block edge travel from launch to launch
 * through the two vectors at the end of `lattice`, which frnnt_mi_forward then
 * requires and which is why the reverse sweep takes it non-const. */
int frnnt_mi_rows_per_block(int dtype);

/* Forward recursion.  Replaces mutual_information_forward(px, py, boundary, p)
 * of the reference's extension module (fast_rnnt/python/csrc/mutual_information.cu:27-45,
 * MutualInformationCuda at fast_rnnt/csrc/mutual_information_cuda.cu:676-728).
 *   p       ([B][S+1][T+1], the reference's layout) may be NULL when the caller
 *           does not need the lattice;
 *   lattice (scratch, see above) may be NULL when no backward sweep will follow
 *           and S+1 <= frnnt_mi_rows_per_block(dtype);
 *   ans     [B] receives p[b][s_end][t_end]. */
int frnnt_mi_forward(int dtype, const void *px, const void *py, const int64_t *boundary,
                     void *p, void *ans, void *lattice, int B, int S, int T, int modified,
                     void *stream);

/* Reverse sweep from the `lattice` written by frnnt_mi_forward (px is not read
 * any more and may be NULL): px_grad [B][S][T1] and py_grad [B][S+1][T] are fully written (exact
 * zeros outside the boundary box).  origin_grad (may be NULL) receives the
 * gradient that reaches p[s_begin][t_begin], which equals ans_grad[b] up to
 * rounding when the sweep is right (the reference overwrites ans_grad with it,
 * mutual_information_cuda.cu:667-669). */
int frnnt_mi_backward_from_lattice(int dtype, const void *px, void *lattice,
                                   const int64_t *boundary, const void *ans_grad, void *px_grad,
                                   void *py_grad, void *origin_grad, int B, int S, int T,
                                   int modified, void *stream);

/* Reverse sweep from a lattice `p` in the reference's layout.  Replaces
 * mutual_information_backward(px, py, boundary, p, ans_grad)
 * (fast_rnnt/python/csrc/mutual_information.cu:47-67, MutualInformationBackwardCuda
 * at mutual_information_cuda.cu:734-805).  `lattice` is scratch of
 * frnnt_mi_lattice_bytes() bytes. */
int frnnt_mi_backward(int dtype, const void *px, const void *py, const int64_t *boundary,
                      const void *p, const void *ans_grad, void *px_grad, void *py_grad,
                      void *origin_grad, void *lattice, int B, int S, int T, int modified,
                      void *stream);

/* Size of the scratch region built into the library for frnnt_mi_fwd_bwd_noalloc. */
#define FRNNT_MI_NOALLOC_SCRATCH_BYTES (32u << 20)

/* Forward + reverse sweep in one call, for callers that may not allocate.
 * (No counterpart in the reference, whose extension allocates its outputs and
 * its p_grad work array itself.)
 *
 * Who needs it: a host program that hands this library a fixed set of buffers
 * and cannot obtain one more -- e.g. a C/C++ training or scoring loop that
 * carved up all of its device memory at start-up, or a plugin host that bans
 * cudaMalloc after initialisation because an allocation stalls every stream of
 * the device.  frnnt_mi_forward / frnnt_mi_backward_from_lattice need a
 * caller-provided scratch of frnnt_mi_lattice_bytes(); this entry point instead
 * keeps the lattice in a region of FRNNT_MI_NOALLOC_SCRATCH_BYTES
 * (32 MiB) that is part of the library image: every GPU whose context loads the
 * library's code holds those 32 MiB until the process exits.  With CUDA's
 * default lazy module loading that happens at the first call into the module,
 * which may itself stall or run out of memory on a host that has given all of
 * it away: make one warm-up call during initialisation (or run with
 * CUDA_MODULE_LOADING=EAGER), after which calls take nothing from the device.
 *
 *   - inputs px, py, boundary, ans_grad [B] and outputs ans [B], px_grad, py_grad
 *     are the caller's, exactly as for the two functions it combines;
 *   - a lattice with frnnt_mi_lattice_bytes(dtype,B,S,T) above the limit is
 *     refused with FRNNT_EUNSUPPORTED before anything is launched;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine;
 *   - the FIRST call on each device looks up the region's device address (with
 *     that device current); make that first call outside of any stream capture.
 *     The address is cached per device ordinal and does not survive a
 *     cudaDeviceReset() of that device: do not reset a device between calls;
 *   - every argument is checked before the first of the two sweeps is launched;
 *   - all calls on a device share the one region, which still holds the previous
 *     call's lattice when the next call starts (nothing needs clearing: each
 *     call overwrites what it later reads).  Two calls whose kernels overlap on
 *     the GPU (different streams, or different host threads on different
 *     streams) race on it: issue them on one stream, or order them yourself. */
int frnnt_mi_fwd_bwd_noalloc(int dtype, const void *px, const void *py, const int64_t *boundary,
                             const void *ans_grad, void *ans, void *px_grad, void *py_grad,
                             int B, int S, int T, int modified, void *stream);

/* ----------------------------------------------------------------------------
 * Log-prob lattices from factorised encoder / decoder outputs ("simple" loss)
 * ------------------------------------------------------------------------- */

/* Bytes of the state the forward keeps for the backward, and of the per-call
 * temporaries, of the two functions below. */
size_t frnnt_simple_saved_bytes(int dtype, int B, int S, int T, int C);
size_t frnnt_simple_scratch_bytes(int dtype, int B, int S, int T, int C);

/* px [B][S][T1], py [B][S+1][T] from lm [B][S+1][C], am [B][T][C], symbols [B][S].
 * smoothed == 0 replaces get_rnnt_logprobs (fast_rnnt/python/fast_rnnt/rnnt_loss.py:66-227);
 * smoothed != 0 replaces get_rnnt_logprobs_smoothed (rnnt_loss.py:1135-1369) with its
 * lm_only_scale / am_only_scale (exact zeros become 1e-20 as in the reference).
 * rnnt_type is FRNNT_REGULAR / FRNNT_MODIFIED / FRNNT_CONSTRAINED; boundary may be NULL.
 * delay_penalty > 0 adds delay_penalty * ((T_b - 1) / 2 - t) to px[b][s][t] as the
 * reference's loss functions do between the lattices and the recursion
 * (rnnt_loss.py:309-324, :516-531, :1101-1116, :1463-1478; T_b = boundary[b][3], or T),
 * with torch's roundings; 0 for the plain get_rnnt_logprobs* functions.  The same argument
 * of frnnt_lsm_gather_forward and frnnt_pruned_joiner_logprobs_forward means the same. */
/* 1 if frnnt_simple_logprobs_forward / _backward accept dtype FRNNT_F16 / FRNNT_BF16 (16-bit lm
 * and am, everything else float32) for these sizes: the float32 tensor-core path must apply
 * (C a multiple of 4, ...) and the am-only branch must be off (not smoothed, or
 * am_only_scale == 0), because only that path reads lm and am in a single kernel.  Otherwise
 * convert the inputs to float32 first (same results). */
int frnnt_simple_reads_16bit_inputs(int S, int T, int C, int rnnt_type, int smoothed,
                                    double am_only_scale);

int frnnt_simple_logprobs_forward(int dtype, const void *lm, const void *am,
                                  const int64_t *symbols, const int64_t *boundary, int blank,
                                  int rnnt_type, int smoothed, double lm_only_scale,
                                  double am_only_scale, double delay_penalty, void *px, void *py,
                                  void *saved, void *scratch, int B, int S, int T, int C,
                                  void *stream);

/* Gradient of the above w.r.t. lm and am given the gradients of px and py
 * (what autograd derives for the reference's composition of ATen ops).
 * lm_grad [B][S+1][C] and am_grad [B][T][C] are fully written. */
int frnnt_simple_logprobs_backward(int dtype, const void *lm, const void *am,
                                   const int64_t *symbols, const int64_t *boundary, int blank,
                                   int rnnt_type, int smoothed, double lm_only_scale,
                                   double am_only_scale, const void *px_grad, const void *py_grad,
                                   const void *saved, void *scratch, void *lm_grad, void *am_grad,
                                   int B, int S, int T, int C, void *stream);

/* ----------------------------------------------------------------------------
 * Log-prob lattices from joiner logits (pruned and unpruned)
 * ------------------------------------------------------------------------- */

/* logits [B][T][R][C] -> lse, px_band, py_band (each [B][T][R]) and, unless px
 * and py are NULL, the lattices px [B][S][T1], py [B][S+1][T].
 * With ranges [B][T][R] this replaces get_rnnt_logprobs_pruned
 * (rnnt_loss.py:856-1024); with ranges == NULL and R == S+1 it replaces
 * get_rnnt_logprobs_joint (rnnt_loss.py:343-449). */
int frnnt_lsm_gather_forward(int dtype, const void *logits, const int64_t *symbols,
                             const int64_t *ranges, const int64_t *boundary, void *lse,
                             void *px_band, void *py_band, void *px, void *py, int B, int T,
                             int R, int S, int C, int blank, int rnnt_type, double delay_penalty,
                             void *stream);

/* Gradient of the above w.r.t. the logits; logits_grad [B][T][R][C] is fully written. */
int frnnt_lsm_gather_backward(int dtype, const void *logits, const int64_t *symbols,
                              const int64_t *ranges, const int64_t *boundary, const void *lse,
                              const void *px_grad, const void *py_grad, void *logits_grad, int B,
                              int T, int R, int S, int C, int blank, int rnnt_type, void *stream);

/* ----------------------------------------------------------------------------
 * Pruning
 * ------------------------------------------------------------------------- */

/* ranges [B][T][s_range] (int64) from the occupancies px_grad [B][S][T1] and
 * py_grad [B][S+1][T].  Replaces the device part of get_rnnt_prune_ranges
 * (rnnt_loss.py:726-777); s_range is the value AFTER the host-side adjustment
 * of rnnt_loss.py:699-724 and must lie in [1, S+1].  boundary is required. */
int frnnt_prune_ranges(int dtype, const void *px_grad, const void *py_grad,
                       const int64_t *boundary, int64_t *ranges, int B, int S, int T, int T1,
                       int s_range, void *stream);

/* out [B][T][R][D] = lm [B][S1][D] gathered at ranges [B][T][R]: the lm half of
 * do_rnnt_pruning (rnnt_loss.py:813-817; the am half is a stride-0 view). */
int frnnt_prune_gather(int dtype, const void *lm, const int64_t *ranges, void *out, int B,
                       int S1, int T, int R, int D, void *stream);

/* lm_grad [B][S1][D] = scatter-add of out_grad [B][T][R][D] (deterministic). */
int frnnt_prune_gather_backward(int dtype, const void *out_grad, const int64_t *ranges,
                                void *lm_grad, int B, int S1, int T, int R, int D, void *stream);

/* ----------------------------------------------------------------------------
 * fp32-accurate matrix products for the caller's joiner (next to the hot path)
 * ------------------------------------------------------------------------- */

/* The reference leaves the joiner between do_rnnt_pruning and rnnt_loss_pruned
 * to the caller (README.md:180-190: a Linear over tanh(am_pruned + lm_pruned));
 * it has no counterpart of these two functions.  They run the three products
 * of a linear layer on the tensor cores with 3xTF32 splitting (fp32-level
 * accuracy), fed by TMA.  All matrices are row-major float32 with 16-byte
 * aligned bases and row lengths that are multiples of 4.
 *
 * D[M][N] = A[M][K] * B[N][K]^T (+ bias[N] if not NULL); if tanh_out [M][N] is not
 * NULL every result is multiplied by 1 - tanh_out^2 (the derivative of a tanh whose
 * output is tanh_out: the backward of the joiner's activation, fused). */
int frnnt_matmul_nt(const float *a, const float *b, const float *bias, const float *tanh_out,
                    float *d, int M, int N, int K, void *stream);

/* D[M][N] = A[R][M]^T * B[R][N].  The reduction over R is split over
 * frnnt_matmul_tn_splits(M, N, R) work items per output tile; `partials` is scratch
 * of splits*M*N floats (may be NULL when splits == 1). */
int frnnt_matmul_tn_splits(int M, int N, int R);
int frnnt_matmul_tn(const float *a, const float *b, float *d, float *partials, int M, int N, int R,
                    void *stream);

/* The same product that, when a_colsum is not NULL, also returns a_colsum[m] =
 * sum over r of A[r][m], taken from the operand tiles as they pass through the
 * split pass (for a linear layer: grad_weight and grad_bias from one read of
 * grad_out).  `scratch` holds frnnt_matmul_tn_scratch_floats(M, N, R) floats. */
size_t frnnt_matmul_tn_scratch_floats(int M, int N, int R);
int frnnt_matmul_tn_colsum(const float *a, const float *b, float *d, float *a_colsum, float *scratch,
                           int M, int N, int R, void *stream);

/* act[B][T][R][D] = tanh(enc[B][T][D] + dec[B][S1][D] gathered at ranges[B][T][R]): the
 * joiner's input, i.e. tanh(am_pruned + lm_pruned) of the reference's usage
 * (README.md:180-186) without materialising the two pruned tensors. */
int frnnt_pruned_tanh(int dtype, const void *enc, const void *dec, const int64_t *ranges,
                      void *act, int B, int S1, int T, int R, int D, void *stream);

/* out[frames][D] = sum over k of gz[frames][R][D] (gradient of the stride-0 am_pruned view). */
int frnnt_sum_over_range(int dtype, const void *gz, void *out, long long frames, int R, int D,
                         void *stream);

/* Both input gradients of the pruned joiner from one pass over gz [B][T][R][D], the
 * gradient with respect to enc[b][t] + dec[b][ranges[b][t][k]] (no counterpart in the
 * reference, which leaves them to autograd through do_rnnt_pruning's expand and gather):
 *   enc_grad [B][T][D]  = sum over k           (what frnnt_sum_over_range gives),
 *   dec_grad [B][S1][D] = the scatter-add over ranges (what frnnt_prune_gather_backward gives).
 * float32, D a multiple of 4, 16-byte aligned pointers; `scratch` holds
 * frnnt_joiner_input_grads_scratch_bytes(B, T, D) bytes.  enc_grad may be NULL: the
 * call is then a faster frnnt_prune_gather_backward.  Sums are taken in a fixed
 * order for ranges whose rows move by less than a row per frame (the ones
 * frnnt_prune_ranges writes); other ranges are handled with atomic adds. */
size_t frnnt_joiner_input_grads_scratch_bytes(int B, int T, int D);
int frnnt_joiner_input_grads(const float *gz, const int64_t *ranges, float *enc_grad, float *dec_grad,
                             void *scratch, int B, int S1, int T, int R, int D, void *stream);

/* ----------------------------------------------------------------------------
 * Pruned joiner and pruned log-prob lattices as one operator
 * ------------------------------------------------------------------------- */

/* px [B][S][T1], py [B][S+1][T] of the pruned loss straight from the joiner's inputs:
 *   logits[b][t][k][:] = weight * tanh(enc[b][t][:] + dec[b][ranges[b][t][k]][:]) + bias
 *   (px, py) = get_rnnt_logprobs_pruned(logits, symbols, ranges, ...)
 * i.e. do_rnnt_pruning (fast_rnnt/python/fast_rnnt/rnnt_loss.py:780-818), the joiner of
 * the reference's documented usage (README.md:180-190, which the reference leaves to the
 * caller) and get_rnnt_logprobs_pruned (rnnt_loss.py:856-1024) in one call; the reference
 * has no counterpart of the combination.  float32 only.
 *   enc [B][T][D], dec [B][S+1][D], ranges [B][T][R], weight [C][D], bias [C] or NULL,
 *   symbols [B][S], boundary [B][4] or NULL; D a multiple of 8, C a multiple of 4.
 * The three products run on the tensor cores from operands stored as pairs of fp16
 * planes (x * 2^e = hi + lo, 22 significant bits, e chosen per operand from its largest
 * magnitude): fp32-level accuracy at the fp16 rate.  The log-sum-exp over C comes out of
 * the forward product's epilogue.
 * input_dtype is FRNNT_F32, or FRNNT_F16 / FRNNT_BF16 for 16-bit enc and dec (the
 * gradients enc_grad / dec_grad of the backward call stay float32).
 * `saved` (frnnt_pruned_joiner_saved_bytes) must stay untouched until the backward call;
 * `scratch` is per-call (…_forward_scratch_bytes / …_backward_scratch_bytes); both
 * 256-byte aligned. */
size_t frnnt_pruned_joiner_saved_bytes(int B, int T, int R, int S, int C, int D);
size_t frnnt_pruned_joiner_forward_scratch_bytes(int B, int T, int R, int S, int C, int D);
size_t frnnt_pruned_joiner_backward_scratch_bytes(int B, int T, int R, int S, int C, int D);
int frnnt_pruned_joiner_logprobs_forward(int input_dtype, const void *enc, const void *dec,
                                         const int64_t *ranges,
                                         const float *weight, const float *bias,
                                         const int64_t *symbols, const int64_t *boundary, float *px,
                                         float *py, void *saved, void *scratch, int B, int T, int R,
                                         int S, int C, int D, int blank, int rnnt_type,
                                         double delay_penalty, void *stream);

/* Gradients of the above given the gradients of px and py: enc_grad [B][T][D] and
 * dec_grad [B][S+1][D] (both or neither), weight_grad [C][D], bias_grad [C] (each may be
 * NULL); all fully written.  Sums are taken in a fixed order (no atomics) for ranges
 * written by frnnt_prune_ranges. */
int frnnt_pruned_joiner_logprobs_backward(const float *px_grad, const float *py_grad,
                                          const int64_t *ranges, const int64_t *symbols,
                                          const int64_t *boundary, void *saved, void *scratch,
                                          float *enc_grad, float *dec_grad, float *weight_grad,
                                          float *bias_grad, int B, int T, int R, int S, int C, int D,
                                          int blank, int rnnt_type, void *stream);

/* Diagnostics (for per-kernel timing; no counterpart in the reference): the same arguments
 * as the two calls above, but only ONE part of the call is launched, on buffers that a
 * complete forward (and, for the backward parts, backward) call has filled before.
 * forward parts: 0 = planes of the weights and of tanh(enc + dec), 1 = the product
 * (logits + log-sum-exp partials), 2 = bands and lattices.  backward parts: 0 = planes of
 * d loss / d logits (+ bias gradient), 1 = grad-input product, 3 = grad-weight product,
 * 4 = enc / dec gradients from the grad-input result. */
int frnnt_pruned_joiner_logprobs_forward_part(int part, const float *enc, const float *dec,
                                              const int64_t *ranges, const float *weight,
                                              const float *bias, const int64_t *symbols,
                                              const int64_t *boundary, float *px, float *py, void *saved,
                                              void *scratch, int B, int T, int R, int S, int C, int D,
                                              int blank, int rnnt_type, void *stream);
int frnnt_pruned_joiner_logprobs_backward_part(int part, const float *px_grad, const float *py_grad,
                                               const int64_t *ranges, const int64_t *symbols,
                                               const int64_t *boundary, void *saved, void *scratch,
                                               float *enc_grad, float *dec_grad, float *weight_grad,
                                               float *bias_grad, int B, int T, int R, int S, int C, int D,
                                               int blank, int rnnt_type, void *stream);

/* ----------------------------------------------------------------------------
 * Products of matrices stored as pairs of fp16 planes (no counterpart in the reference)
 * ------------------------------------------------------------------------- */

/* The engine behind the fused joiner on its own.  A float32 matrix x [rows][cols] becomes
 * two fp16 planes hi, lo [rows][pitch] (pitch >= cols, a multiple of 8) with
 * x * 2^e = hi + lo, e chosen from the largest |x|; *inv_scale (device) receives 2^-e.
 * `scratch` holds frnnt_pairs_scratch_floats() floats. */
size_t frnnt_pairs_scratch_floats(void);
int frnnt_pairs_from_f32(const float *x, long long rows, int cols, long long pitch, void *hi, void *lo,
                         float *inv_scale, float *scratch, void *stream);

/* D[M][N] = A[M][K] * B[N][K]^T (+ bias[N]), A and B given as planes with row pitches
 * pitch_a / pitch_b (in halves) and their inverse scales (device pointers). */
int frnnt_pair_matmul_nt(const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
                         const float *inv_scale_a, const float *inv_scale_b, const float *bias,
                         float *d, int M, int N, int K, long long pitch_a, long long pitch_b,
                         void *stream);

/* D[M][N] = A[R][M]^T * B[R][N]; the reduction over R is split over
 * frnnt_pair_matmul_tn_splits(M, N, R) work items per output tile, `partials` is scratch of
 * splits*M*N floats (may be NULL when splits == 1); partial sums are added in order. */
int frnnt_pair_matmul_tn_splits(int M, int N, long long R);
int frnnt_pair_matmul_tn(const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
                         const float *inv_scale_a, const float *inv_scale_b, float *d, float *partials,
                         int M, int N, long long R, long long pitch_a, long long pitch_b, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FRNNT_H_ */
