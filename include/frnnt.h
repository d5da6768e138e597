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
 *   - symbols, boundaries and ranges are int64, as in the reference's API;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and
 *     nothing synchronises;
 *   - nothing allocates device memory: outputs and scratch are the caller's
 *     (scratch sizes come from the *_workspace_bytes functions);
 *   - re-entrant; no global state besides the thread-local error string.
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

/* Replaces the pybind function with_cuda()
 * (fast_rnnt/python/csrc/mutual_information.cu:69-75): always 1. */
int frnnt_with_cuda(void);

/* ----------------------------------------------------------------------------
 * Mutual-information recursion
 * ------------------------------------------------------------------------- */

/* Bytes of the `branch` scratch of the three functions below: for every lattice
 * cell the weight exp(p[s-1][t']+px[s-1][t']-p[s][t]) of its "x" predecessor,
 * stored by anti-diagonal so that the backward sweep reads it coalesced. */
size_t frnnt_mi_branch_bytes(int dtype, int B, int S, int T);

/* Forward recursion.  Replaces mutual_information_forward(px, py, boundary, p)
 * of the reference's extension module (fast_rnnt/python/csrc/mutual_information.cu:27-45,
 * MutualInformationCuda at fast_rnnt/csrc/mutual_information_cuda.cu:676-728).
 *   p      may be NULL when the caller does not need the lattice;
 *   branch may be NULL when no backward sweep will follow;
 *   ans    [B] receives p[b][s_end][t_end]. */
int frnnt_mi_forward(int dtype, const void *px, const void *py, const int64_t *boundary,
                     void *p, void *ans, void *branch, int B, int S, int T, int modified,
                     void *stream);

/* Reverse sweep from the `branch` weights written by frnnt_mi_forward:
 * px_grad [B][S][T1] and py_grad [B][S+1][T] are fully written (exact zeros
 * outside the boundary box).  origin_grad (may be NULL) receives the gradient
 * that reaches p[s_begin][t_begin], which equals ans_grad[b] up to rounding
 * when the sweep is right (the reference overwrites ans_grad with it,
 * mutual_information_cuda.cu:667-669). */
int frnnt_mi_backward_from_branch(int dtype, const void *branch, const int64_t *boundary,
                                  const void *ans_grad, void *px_grad, void *py_grad,
                                  void *origin_grad, int B, int S, int T, int modified,
                                  void *stream);

/* Reverse sweep from a lattice `p` in the reference's layout.  Replaces
 * mutual_information_backward(px, py, boundary, p, ans_grad)
 * (fast_rnnt/python/csrc/mutual_information.cu:47-67, MutualInformationBackwardCuda
 * at mutual_information_cuda.cu:734-805).  `branch` is scratch of
 * frnnt_mi_branch_bytes() bytes. */
int frnnt_mi_backward(int dtype, const void *px, const void *py, const int64_t *boundary,
                      const void *p, const void *ans_grad, void *px_grad, void *py_grad,
                      void *origin_grad, void *branch, int B, int S, int T, int modified,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FRNNT_H_ */
