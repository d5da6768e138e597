/*
 * TEST INFRASTRUCTURE ONLY -- the checker, never the product.
 *
 * Plain-C restatement of the reference's CPU mutual-information recursion
 * (k2-fsa/fast_rnnt).  Only tests, the smoke check and the CPU-baseline leg of
 * the benchmark may load this library; the product path is the CUDA library
 * and must fail when that is missing.
 *
 * Parity status: PINNED.  tests/test_oracle_pin.py compares this file
 * bit-for-bit with the reference's own compiled CPU extension
 * (oracle/_ref/_fast_rnnt.so, built by oracle/Makefile target "ref") on seeded
 * random lattices (both dtypes, both recursion types, random boundaries with
 * non-zero begins and empty sequences), and against the committed golden
 * vectors under tests/golden/ that were produced by the reference itself.
 *
 * What follows which reference lines:
 *   logadd_*            fast_rnnt/csrc/mutual_information.h:36-65
 *   mi_oracle_forward_* fast_rnnt/csrc/mutual_information_cpu.cu:50-124
 *   mi_oracle_backward_* fast_rnnt/csrc/mutual_information_cpu.cu:128-256
 *
 * Layouts (row-major, contiguous):
 *   px  [B][S][T1]   T1 = T+1 (regular) or T (modified)
 *   py  [B][S+1][T]
 *   p   [B][S+1][T+1]
 *   boundary [B][4] int64 = (s_begin, t_begin, s_end, t_end), or NULL = (0,0,S,T)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DEFINE_MI(SUFFIX, real, EXP, LOG1P)                                      \
                                                                                 \
  /* log(exp(x)+exp(y)); returns the larger one when the difference is not      \
     finite (mutual_information.h:45-46, :61-62). */                             \
  static real logadd_##SUFFIX(real x, real y) {                                  \
    real diff;                                                                   \
    if (x < y) {                                                                 \
      diff = x - y;                                                              \
      x = y;                                                                     \
    } else {                                                                     \
      diff = y - x;                                                              \
    }                                                                            \
    if (diff - diff != 0) return x;                                              \
    return x + LOG1P(EXP(diff));                                                 \
  }                                                                              \
                                                                                 \
  int mi_oracle_forward_##SUFFIX(const real *px, const real *py,                 \
                                 const int64_t *boundary, real *p, real *ans,    \
                                 int B, int S, int T, int modified) {            \
    const int T1 = modified ? T : T + 1;                                         \
    const int off = modified ? -1 : 0;                                           \
    for (int b = 0; b < B; ++b) {                                                \
      const real *X = px + (size_t)b * S * T1;                                   \
      const real *Y = py + (size_t)b * (S + 1) * T;                              \
      real *P = p + (size_t)b * (S + 1) * (T + 1);                               \
      int s0 = 0, t0 = 0, s1 = S, t1 = T;                                        \
      if (boundary) {                                                            \
        s0 = (int)boundary[4 * b + 0];                                           \
        t0 = (int)boundary[4 * b + 1];                                           \
        s1 = (int)boundary[4 * b + 2];                                           \
        t1 = (int)boundary[4 * b + 3];                                           \
      }                                                                          \
      P[(size_t)s0 * (T + 1) + t0] = 0;                                          \
      /* first column (cpu.cu:94-102) */                                         \
      for (int s = s0 + 1; s <= s1; ++s) {                                       \
        if (modified)                                                            \
          P[(size_t)s * (T + 1) + t0] = -(real)INFINITY;                         \
        else                                                                     \
          P[(size_t)s * (T + 1) + t0] =                                          \
              P[(size_t)(s - 1) * (T + 1) + t0] + X[(size_t)(s - 1) * T1 + t0];  \
      }                                                                          \
      /* first row (cpu.cu:103-105) */                                           \
      for (int t = t0 + 1; t <= t1; ++t)                                         \
        P[(size_t)s0 * (T + 1) + t] =                                            \
            P[(size_t)s0 * (T + 1) + t - 1] + Y[(size_t)s0 * T + t - 1];         \
      /* interior (cpu.cu:106-119) */                                            \
      for (int s = s0 + 1; s <= s1; ++s) {                                       \
        real left = P[(size_t)s * (T + 1) + t0];                                 \
        for (int t = t0 + 1; t <= t1; ++t) {                                     \
          real up = P[(size_t)(s - 1) * (T + 1) + t + off] +                     \
                    X[(size_t)(s - 1) * T1 + t + off];                           \
          left = logadd_##SUFFIX(up, left + Y[(size_t)s * T + t - 1]);           \
          P[(size_t)s * (T + 1) + t] = left;                                     \
        }                                                                        \
      }                                                                          \
      ans[b] = P[(size_t)s1 * (T + 1) + t1];                                     \
    }                                                                            \
    return 0;                                                                    \
  }                                                                              \
                                                                                 \
  /* px_grad [B][S][T1] and py_grad [B][S+1][T] are fully written (zeros         \
     outside the boundary box, cpu.cu:161-166). */                               \
  int mi_oracle_backward_##SUFFIX(const real *px, const real *py,                \
                                  const int64_t *boundary, const real *p,        \
                                  const real *ans_grad, real *px_grad,           \
                                  real *py_grad, int B, int S, int T,            \
                                  int modified) {                                \
    (void)py;                                                                    \
    const int T1 = modified ? T : T + 1;                                         \
    const int off = modified ? -1 : 0;                                           \
    const size_t np = (size_t)(S + 1) * (T + 1);                                 \
    real *G = (real *)malloc(np * sizeof(real));                                 \
    if (!G) return -1;                                                           \
    memset(px_grad, 0, (size_t)B * S * T1 * sizeof(real));                       \
    memset(py_grad, 0, (size_t)B * (S + 1) * T * sizeof(real));                  \
    for (int b = 0; b < B; ++b) {                                                \
      const real *X = px + (size_t)b * S * T1;                                   \
      const real *P = p + (size_t)b * np;                                        \
      real *GX = px_grad + (size_t)b * S * T1;                                   \
      real *GY = py_grad + (size_t)b * (S + 1) * T;                              \
      int s0 = 0, t0 = 0, s1 = S, t1 = T;                                        \
      if (boundary) {                                                            \
        s0 = (int)boundary[4 * b + 0];                                           \
        t0 = (int)boundary[4 * b + 1];                                           \
        s1 = (int)boundary[4 * b + 2];                                           \
        t1 = (int)boundary[4 * b + 3];                                           \
      }                                                                          \
      memset(G, 0, np * sizeof(real));                                           \
      G[(size_t)s1 * (T + 1) + t1] = ans_grad[b];                                \
      /* interior, reverse order (cpu.cu:188-218) */                             \
      for (int s = s1; s > s0; --s) {                                            \
        for (int t = t1; t > t0; --t) {                                          \
          real term1 = P[(size_t)(s - 1) * (T + 1) + t + off] +                  \
                       X[(size_t)(s - 1) * T1 + t + off];                        \
          real total = P[(size_t)s * (T + 1) + t];                               \
          if (total - total != 0) total = 0;                                     \
          real d1 = EXP(term1 - total);                                          \
          real d2 = (real)(1.0 - d1);                                            \
          real g = G[(size_t)s * (T + 1) + t];                                   \
          real g1, g2;                                                           \
          if (d1 - d1 == 0.0) {                                                  \
            g1 = d1 * g;                                                         \
            g2 = d2 * g;                                                         \
          } else {                                                               \
            g1 = g2 = 0;                                                         \
          }                                                                      \
          GX[(size_t)(s - 1) * T1 + t + off] = g1;                               \
          G[(size_t)(s - 1) * (T + 1) + t + off] = g1;                           \
          GY[(size_t)s * T + t - 1] = g2;                                        \
          G[(size_t)s * (T + 1) + t - 1] += g2;                                  \
        }                                                                        \
      }                                                                          \
      /* first row (cpu.cu:219-226) */                                           \
      for (int t = t1; t > t0; --t) {                                            \
        real g = G[(size_t)s0 * (T + 1) + t];                                    \
        G[(size_t)s0 * (T + 1) + t - 1] += g;                                    \
        GY[(size_t)s0 * T + t - 1] = g;                                          \
      }                                                                          \
      /* first column, regular recursion only (cpu.cu:227-236) */                \
      if (!modified) {                                                           \
        for (int s = s1; s > s0; --s) {                                          \
          real g = G[(size_t)s * (T + 1) + t0];                                  \
          G[(size_t)(s - 1) * (T + 1) + t0] += g;                                \
          GX[(size_t)(s - 1) * T1 + t0] = g;                                     \
        }                                                                        \
      }                                                                          \
    }                                                                            \
    free(G);                                                                     \
    return 0;                                                                    \
  }

DEFINE_MI(f32, float, expf, log1pf)
DEFINE_MI(f64, double, exp, log1p)
