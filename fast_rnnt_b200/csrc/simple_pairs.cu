// The "simple" lattices (get_rnnt_logprobs / get_rnnt_logprobs_smoothed,
// fast_rnnt/python/fast_rnnt/rnnt_loss.py:66-227 and :1135-1369) on the fp16-pair
// tensor-core engine (umma_pairs.cuh), float32 path:
//
//   forward   one pass over lm and am takes the row maxima and writes
//             exp(x - rowmax) as fp16 planes (the operands of every product below; they
//             are kept for the backward) plus a few per-row scalars;
//             N^T[t][s] = sum_c A[t][c] L[s][c] per utterance on the tensor cores (TMA-fed),
//             whose epilogue takes the log, adds the maxima back, gathers am[t][symbol],
//             am[t][blank], applies the smoothing interpolation, the -inf at t_end and
//             px += py[s+1] (constrained) and writes the normalizer, px and py -- lane <->
//             frame, so every store is a coalesced row segment of the [s][t] lattices
//             (rnnt_loss.py:174-227, :1296-1367);
//   backward  the gradient weights Rw[s][t] (simple.cu) become planes, and
//             dlm[s][c] = -L[s][c] * sum_t Rw[s][t] A[t][c],
//             dam[t][c] = -A[t][c] * sum_s Rw[s][t] L[s][c]
//             run on the same engine, L and A read back from the planes in the epilogue.
#include <cuda_fp16.h>

#include "lsm_band.cuh"
#include "simple_pairs.cuh"
#include "umma_pairs.cuh"

namespace frnnt {

constexpr float kExpScale = 16384.f;             // exp(x - max) <= 1
constexpr float kExpInv2 = 1.f / (16384.f * 16384.f);
constexpr int kSpParts = 1024;

static inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

SimplePairsLayout::SimplePairsLayout(int B, int S, int T, int C) {
  const size_t S1 = (size_t)S + 1;
  Cp = (C + 63) / 64 * 64;
  Tq = (T + 63) / 64 * 64;
  Sp = (S + 31) / 32 * 32;
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t r = o;
    o += up256(bytes);
    return r;
  };
  lp_hi = take((size_t)B * S1 * Cp * 2);
  lp_lo = take((size_t)B * S1 * Cp * 2);
  ap_hi = take((size_t)B * T * Cp * 2);
  ap_lo = take((size_t)B * T * Cp * 2);
  lm_blk = take((size_t)B * S1 * 4);
  lm_sym = take((size_t)B * S1 * 4);
  lnorm = take((size_t)B * S1 * 4);
  am_blk = take((size_t)B * T * 4);
  am_sym = take((size_t)B * T * Sp * 4);
  saved_bytes = o;
  o = 0;
  rw_hi = take((size_t)B * S1 * Tq * 2);
  rw_lo = take((size_t)B * S1 * Tq * 2);
  parts = take(std::max<size_t>(kSpParts, (size_t)B * S1) * 4);
  inv_scale = take(64);
  scratch_bytes = o;
}

size_t simple_pairs_rowmax_offset(int B, int S, int T, int C) { return SimplePairsLayout(B, S, T, C).parts; }

bool simple_pairs_supported(const void *lm, const void *am, int S1, int T, int C, int rnnt_type) {
  if (C % 4 != 0 || C < 4 || S1 < 1 || T < 1) return false;
  if ((uintptr_t)lm % 16 != 0 || (uintptr_t)am % 16 != 0) return false;
  // px += py[s+1] is carried from column to column inside one tile of 128 lattice rows
  if (rnnt_type == FRNNT_CONSTRAINED && S1 > kPairTile) return false;
  return true;
}

// ---- forward, pass 1: row maxima, exp planes, per-row scalars -----------------------------------
// one warp per row of lm (rows 0 .. B*S1-1) or am (the rest); 16-byte loads
template <typename TIn>
__global__ void __launch_bounds__(256)
exp_planes_kernel(const TIn *__restrict__ lm, const TIn *__restrict__ am,
                  const int64_t *__restrict__ symbols, __half *__restrict__ lp_hi,
                  __half *__restrict__ lp_lo, __half *__restrict__ ap_hi, __half *__restrict__ ap_lo,
                  float *__restrict__ lmmax, float *__restrict__ lmsum, float *__restrict__ ammax,
                  float *__restrict__ lm_blk, float *__restrict__ lm_sym, float *__restrict__ lnorm,
                  float *__restrict__ am_blk, float *__restrict__ am_sym, float *__restrict__ px, int B,
                  int S, int T, int C, int Cp, int Sp, int blank, int regular) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int S1 = S + 1, nvec = C / 4;
  const long long rows_lm = (long long)B * S1, rows = rows_lm + (long long)B * T;
  for (long long row = warp0; row < rows; row += nwarps) {
    const bool is_lm = row < rows_lm;
    const long long r = is_lm ? row : row - rows_lm;
    const TIn *src = (is_lm ? lm : am) + r * C;
    uint2 *dh = reinterpret_cast<uint2 *>((is_lm ? lp_hi : ap_hi) + r * Cp);
    uint2 *dl = reinterpret_cast<uint2 *>((is_lm ? lp_lo : ap_lo) + r * Cp);
    // the first four vectors of a lane stay in registers (rows up to 512 entries are read once)
    float4 keep[4];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec) {
        keep[j] = in_load4(src, v);
        m = fmaxf(fmaxf(m, fmaxf(keep[j].x, keep[j].y)), fmaxf(keep[j].z, keep[j].w));
      }
    }
    for (int v = lane + 128; v < nvec; v += 32) {
      const float4 q = in_load4(src, v);
      m = fmaxf(fmaxf(m, fmaxf(q.x, q.y)), fmaxf(q.z, q.w));
    }
    m = warp_max(m);
    float sum = 0.f;
    auto one = [&](int v, const float4 &q) {
      const float e[4] = {expf(q.x - m), expf(q.y - m), expf(q.z - m), expf(q.w - m)};
#pragma unroll
      for (int i = 0; i < 4; ++i) sum += e[i];
      uint2 hi, lo;
      fp16_pair4(e, kExpScale, hi, lo);
      dh[v] = hi;
      dl[v] = lo;
    };
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = lane + 32 * j;
      if (v < nvec) one(v, keep[j]);
    }
    for (int v = lane + 128; v < nvec; v += 32) one(v, in_load4(src, v));
    sum = warp_sum(sum);
    if (!is_lm) {
      // am[t][symbol of every lattice row]: gathered here, where the row has just been read
      // (L1 hits), so that the product's epilogue reads them as whole 128-byte lines
      const TIn *x = am + r * C;
      const int64_t *sy = symbols + (size_t)div_rows(r, T) * S;
      float *dst = am_sym + (size_t)r * Sp;
      for (int s = lane; s < Sp; s += 32) {
        float v = 0.f;
        if (s < S) {
          long long y = sy[s];
          if (y < 0 || y >= C) y = blank;
          v = in_f32(x[y]);
        }
        dst[s] = v;
      }
    }
    if (lane == 0) {
      const TIn *x = (is_lm ? lm : am) + r * C;
      if (is_lm) {
        const int b = (int)div_rows(r, S1), s = mod_rows(r, S1);
        lmmax[r] = m;
        lmsum[r] = sum;
        lnorm[r] = logf(sum) + m;
        lm_blk[r] = in_f32(x[blank]);
        if (s < S) {
          long long y = symbols[(size_t)b * S + s];
          if (y < 0 || y >= C) y = blank;
          lm_sym[r] = in_f32(x[y]);
          // the -inf column of the regular type, which no frame owns
          if (regular) px[((size_t)b * S + s) * (T + 1) + T] = -INFINITY;
        }
      } else {
        ammax[r] = m;
        am_blk[r] = in_f32(x[blank]);
      }
    }
  }
}

// ---- forward, pass 2: the normalizer product and the lattices ----------------------------------
// tile rows = frames t, tile columns = lattice rows s
struct NormPairExt {
  static constexpr bool kBatched = true, kCustomStore = true;
  float *norm, *px, *py;
  const float *am_sym;  // [B][T][Sp]
  const int64_t *symbols, *boundary;
  const float *lmmax, *ammax, *lm_blk, *lm_sym, *lnorm, *am_blk, *amonly, *loguni;
  int S, T, C, blank, rnnt_type;
  int smoothed, am_only_off;
  float both, ls, as;
  int Sp;
  double delay_penalty;
  struct Row {
    float ammax_t, am_blk_t, amonly_t, py_next, pen;
    const float *amrow;
    long long t_end;
  };
  __device__ void row_begin(Row &r, int b, int t, int) const {
    const size_t bt = (size_t)b * T + t;
    r.ammax_t = ammax[bt];
    r.am_blk_t = am_blk[bt];
    r.amonly_t = (smoothed && !am_only_off) ? amonly[bt] : 0.f;
    r.amrow = am_sym + bt * Sp;
    r.t_end = (rnnt_type == FRNNT_REGULAR && boundary != nullptr) ? (long long)boundary[4 * b + 3] : -1;
    r.py_next = 0.f;
    r.pen = delay_penalty_at<float>(boundary, b, T, t, delay_penalty);
  }
  __device__ void prefetch(Row &, int, int, int) const {}
  __device__ void finish(Row &, int, int, int, float (&)[16], int) const {}
  __device__ void row_end(Row &, int, int, int) const {}
  // per-column data of a tile in the warp's 4 KB of shared memory: one 16-byte entry
  // (lmmax, lm[blank], lm[symbol], lm-only normalizer) and the symbol per lattice row
  struct Cols {
    float4 q[kPairTile];
    int sym[kPairTile];
  };
  __device__ void tile_begin(int b, int s0, uint8_t *box, int lane) const {
    Cols *c = reinterpret_cast<Cols *>(box);
    const int S1 = S + 1;
#pragma unroll
    for (int j = 0; j < kPairTile / 32; ++j) {
      const int i = lane + 32 * j, s = s0 + i;
      if (s < S1) {
        const size_t bs = (size_t)b * S1 + s;
        long long y = blank;
        float ls_ = 0.f;
        if (s < S) {
          ls_ = lm_sym[bs];
          y = symbols[(size_t)b * S + s];
          if (y < 0 || y >= C) y = blank;
        }
        c->q[i] = make_float4(lmmax[bs], lm_blk[bs], ls_, lnorm[bs]);
        c->sym[i] = (int)y;
      }
    }
  }
  // columns from the last to the first: px of row s needs py of row s + 1 (constrained).
  // The epilogue runs on one warp per scheduler, i.e. at the latency of its instructions:
  // it is written to be short (one 16-byte shared-memory load per cell, the log on the
  // special-function unit: |error| of lg2.approx is 2^-22, i.e. 1.6e-7 on the normalizer,
  // no more than the rounding of an exact float32 log of this magnitude).
  __device__ void store_box(Row &r, int b, int t, int s0, int c0, float (&v0)[16], float (&v1)[16],
                            const uint8_t *box) const {
    const Cols *c = reinterpret_cast<const Cols *>(box);
    const int S1 = S + 1, T1 = rnnt_type == FRNNT_REGULAR ? T + 1 : T;
    // am[t][symbol] of the box's lattice rows: one 128-byte line per frame
    float pxam[32];
    if (s0 + c0 < Sp) {
      const float4 *g = reinterpret_cast<const float4 *>(r.amrow + s0 + c0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 q = g[i];
        pxam[4 * i] = q.x, pxam[4 * i + 1] = q.y, pxam[4 * i + 2] = q.z, pxam[4 * i + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) pxam[i] = 0.f;
    }
    float *nrow = norm + ((size_t)b * S1 + s0 + c0 + 31) * T + t;
    float *yrow = py + ((size_t)b * S1 + s0 + c0 + 31) * T + t;
    float *xrow = px + ((size_t)b * S + s0 + c0 + 31) * T1 + t;
    const bool am_on = smoothed && !am_only_off;
    const float lu_blank = am_on ? loguni[blank] : 0.f;
    const float am_y = am_on ? (r.am_blk_t + lu_blank - r.amonly_t) * as : 0.f;
#pragma unroll
    for (int i = 31; i >= 0; --i, nrow -= T, yrow -= T, xrow -= T1) {
      const int s = s0 + c0 + i;
      if (s > S) continue;
      const float acc = i < 16 ? v0[i & 15] : v1[i & 15];
      const float4 q = c->q[c0 + i];
      const float nv = __logf(acc * kExpInv2 + 1.17549435e-38f) + q.x + r.ammax_t;
      *nrow = nv;
      float vy = r.am_blk_t + q.y - nv;
      if (smoothed) vy = vy * both + (q.y - q.w) * ls + am_y;
      *yrow = vy;
      if (s < S) {
        float v = pxam[i] + q.z - nv;
        if (smoothed) {
          v = v * both + (q.z - q.w) * ls;
          if (am_on) v += (pxam[i] + loguni[c->sym[c0 + i]] - r.amonly_t) * as;
        }
        if (rnnt_type == FRNNT_REGULAR) {
          if ((long long)t == r.t_end) v = -INFINITY;
        } else if (rnnt_type == FRNNT_CONSTRAINED) {
          v += r.py_next;
        }
        if (delay_penalty > 0.0) v = __fadd_rn(v, r.pen);
        *xrow = v;
      }
      r.py_next = vy;
    }
  }
};

// ---- backward products --------------------------------------------------------------------------
// what both epilogues share: the 32 plane values (exp(x - max) * 2^14) of the row's next box
struct PlaneRow {
  uint4 h[4], l[4];
  __device__ void load(const __half *hi, const __half *lo, size_t off) {
    const uint4 *ph = reinterpret_cast<const uint4 *>(hi + off);
    const uint4 *pl = reinterpret_cast<const uint4 *>(lo + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = ph[i], l[i] = pl[i];
  }
  __device__ void get(int half, float (&e)[16]) const {
    __align__(16) __half hh[16], ll[16];
    *reinterpret_cast<uint4 *>(hh) = h[2 * half];
    *reinterpret_cast<uint4 *>(hh + 8) = h[2 * half + 1];
    *reinterpret_cast<uint4 *>(ll) = l[2 * half];
    *reinterpret_cast<uint4 *>(ll + 8) = l[2 * half + 1];
#pragma unroll
    for (int i = 0; i < 16; ++i) e[i] = (__half2float(hh[i]) + __half2float(ll[i])) * (1.f / kExpScale);
  }
};

// dlm[s][c] = -L[s][c] * sum_t Rw[s][t] A[t][c]  (+ lm-only / unigram terms)
struct LmGradPairExt {
  static constexpr bool kBatched = true, kCustomStore = false;
  const __half *lp_hi, *lp_lo;
  const float *inv_rw, *lmsum, *gl, *dp, *rowdot;
  int S1, C, Cp;
  struct Row {
    float sc, inv_sum, g, rd;
    PlaneRow pl;
  };
  __device__ void row_begin(Row &r, int b, int s, int n0) const {
    const size_t row = (size_t)b * S1 + s;
    r.sc = *inv_rw * (1.f / kExpScale);
    r.inv_sum = gl != nullptr ? 1.f / lmsum[row] : 0.f;
    r.g = gl != nullptr ? gl[row] : 0.f;
    r.rd = (gl != nullptr && dp != nullptr) ? rowdot[row] : 0.f;
    (void)n0;
  }
  // the planes are padded to whole 64-entry blocks, so a box is always readable
  __device__ void prefetch(Row &r, int b, int s, int n) const {
    if (n < Cp) r.pl.load(lp_hi, lp_lo, ((size_t)b * S1 + s) * Cp + n);
  }
  __device__ void finish(Row &r, int, int, int c0, float (&v)[16], int half) const {
    float L[16];
    r.pl.get(half, L);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float o = -(L[i] * (v[i] * r.sc));
      if (gl != nullptr) {
        const float P = L[i] * r.inv_sum;
        o -= r.g * P;
        if (dp != nullptr && c0 + i < C) o += P * (dp[c0 + i] - r.rd);
      }
      v[i] = o;
    }
  }
  __device__ void row_end(Row &, int, int, int) const {}
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
};

// dam[t][c] = -A[t][c] * sum_s Rw[s][t] L[s][c]  (+ am-only term)
struct AmGradPairExt {
  static constexpr bool kBatched = true, kCustomStore = false;
  const __half *ap_hi, *ap_lo;
  const float *inv_rw, *ammax, *h, *uni, *amonly;
  int T, C, Cp;
  struct Row {
    float sc, w;
    PlaneRow pl;
  };
  __device__ void row_begin(Row &r, int b, int t, int) const {
    const size_t row = (size_t)b * T + t;
    r.sc = *inv_rw * (1.f / kExpScale);
    r.w = h != nullptr ? h[row] * expf(ammax[row] - amonly[row]) : 0.f;
  }
  __device__ void prefetch(Row &r, int b, int t, int n) const {
    if (n < Cp) r.pl.load(ap_hi, ap_lo, ((size_t)b * T + t) * Cp + n);
  }
  __device__ void finish(Row &r, int, int, int c0, float (&v)[16], int half) const {
    float A[16];
    r.pl.get(half, A);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float o = -(A[i] * (v[i] * r.sc));
      if (h != nullptr && c0 + i < C) o -= r.w * A[i] * uni[c0 + i];
      v[i] = o;
    }
  }
  __device__ void row_end(Row &, int, int, int) const {}
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
};

// Rw [rows][Tp] float -> planes [rows][Tq], columns Tp..Tq-1 zero (they are inside the
// tensor maps only as padding up to T, never beyond it, but the backward's second product
// reads rows as its reduction index and must not meet stale data)
__global__ void __launch_bounds__(256)
sp_split_kernel(const float *__restrict__ x, long long rows, int Tp, int Tq,
                const float *__restrict__ part, int nparts, __half *__restrict__ hi,
                __half *__restrict__ lo, float *__restrict__ inv_scale) {
  __shared__ float slot;
  if (threadIdx.x < 32) {
    float m = 0.f;
    for (int i = threadIdx.x; i < nparts; i += 32) m = fmaxf(m, part[i]);
    m = warp_max(m);
    if (threadIdx.x == 0) slot = m;
  }
  __syncthreads();
  const float scale = fp16_pair_scale(slot);
  if (blockIdx.x == 0 && threadIdx.x == 0) *inv_scale = 1.f / scale;
  const long long n = rows * Tq;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const long long r = i / Tq;
    const int c = (int)(i - r * Tq);
    __half h = __float2half_rn(0.f), l = h;
    if (c < Tp) fp16_pair(x[r * Tp + c], scale, h, l);
    hi[i] = h;
    lo[i] = l;
  }
}

int launch_simple_forward_pairs(const void *lm, const void *am, const int64_t *symbols,
                                const int64_t *boundary, int blank, int rnnt_type, int smoothed,
                                int am_only_off, float both, float ls, float as, float *px, float *py,
                                float *norm, float *lmmax, float *lmsum, float *ammax,
                                const float *amonly, const float *loguni, void *pairs_saved, int B, int S,
                                int T, int C, int stage, cudaStream_t st, double delay_penalty, int input_dtype) {
  const SimplePairsLayout L(B, S, T, C);
  uint8_t *sv = (uint8_t *)pairs_saved;
  __half *lp_hi = (__half *)(sv + L.lp_hi), *lp_lo = (__half *)(sv + L.lp_lo);
  __half *ap_hi = (__half *)(sv + L.ap_hi), *ap_lo = (__half *)(sv + L.ap_lo);
  float *lm_blk = (float *)(sv + L.lm_blk), *lm_sym = (float *)(sv + L.lm_sym);
  float *lnorm = (float *)(sv + L.lnorm), *am_blk = (float *)(sv + L.am_blk);
  float *am_sym = (float *)(sv + L.am_sym);
  const int S1 = S + 1;
  if (stage == 0) {
    const long long rows = (long long)B * (S1 + T);
    long long want = (rows + 7) / 8;
    const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
#define FRNNT_EXP_PLANES(TIn)                                                                                   \
  FRNNT_KERNEL(exp_planes_kernel<TIn><<<grid, 256, 0, st>>>((const TIn *)lm, (const TIn *)am, symbols, lp_hi, lp_lo,  \
                                                           ap_hi, ap_lo, lmmax, lmsum, ammax, lm_blk, lm_sym, lnorm, \
                                                           am_blk, am_sym, px, B, S, T, C, L.Cp, L.Sp, blank,        \
                                                           rnnt_type == FRNNT_REGULAR))
    if (input_dtype == FRNNT_F16) {
      FRNNT_EXP_PLANES(__half);
    } else if (input_dtype == FRNNT_BF16) {
      FRNNT_EXP_PLANES(__nv_bfloat16);
    } else {
      FRNNT_EXP_PLANES(float);
    }
#undef FRNNT_EXP_PLANES
    FRNNT_CUDA(cudaGetLastError());
    return FRNNT_OK;
  }
  CUtensorMap mah, mal, mbh, mbl;
  int rc = make_pair_map(&mah, ap_hi, T, C, L.Cp, false, B, (long long)T * L.Cp);
  if (rc == FRNNT_OK) rc = make_pair_map(&mal, ap_lo, T, C, L.Cp, false, B, (long long)T * L.Cp);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbh, lp_hi, S1, C, L.Cp, false, B, (long long)S1 * L.Cp);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbl, lp_lo, S1, C, L.Cp, false, B, (long long)S1 * L.Cp);
  if (rc != FRNNT_OK) return rc;
  const LinShape shape{T, S1, C, ((C + kPairBK - 1) / kPairBK) * kPairBK, (T + kPairTile - 1) / kPairTile,
                       (S1 + kPairTile - 1) / kPairTile, B};
  const NormPairExt ext{norm,   px,     py,     am_sym, symbols, boundary, lmmax,    ammax,       lm_blk, lm_sym,
                        lnorm,  am_blk, amonly, loguni, S,       T,        C,        blank,       rnnt_type,
                        smoothed, am_only_off, both, ls, as, L.Sp, delay_penalty};
  // the policy stores the lattices itself; the engine's output map is unused and is made
  // over the normalizer buffer only because it has to be a valid map
  return launch_pair_umma<false, false>(mah, mal, mbh, mbl, norm, shape, ext, st);
}

int launch_simple_grads_pairs(const float *rw, const float *lmsum, const float *ammax, const float *amonly,
                              const float *uni, const float *gl, const float *h, const float *dp,
                              const float *rowdot, float *lm_grad, float *am_grad, const void *pairs_saved,
                              void *pairs_scratch, int B, int S, int T, int C, int Tp, cudaStream_t st) {
  const SimplePairsLayout L(B, S, T, C);
  const uint8_t *sv = (const uint8_t *)pairs_saved;
  uint8_t *sc = (uint8_t *)pairs_scratch;
  const __half *lp_hi = (const __half *)(sv + L.lp_hi), *lp_lo = (const __half *)(sv + L.lp_lo);
  const __half *ap_hi = (const __half *)(sv + L.ap_hi), *ap_lo = (const __half *)(sv + L.ap_lo);
  __half *rw_hi = (__half *)(sc + L.rw_hi), *rw_lo = (__half *)(sc + L.rw_lo);
  float *parts = (float *)(sc + L.parts), *inv_rw = (float *)(sc + L.inv_scale);
  const int S1 = S + 1, Cp = L.Cp, Tq = L.Tq;
  const long long rows = (long long)B * S1;

  CUtensorMap a1h, a1l, b1h, b1l, a2h, a2l, b2h, b2l;
  int rc = make_pair_map(&a1h, rw_hi, S1, T, Tq, false, B, (long long)S1 * Tq);      // Rw [s][t], K = t
  if (rc == FRNNT_OK) rc = make_pair_map(&a1l, rw_lo, S1, T, Tq, false, B, (long long)S1 * Tq);
  if (rc == FRNNT_OK) rc = make_pair_map(&b1h, ap_hi, T, C, Cp, true, B, (long long)T * Cp);   // A [t][c], K = t rows
  if (rc == FRNNT_OK) rc = make_pair_map(&b1l, ap_lo, T, C, Cp, true, B, (long long)T * Cp);
  if (rc == FRNNT_OK) rc = make_pair_map(&a2h, rw_hi, S1, T, Tq, true, B, (long long)S1 * Tq);  // Rw^T: K = s rows
  if (rc == FRNNT_OK) rc = make_pair_map(&a2l, rw_lo, S1, T, Tq, true, B, (long long)S1 * Tq);
  if (rc == FRNNT_OK) rc = make_pair_map(&b2h, lp_hi, S1, C, Cp, true, B, (long long)S1 * Cp);  // L [s][c], K = s rows
  if (rc == FRNNT_OK) rc = make_pair_map(&b2l, lp_lo, S1, C, Cp, true, B, (long long)S1 * Cp);
  if (rc != FRNNT_OK) return rc;

  // the caller left max |rw| per row in `parts`
  const int nparts = (int)rows;
  const long long nq = rows * Tq;
  const int grid = (int)std::min<long long>((nq + 255) / 256, (long long)sm_count() * 16);
  FRNNT_KERNEL(sp_split_kernel<<<grid, 256, 0, st>>>(rw, rows, Tp, Tq, parts, nparts, rw_hi, rw_lo, inv_rw));
  FRNNT_CUDA(cudaGetLastError());

  const int ctiles = (C + kPairTile - 1) / kPairTile;
  {
    const LinShape shape{S1, C, T, ((T + kPairBK - 1) / kPairBK) * kPairBK, (S1 + kPairTile - 1) / kPairTile, ctiles, B};
    const LmGradPairExt ext{lp_hi, lp_lo, inv_rw, lmsum, gl, dp, rowdot, S1, C, Cp};
    rc = launch_pair_umma<false, true>(a1h, a1l, b1h, b1l, lm_grad, shape, ext, st);
    if (rc != FRNNT_OK) return rc;
  }
  {
    const LinShape shape{T, C, S1, ((S1 + kPairBK - 1) / kPairBK) * kPairBK, (T + kPairTile - 1) / kPairTile, ctiles, B};
    const AmGradPairExt ext{ap_hi, ap_lo, inv_rw, ammax, h, uni, amonly, T, C, Cp};
    rc = launch_pair_umma<true, true>(a2h, a2l, b2h, b2l, am_grad, shape, ext, st);
    if (rc != FRNNT_OK) return rc;
  }
  return FRNNT_OK;
}

}  // namespace frnnt
