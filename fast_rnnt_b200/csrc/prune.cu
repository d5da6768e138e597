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
#include <climits>

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

// Stage 1: kArgParts threads per frame, each scanning a contiguous share of the window
// positions (lane <-> frame, so the loads of a warp are contiguous; warp <-> share);
// the shares are combined in ascending order with a strict comparison, which keeps
// the FIRST maximum exactly as a single scan would.  s_begin[b][t] is parked in
// ranges[b][t][0] for stage 2.  RT > 0: the window width is a compile-time constant
// and the window lives in registers.
constexpr int kArgParts = 8;

template <typename real, int RT>
__global__ void __launch_bounds__(32 * kArgParts)
prune_argmax_kernel(const real *__restrict__ px_grad, const real *__restrict__ py_grad,
                    const int64_t *__restrict__ boundary, int64_t *__restrict__ ranges, int S,
                    int T, int T1, int Rdyn) {
  __shared__ real part_best[kArgParts][32];
  __shared__ int part_s[kArgParts][32];
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int t = blockIdx.x * 32 + lane;
  const int R = RT > 0 ? RT : Rdyn;
  const int S1 = S + 1;
  const int n_win = S1 - R + 1;
  const long long Sb = boundary[4 * b + 2], Tb = boundary[4 * b + 3];
  const bool scan = t < T && (long long)t < Tb - 1;
  const int per = (n_win + kArgParts - 1) / kArgParts;
  const int s_lo = part * per, s_hi = min(n_win, s_lo + per);
  int best_s = -1;
  real best = 0;
  if (scan && s_lo < s_hi) {
    const real *GX = px_grad + (size_t)b * S * T1 + t;
    const real *GY = py_grad + (size_t)b * S1 * T + t;
    if (RT > 0) {
      real w[RT > 0 ? RT : 1];
#pragma unroll
      for (int k = 0; k < RT; ++k) w[k] = GY[(size_t)(s_lo + k) * T];
      for (int s = s_lo; s < s_hi; ++s) {
        real acc = w[0];
#pragma unroll
        for (int k = 1; k < RT; ++k) acc = acc + w[k];
        const real score = acc - (s == 0 ? (real)0 : GX[(size_t)(s - 1) * T1]);
        if (s == s_lo || score > best) {
          best = score;
          best_s = s;
        }
#pragma unroll
        for (int k = 0; k + 1 < RT; ++k) w[k] = w[k + 1];
        if (s + RT < S1) w[RT - 1] = GY[(size_t)(s + RT) * T];
      }
    } else {
      for (int s = s_lo; s < s_hi; ++s) {
        real acc = GY[(size_t)s * T];
        for (int k = 1; k < R; ++k) acc = acc + GY[(size_t)(s + k) * T];
        const real score = acc - (s == 0 ? (real)0 : GX[(size_t)(s - 1) * T1]);
        if (s == s_lo || score > best) {
          best = score;
          best_s = s;
        }
      }
    }
  }
  part_best[part][lane] = best;
  part_s[part][lane] = best_s;
  __syncthreads();
  if (part != 0 || t >= T) return;
  int out_s;
  if (scan) {
    out_s = part_s[0][lane];
    real top = part_best[0][lane];
    for (int q = 1; q < kArgParts; ++q) {
      if (part_s[q][lane] >= 0 && part_best[q][lane] > top) {
        top = part_best[q][lane];
        out_s = part_s[q][lane];
      }
    }
  } else {
    long long pad = Sb - R + 1;
    if (pad < 0) pad = 0;
    if (pad > n_win - 1) pad = n_win - 1;  // keeps ranges inside [0, S] for malformed rows
    out_s = (int)pad;
  }
  ranges[((size_t)b * T + t) * R] = out_s;
}

// Stage 2: one CTA per utterance: monotone fix-up (integer scans) and expansion.
__global__ void __launch_bounds__(kPruneThreads)
prune_fixup_kernel(int64_t *__restrict__ ranges, int T, int T1, int R) {
  extern __shared__ int sm[];
  int *arr = sm;        // [T]
  int *part = sm + T;   // [kPruneThreads]
  const int b = blockIdx.x;
  int64_t *out = ranges + (size_t)b * T * R;
  for (int t = threadIdx.x; t < T; t += kPruneThreads) arr[t] = (int)out[(size_t)t * R];
  __syncthreads();
  // _adjust_pruning_lower_bound with window 2 (modified shapes) or R (regular)
  const int step = (T1 == T ? 2 : R) - 1;
  block_suffix_min(arr, T, part);
  for (int t = threadIdx.x; t < T; t += kPruneThreads) arr[t] = step * t - arr[t];
  __syncthreads();
  block_suffix_min(arr, T, part);
  for (int t = threadIdx.x; t < T; t += kPruneThreads) arr[t] = step * t - max(arr[t], 0);
  __syncthreads();
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
    const long long b = div_rows(row, TR);
    long long s = ranges[row];
    s = s < 0 ? 0 : (s >= S1 ? S1 - 1 : s);  // never read outside lm
    const vec *src = lm + ((size_t)b * S1 + s) * dvec;
    vec *dst = out + (size_t)row * dvec;
    for (int v = lane; v < dvec; v += 32) dst[v] = src[v];
  }
}

// lm_grad[b][s][:] = sum over (t,k) with ranges[b][t][k] == s of g[b][t][k][:]
// One CTA (4 warps) per (b, s).  Step 1: the warps scan the utterance's T*R
// range entries (a quarter each, 32 entries per ballot) and list the matching
// entries in shared memory, in entry order.  Step 2: every warp walks the whole
// list for its share of the D columns, eight gradient rows in flight at a time,
// adding them in list order.  Deterministic, no atomics, any ranges (not only
// the monotone ones get_rnnt_prune_ranges produces).
constexpr int kGbThreads = 128;
constexpr int kGbSegment = 8192;  // range entries listed per pass

template <typename real, typename vec, int VW>
__global__ void __launch_bounds__(kGbThreads)
prune_gather_backward_kernel(const real *__restrict__ g, const int64_t *__restrict__ ranges,
                             real *__restrict__ lm_grad, int TR, int S1, int D) {
  constexpr int NW = kGbThreads / 32;
  constexpr int kBatch = 8;
  __shared__ int list[NW][kGbSegment / NW];
  __shared__ int count[NW];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, s = blockIdx.x;
  const int64_t *rg = ranges + (size_t)b * TR;
  const real *G = g + (size_t)b * TR * D;
  const int dvec = D / VW;
  vec *out = reinterpret_cast<vec *>(lm_grad + ((size_t)b * S1 + s) * D);

  for (int v0 = 0; v0 < dvec; v0 += kGbThreads) {
    const int v = v0 + threadIdx.x;
    real acc[VW];
#pragma unroll
    for (int c = 0; c < VW; ++c) acc[c] = 0;
    for (int seg = 0; seg < TR; seg += kGbSegment) {
      const int seg_n = min(kGbSegment, TR - seg);
      const int per = ((seg_n + NW * 32 - 1) / (NW * 32)) * 32;  // entries per warp, multiple of 32
      __syncthreads();
      int n = 0;
      for (int base = warp * per; base < min(seg_n, (warp + 1) * per); base += 32) {
        const int e = base + lane;
        const bool hit = e < seg_n && (long long)rg[seg + e] == (long long)s;
        const unsigned mask = __ballot_sync(0xffffffffu, hit);
        if (hit) list[warp][n + __popc(mask & ((1u << lane) - 1))] = seg + e;
        n += __popc(mask);
      }
      if (lane == 0) count[warp] = n;
      __syncthreads();
      if (v < dvec) {
        for (int w = 0; w < NW; ++w) {
          const int cnt = count[w];
          for (int i0 = 0; i0 < cnt; i0 += kBatch) {
            vec x[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              if (i0 + u < cnt)
                x[u] = reinterpret_cast<const vec *>(G + (size_t)list[w][i0 + u] * D)[v];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              if (i0 + u < cnt) {
                const real *xe = reinterpret_cast<const real *>(&x[u]);
#pragma unroll
                for (int c = 0; c < VW; ++c) acc[c] += xe[c];
              }
          }
        }
      }
    }
    if (v < dvec) {
      vec o;
      real *oe = reinterpret_cast<real *>(&o);
#pragma unroll
      for (int c = 0; c < VW; ++c) oe[c] = acc[c];
      out[v] = o;
    }
  }
}

// act[b][t][k][:] = tanh(enc[b][t][:] + dec[b][ranges[b][t][k]][:]): the joiner's input
// without materialising am_pruned / lm_pruned (one warp per output row)
template <typename real, typename vec, int VW>
__global__ void pruned_tanh_kernel(const real *__restrict__ enc, const real *__restrict__ dec,
                                   const int64_t *__restrict__ ranges, real *__restrict__ act,
                                   long long rows, int R, int TR, int S1, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int dvec = D / VW;
  for (long long row = warp0; row < rows; row += nwarps) {
    const long long b = div_rows(row, TR), bt = div_rows(row, R);
    long long s = ranges[row];
    s = s < 0 ? 0 : (s >= S1 ? S1 - 1 : s);
    const vec *e = reinterpret_cast<const vec *>(enc + (size_t)bt * D);
    const vec *d = reinterpret_cast<const vec *>(dec + ((size_t)b * S1 + s) * D);
    vec *o = reinterpret_cast<vec *>(act + (size_t)row * D);
    for (int v = lane; v < dvec; v += 32) {
      const vec x = e[v], y = d[v];
      vec r;
      const real *xe = reinterpret_cast<const real *>(&x), *ye = reinterpret_cast<const real *>(&y);
      real *re = reinterpret_cast<real *>(&r);
#pragma unroll
      for (int c = 0; c < VW; ++c) re[c] = tanh(xe[c] + ye[c]);
      o[v] = r;
    }
  }
}

// enc_grad[b][t][:] = sum_k gz[b][t][k][:]  (one warp per frame, k in order)
template <typename real, typename vec, int VW>
__global__ void sum_over_range_kernel(const real *__restrict__ gz, real *__restrict__ out,
                                      long long frames, int R, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int dvec = D / VW;
  for (long long f = warp0; f < frames; f += nwarps) {
    const vec *src = reinterpret_cast<const vec *>(gz + (size_t)f * R * D);
    vec *dst = reinterpret_cast<vec *>(out + (size_t)f * D);
    for (int v = lane; v < dvec; v += 32) {
      real acc[VW];
#pragma unroll
      for (int c = 0; c < VW; ++c) acc[c] = 0;
      for (int k = 0; k < R; ++k) {
        const vec x = src[(size_t)k * dvec + v];
        const real *xe = reinterpret_cast<const real *>(&x);
#pragma unroll
        for (int c = 0; c < VW; ++c) acc[c] += xe[c];
      }
      vec r;
      real *re = reinterpret_cast<real *>(&r);
#pragma unroll
      for (int c = 0; c < VW; ++c) re[c] = acc[c];
      dst[v] = r;
    }
  }
}

// ---- both input gradients of the pruned joiner from ONE pass over gz -----------------------
// enc_grad[b][t][:] = sum_k gz[b][t][k][:]
// dec_grad[b][s][:] = sum over (t,k) with ranges[b][t][k] == s of gz[b][t][k][:]
// One CTA per (utterance, chunk of kJgFrames frames); thread <-> 4 columns of D.  The
// rows of a chunk land on a few neighbouring s (get_rnnt_prune_ranges moves the window
// by less than one row per frame), so the CTA keeps a window of kJgWindow rows of partial
// sums in shared memory, each thread adding into its own columns in (t, k) order, and
// writes the used rows to a scratch; joiner_dec_reduce_kernel then adds the chunks'
// partial rows per (b, s) in chunk order.  Rows that fall outside the window (possible
// only for ranges that are not the monotone ones this library produces) go to dec_grad
// with atomicAdd, which is why dec_grad is cleared first.
constexpr int kJgFrames = 16;
constexpr int kJgWindow = 16;
constexpr int kJgThreads = 128;

template <bool WITH_ENC>
__global__ void __launch_bounds__(kJgThreads)
joiner_input_grads_kernel(const float *__restrict__ gz, const int64_t *__restrict__ ranges,
                          float *__restrict__ enc_grad, float *__restrict__ dec_grad,
                          float *__restrict__ partial, int *__restrict__ window, int T, int R, int S1,
                          int D) {
  extern __shared__ float4 jg_smem[];  // [kJgWindow][D / 4]
  __shared__ int s_lo_sh, s_hi_sh;
  const int b = blockIdx.y, ch = blockIdx.x, nch = gridDim.x;
  const int t0 = ch * kJgFrames, t1 = min(T, t0 + kJgFrames);
  const int dvec = D / 4;
  const int64_t *rg = ranges + ((size_t)b * T + t0) * R;
  const int n_entries = (t1 - t0) * R;
  if (threadIdx.x == 0) {
    s_lo_sh = INT_MAX;
    s_hi_sh = -1;
  }
  __syncthreads();
  {
    int lo = INT_MAX, hi = -1;
    for (int e = threadIdx.x; e < n_entries; e += kJgThreads) {
      const long long s = rg[e];
      if (s >= 0 && s < S1) {
        lo = min(lo, (int)s);
        hi = max(hi, (int)s);
      }
    }
    if (hi >= 0) {
      atomicMin(&s_lo_sh, lo);
      atomicMax(&s_hi_sh, hi);
    }
  }
  for (int i = threadIdx.x; i < kJgWindow * dvec; i += kJgThreads) jg_smem[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  const int s_lo = s_lo_sh, s_hi = s_hi_sh;
  const int rows_used = s_hi >= 0 ? min(kJgWindow, s_hi - s_lo + 1) : 0;
  if (threadIdx.x == 0) {
    window[((size_t)b * nch + ch) * 2] = s_lo;
    window[((size_t)b * nch + ch) * 2 + 1] = rows_used;
  }
  const float4 *G = reinterpret_cast<const float4 *>(gz) + ((size_t)b * T + t0) * R * dvec;
  float4 *E = WITH_ENC ? reinterpret_cast<float4 *>(enc_grad) + ((size_t)b * T + t0) * dvec : nullptr;
  // this thread's columns of one gradient row: into the frame sum and the window row
  auto consume = [&](const float4 &x, int entry, int v, float4 &e) {
    e.x += x.x, e.y += x.y, e.z += x.z, e.w += x.w;
    const long long s = rg[entry];
    if (s < 0 || s >= S1) return;
    const int sl = (int)s - s_lo;
    if (sl < kJgWindow) {
      float4 a = jg_smem[sl * dvec + v];
      a.x += x.x, a.y += x.y, a.z += x.z, a.w += x.w;
      jg_smem[sl * dvec + v] = a;
    } else {
      float *dst = dec_grad + ((size_t)b * S1 + s) * D + 4 * v;
      atomicAdd(dst, x.x), atomicAdd(dst + 1, x.y);
      atomicAdd(dst + 2, x.z), atomicAdd(dst + 3, x.w);
    }
  };
  for (int v = threadIdx.x; v < dvec; v += kJgThreads) {
    const int nt = t1 - t0;
    if (R <= 8) {
      // two frames per round: up to 16 independent row loads in flight per thread
      for (int t = 0; t < nt; t += 2) {
        float4 x[2][8];
        const bool two = t + 1 < nt;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (u < R) {
            x[0][u] = G[((size_t)t * R + u) * dvec + v];
            if (two) x[1][u] = G[((size_t)(t + 1) * R + u) * dvec + v];
          }
        }
#pragma unroll
        for (int f = 0; f < 2; ++f) {
          if (f == 1 && !two) break;
          float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (u < R) consume(x[f][u], (t + f) * R + u, v, e);
          if (WITH_ENC) E[(size_t)(t + f) * dvec + v] = e;
        }
      }
    } else {
      for (int t = 0; t < nt; ++t) {
        float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k0 = 0; k0 < R; k0 += 8) {
          float4 x[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (k0 + u < R) x[u] = G[((size_t)t * R + k0 + u) * dvec + v];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (k0 + u < R) consume(x[u], t * R + k0 + u, v, e);
        }
        if (WITH_ENC) E[(size_t)t * dvec + v] = e;
      }
    }
    float4 *P = reinterpret_cast<float4 *>(partial) + ((size_t)b * nch + ch) * kJgWindow * dvec;
    for (int r = 0; r < rows_used; ++r) P[(size_t)r * dvec + v] = jg_smem[r * dvec + v];
  }
}

// The same pass with the window in REGISTERS instead of shared memory, for ranges whose R rows
// per frame are consecutive and whose first row never moves back (what get_rnnt_prune_ranges
// writes): acc[i] holds the partial sum of lattice row base + i; when the frame's first row has
// moved on, the rows left behind are complete for this chunk and leave for the scratch (or,
// beyond kJgWindow rows per chunk, for dec_grad by atomicAdd, as in the kernel above).  No
// shared-memory traffic for the window, no barrier per chunk: 0.116 -> 0.096 ms at B=64, T=500,
// R=5, D=512.  A chunk whose ranges are not of that form adds every row to dec_grad with
// atomicAdd.
template <bool WITH_ENC, int R>
__global__ void __maxnreg__(88)
joiner_input_grads_ring_kernel(const float *__restrict__ gz, const int64_t *__restrict__ ranges,
                               float *__restrict__ enc_grad, float *__restrict__ dec_grad,
                               float *__restrict__ partial, int *__restrict__ window, int T, int S1, int D) {
  __shared__ int s0_sh[kJgFrames];
  const int b = blockIdx.y, ch = blockIdx.x, nch = gridDim.x;
  const int t0 = ch * kJgFrames, t1 = min(T, t0 + kJgFrames), nt = t1 - t0;
  const int dvec = D / 4;
  const int64_t *rg = ranges + ((size_t)b * T + t0) * R;
  // is this chunk of the regular form?  (one entry per thread; nt * R <= 128)
  bool ok = true;
  for (int e = threadIdx.x; e < nt * R; e += kJgThreads) {
    const int t = e / R, k = e - t * R;
    const long long first = rg[(size_t)t * R], s = rg[e];
    ok = ok && s == first + k && first >= 0 && first + R <= S1;
    if (k == 0) {
      s0_sh[t] = (int)first;
      if (t > 0) {
        const long long step = first - rg[(size_t)(t - 1) * R];
        ok = ok && step >= 0 && step <= kJgWindow;
      }
    }
  }
  const bool regular = __syncthreads_and(ok);
  const int s_lo = regular ? s0_sh[0] : 0;
  if (threadIdx.x == 0) {
    window[((size_t)b * nch + ch) * 2] = s_lo;
    window[((size_t)b * nch + ch) * 2 + 1] = regular ? min(kJgWindow, s0_sh[nt - 1] + R - s_lo) : 0;
  }
  const float4 *G = reinterpret_cast<const float4 *>(gz) + ((size_t)b * T + t0) * R * dvec;
  float4 *E = WITH_ENC ? reinterpret_cast<float4 *>(enc_grad) + ((size_t)b * T + t0) * dvec : nullptr;
  float4 *P = reinterpret_cast<float4 *>(partial) + ((size_t)b * nch + ch) * kJgWindow * dvec;
  auto add4 = [](float4 &a, const float4 &x) { a.x += x.x, a.y += x.y, a.z += x.z, a.w += x.w; };
  auto to_dec = [&](long long s, int v, const float4 &x) {
    if (s < 0 || s >= S1) return;
    float *dst = dec_grad + ((size_t)b * S1 + s) * D + 4 * v;
    atomicAdd(dst, x.x), atomicAdd(dst + 1, x.y), atomicAdd(dst + 2, x.z), atomicAdd(dst + 3, x.w);
  };
  for (int v = threadIdx.x; v < dvec; v += kJgThreads) {
    if (!regular) {
      for (int t = 0; t < nt; ++t) {
        float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < R; ++k) {
          const float4 x = G[((size_t)t * R + k) * dvec + v];
          add4(e, x);
          to_dec(rg[(size_t)t * R + k], v, x);
        }
        if (WITH_ENC) E[(size_t)t * dvec + v] = e;
      }
      continue;
    }
    float4 acc[R];
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    int base = s_lo;  // lattice row of acc[0]
    // the row that leaves the ring: complete for this chunk
    auto retire = [&](const float4 &a) {
      const int sl = base - s_lo;
      if (sl < kJgWindow) P[(size_t)sl * dvec + v] = a;
      else to_dec(base, v, a);
      ++base;
    };
    constexpr int F = R <= 5 ? 2 : 1;  // frames per round: their F * R row loads are in flight together
    for (int t = 0; t < nt; t += F) {
      const bool two = F == 2 && t + 1 < nt;
      float4 x[F][R];
#pragma unroll
      for (int k = 0; k < R; ++k) {
        x[0][k] = G[((size_t)t * R + k) * dvec + v];
        if (F == 2 && two) x[F - 1][k] = G[((size_t)(t + 1) * R + k) * dvec + v];
      }
#pragma unroll
      for (int f = 0; f < F; ++f) {
        if (f == 1 && !two) break;
        for (int d = s0_sh[t + f] - base; d > 0; --d) {  // the same for the whole CTA
          retire(acc[0]);
#pragma unroll
          for (int i = 0; i + 1 < R; ++i) acc[i] = acc[i + 1];
          acc[R - 1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < R; ++k) {
          add4(e, x[f][k]);
          add4(acc[k], x[f][k]);
        }
        if (WITH_ENC) E[(size_t)(t + f) * dvec + v] = e;
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) retire(acc[i]);
  }
}

// dec_grad[b][s][:] += the chunks' partial rows for s, in chunk order.  Each warp first finds
// the chunks whose window holds s (lane <-> chunk, one ballot per 32 chunks), then fetches their
// rows four at a time, so that the loads of a round are in flight together.
__global__ void __launch_bounds__(kJgThreads)
joiner_dec_reduce_kernel(const float *__restrict__ partial, const int *__restrict__ window,
                         float *__restrict__ dec_grad, int nch, int S1, int D) {
  const int b = blockIdx.y, s = blockIdx.x;
  const int dvec = D / 4, lane = threadIdx.x & 31;
  const int *win = window + (size_t)b * nch * 2;
  const float4 *P = reinterpret_cast<const float4 *>(partial) + (size_t)b * nch * kJgWindow * dvec;
  float4 *out = reinterpret_cast<float4 *>(dec_grad) + ((size_t)b * S1 + s) * dvec;
  // whole warps walk the columns together (the ballots and shuffles below need all lanes)
  for (int v0 = (threadIdx.x & ~31); v0 < dvec; v0 += kJgThreads) {
    const int v = v0 + lane;
    const bool col = v < dvec;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < nch; base += 32) {
      const int ch = base + lane;
      const int lo = ch < nch ? win[2 * ch] : 0, n = ch < nch ? win[2 * ch + 1] : 0;
      unsigned mask = __ballot_sync(0xffffffffu, s >= lo && s < lo + n);
      while (mask) {
        float4 x[4];
        int cnt = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (mask) {
            const int bit = __ffs(mask) - 1;
            mask &= mask - 1;
            const int row = s - __shfl_sync(0xffffffffu, lo, bit);
            if (col) x[u] = P[((size_t)(base + bit) * kJgWindow + row) * dvec + v];
            cnt = u + 1;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (u < cnt && col) acc.x += x[u].x, acc.y += x[u].y, acc.z += x[u].z, acc.w += x[u].w;
      }
    }
    if (col) {
      float4 o = out[v];
      o.x += acc.x, o.y += acc.y, o.z += acc.z, o.w += acc.w;
      out[v] = o;
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
  FRNNT_REQUIRE(B <= 65535, FRNNT_EUNSUPPORTED, "B too large for the grid");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid1((unsigned)((T + 31) / 32), (unsigned)B);
#define PRUNE_ARGMAX(real, RT)                                                                  \
  FRNNT_KERNEL(prune_argmax_kernel<real, RT><<<grid1, 32 * kArgParts, 0, st>>>(                            \
      (const real *)px_grad, (const real *)py_grad, boundary, ranges, S, T, T1, s_range))
#define PRUNE_ARGMAX_R(real)                                   \
  switch (s_range) {                                           \
    case 2: PRUNE_ARGMAX(real, 2); break;                      \
    case 3: PRUNE_ARGMAX(real, 3); break;                      \
    case 4: PRUNE_ARGMAX(real, 4); break;                      \
    case 5: PRUNE_ARGMAX(real, 5); break;                      \
    case 6: PRUNE_ARGMAX(real, 6); break;                      \
    case 7: PRUNE_ARGMAX(real, 7); break;                      \
    case 8: PRUNE_ARGMAX(real, 8); break;                      \
    default: PRUNE_ARGMAX(real, 0); break;                     \
  }
  if (dtype == FRNNT_F32) {
    PRUNE_ARGMAX_R(float)
  } else {
    PRUNE_ARGMAX_R(double)
  }
#undef PRUNE_ARGMAX_R
#undef PRUNE_ARGMAX
  FRNNT_CUDA(cudaGetLastError());
  if (smem > 48 * 1024)
    FRNNT_CUDA(cudaFuncSetAttribute(prune_fixup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)smem));
  FRNNT_KERNEL(prune_fixup_kernel<<<B, kPruneThreads, smem, st>>>(ranges, T, T1, s_range));
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
  const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
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
  const bool vec_ok = (uintptr_t)out_grad % 16 == 0 && (uintptr_t)lm_grad % 16 == 0;
  if (dtype == FRNNT_F32) {
    if (vec_ok && D % 4 == 0)
      FRNNT_KERNEL(prune_gather_backward_kernel<float, float4, 4><<<grid, kGbThreads, 0, st>>>(
          (const float *)out_grad, ranges, (float *)lm_grad, T * R, S1, D));
    else
      FRNNT_KERNEL(prune_gather_backward_kernel<float, float, 1><<<grid, kGbThreads, 0, st>>>(
          (const float *)out_grad, ranges, (float *)lm_grad, T * R, S1, D));
  } else {
    if (vec_ok && D % 2 == 0)
      FRNNT_KERNEL(prune_gather_backward_kernel<double, double2, 2><<<grid, kGbThreads, 0, st>>>(
          (const double *)out_grad, ranges, (double *)lm_grad, T * R, S1, D));
    else
      FRNNT_KERNEL(prune_gather_backward_kernel<double, double, 1><<<grid, kGbThreads, 0, st>>>(
          (const double *)out_grad, ranges, (double *)lm_grad, T * R, S1, D));
  }
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_pruned_tanh(int dtype, const void *enc, const void *dec, const int64_t *ranges,
                                 void *act, int B, int S1, int T, int R, int D, void *stream) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(B >= 0 && S1 >= 1 && T >= 0 && R >= 1 && D >= 1, FRNNT_EINVAL, "bad sizes");
  const long long rows = (long long)B * T * R;
  if (rows == 0) return FRNNT_OK;
  FRNNT_REQUIRE(enc && dec && ranges && act, FRNNT_EINVAL, "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  long long want = (rows + 7) / 8;
  const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
  const bool al = (uintptr_t)enc % 16 == 0 && (uintptr_t)dec % 16 == 0 && (uintptr_t)act % 16 == 0;
  if (dtype == FRNNT_F32) {
    if (al && D % 4 == 0)
      FRNNT_KERNEL(pruned_tanh_kernel<float, float4, 4><<<grid, 256, 0, st>>>(
          (const float *)enc, (const float *)dec, ranges, (float *)act, rows, R, T * R, S1, D));
    else
      FRNNT_KERNEL(pruned_tanh_kernel<float, float, 1><<<grid, 256, 0, st>>>(
          (const float *)enc, (const float *)dec, ranges, (float *)act, rows, R, T * R, S1, D));
  } else {
    if (al && D % 2 == 0)
      FRNNT_KERNEL(pruned_tanh_kernel<double, double2, 2><<<grid, 256, 0, st>>>(
          (const double *)enc, (const double *)dec, ranges, (double *)act, rows, R, T * R, S1, D));
    else
      FRNNT_KERNEL(pruned_tanh_kernel<double, double, 1><<<grid, 256, 0, st>>>(
          (const double *)enc, (const double *)dec, ranges, (double *)act, rows, R, T * R, S1, D));
  }
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_sum_over_range(int dtype, const void *gz, void *out, long long frames, int R,
                                    int D, void *stream) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64");
  FRNNT_REQUIRE(frames >= 0 && R >= 1 && D >= 1, FRNNT_EINVAL, "bad sizes");
  if (frames == 0) return FRNNT_OK;
  FRNNT_REQUIRE(gz && out, FRNNT_EINVAL, "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  long long want = (frames + 7) / 8;
  const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
  const bool al = (uintptr_t)gz % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (dtype == FRNNT_F32) {
    if (al && D % 4 == 0)
      FRNNT_KERNEL(sum_over_range_kernel<float, float4, 4><<<grid, 256, 0, st>>>(
          (const float *)gz, (float *)out, frames, R, D));
    else
      FRNNT_KERNEL(sum_over_range_kernel<float, float, 1><<<grid, 256, 0, st>>>(
          (const float *)gz, (float *)out, frames, R, D));
  } else {
    if (al && D % 2 == 0)
      FRNNT_KERNEL(sum_over_range_kernel<double, double2, 2><<<grid, 256, 0, st>>>(
          (const double *)gz, (double *)out, frames, R, D));
    else
      FRNNT_KERNEL(sum_over_range_kernel<double, double, 1><<<grid, 256, 0, st>>>(
          (const double *)gz, (double *)out, frames, R, D));
  }
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" size_t frnnt_joiner_input_grads_scratch_bytes(int B, int T, int D) {
  if (B <= 0 || T <= 0 || D <= 0) return 0;
  const size_t nch = (size_t)(T + kJgFrames - 1) / kJgFrames;
  return (size_t)B * nch * ((size_t)kJgWindow * D * sizeof(float) + 2 * sizeof(int));
}

extern "C" int frnnt_joiner_input_grads(const float *gz, const int64_t *ranges, float *enc_grad,
                                        float *dec_grad, void *scratch, int B, int S1, int T, int R,
                                        int D, void *stream) {
  FRNNT_REQUIRE(B >= 0 && S1 >= 1 && T >= 0 && R >= 1 && D >= 1, FRNNT_EINVAL, "bad sizes");
  FRNNT_REQUIRE(B <= 65535, FRNNT_EUNSUPPORTED, "B too large for the grid");
  FRNNT_REQUIRE(D % 4 == 0 && (size_t)kJgWindow * D * sizeof(float) <= 200 * 1024, FRNNT_EUNSUPPORTED,
                "D must be a multiple of 4 and at most %d", 200 * 1024 / (kJgWindow * 4));
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(dec_grad != nullptr, FRNNT_EINVAL, "dec_grad is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  FRNNT_CUDA(cudaMemsetAsync(dec_grad, 0, (size_t)B * S1 * D * sizeof(float), st));
  if (T == 0) return FRNNT_OK;
  FRNNT_REQUIRE(gz && ranges && scratch, FRNNT_EINVAL, "NULL argument");
  FRNNT_REQUIRE((uintptr_t)gz % 16 == 0 && (uintptr_t)enc_grad % 16 == 0 && (uintptr_t)dec_grad % 16 == 0 &&
                    (uintptr_t)scratch % 16 == 0,
                FRNNT_EUNSUPPORTED, "pointers must be 16-byte aligned");
  const int nch = (T + kJgFrames - 1) / kJgFrames;
  float *partial = (float *)scratch;
  int *window = (int *)(partial + (size_t)B * nch * kJgWindow * D);
  const size_t smem = (size_t)kJgWindow * D * sizeof(float);
  if (R <= 8) {  // the window in registers; wider bands keep it in shared memory
    const dim3 grid((unsigned)nch, (unsigned)B);
#define FRNNT_JG_RING(RR)                                                                                         \
  case RR:                                                                                                        \
    if (enc_grad != nullptr)                                                                                      \
      FRNNT_KERNEL(joiner_input_grads_ring_kernel<true, RR><<<grid, kJgThreads, 0, st>>>(gz, ranges, enc_grad,     \
                                                                                       dec_grad, partial, window, \
                                                                                       T, S1, D));                \
    else                                                                                                          \
      FRNNT_KERNEL(joiner_input_grads_ring_kernel<false, RR><<<grid, kJgThreads, 0, st>>>(gz, ranges, nullptr,     \
                                                                                        dec_grad, partial, window,\
                                                                                        T, S1, D));               \
    break;
    switch (R) {
      FRNNT_JG_RING(1) FRNNT_JG_RING(2) FRNNT_JG_RING(3) FRNNT_JG_RING(4)
      FRNNT_JG_RING(5) FRNNT_JG_RING(6) FRNNT_JG_RING(7) FRNNT_JG_RING(8)
    }
#undef FRNNT_JG_RING
  } else if (enc_grad != nullptr) {
    FRNNT_CUDA(cudaFuncSetAttribute(joiner_input_grads_kernel<true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FRNNT_KERNEL(joiner_input_grads_kernel<true><<<dim3((unsigned)nch, (unsigned)B), kJgThreads, smem, st>>>(
        gz, ranges, enc_grad, dec_grad, partial, window, T, R, S1, D));
  } else {
    FRNNT_CUDA(cudaFuncSetAttribute(joiner_input_grads_kernel<false>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FRNNT_KERNEL(joiner_input_grads_kernel<false><<<dim3((unsigned)nch, (unsigned)B), kJgThreads, smem, st>>>(
        gz, ranges, nullptr, dec_grad, partial, window, T, R, S1, D));
  }
  FRNNT_KERNEL(joiner_dec_reduce_kernel<<<dim3((unsigned)S1, (unsigned)B), kJgThreads, 0, st>>>(
      partial, window, dec_grad, nch, S1, D));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}
