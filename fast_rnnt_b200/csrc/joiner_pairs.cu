// The pruned joiner and the pruned log-prob lattices as ONE operator:
//
//   px, py = get_rnnt_logprobs_pruned(Linear(tanh(am_pruned + lm_pruned)), symbols, ranges, ...)
//   with am_pruned, lm_pruned = do_rnnt_pruning(enc, dec, ranges)
//
// i.e. the caller's network between do_rnnt_pruning and rnnt_loss_pruned in the
// reference's documented usage (README.md:180-190) together with
// fast_rnnt/python/fast_rnnt/rnnt_loss.py:810-817 (pruning) and :940-1022 (log-softmax,
// symbol / blank gather, placement into the lattices), forward and backward.  No
// counterpart in the reference, which leaves the joiner to the caller and therefore
// cannot fuse across it.
//
// What the fusion buys: every matrix that feeds a tensor-core product is written by its
// producer as a pair of fp16 planes (umma_pairs.cuh), so the three products run as pure
// TMA -> tcgen05 pipelines at the fp16 rate with fp32-level accuracy:
//   forward    tanh(enc + dec[ranges]) -> act planes;  W -> planes (both orientations);
//              logits = act * W^T + bias on the tensor cores, whose epilogue also leaves
//              a (max, sum exp) pair per row and 128-column tile, so that no second pass
//              over the logits is needed for the log-sum-exp; a small kernel combines the
//              pairs, picks logit[symbol] and logit[blank] and the bands go into px, py.
//   backward   g = d loss / d logits from logits, lse and the lattice gradients -> planes,
//              with the column sums of g (the bias gradient) taken on the way;
//              gz = (g * W) * (1 - act^2) on the tensor cores (tanh' in the epilogue);
//              enc_grad / dec_grad from one pass over gz;  W_grad = g^T * act, split-K.
#include <cuda_fp16.h>

#include <stdlib.h>

#include <algorithm>

#include "lsm_band.cuh"
#include "umma_pairs256.cuh"

namespace frnnt {

constexpr float kActScale = 16384.f;  // 2^14: |tanh| <= 1, so the planes stay below 2^14
constexpr int kMaxParts = 1024;       // per-CTA partial maxima of a reduction

enum { kScaleAct = 0, kScaleW = 1, kScaleG = 2 };  // slots of the inverse scales

static inline size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

// rows of an output tile.  The large-tile kernel (umma_pairs256.cuh: 256 x 128, or 128 x 256
// where the output is wider than 128 columns) moves a quarter fewer bytes per flop, but its
// eight warps do both folding and epilogue with the running sums in registers; measured at C3
// it wins where the epilogue is trivial and the reduction long (grad-weight, plain products:
// 0.235 -> 0.21 -> 0.20 ms) and loses where the epilogue carries the log-sum-exp partials or the
// tanh' activations (forward product 0.254 -> 0.260 ms, grad-input 0.28 -> 0.39 ms with 128 x 256),
// so only the former use it.  FRNNT_PAIR_TILE=128 forces the 128 x 128 kernel everywhere.
static int pair_tile_m(int M, bool light_epilogue) {
  const char *e = getenv("FRNNT_PAIR_TILE");  // read at every call: tests switch it
  const bool forced = e != nullptr && atoi(e) == 128;
  return (forced || !light_epilogue || M <= kPairTile) ? kPairTile : kP2TileM;
}

template <bool A_MN, bool B_MN, class Ext>
static int launch_pair(const CUtensorMap &mah, const CUtensorMap &mal, const CUtensorMap &mbh,
                       const CUtensorMap &mbl, float *out, LinShape shape, const Ext &ext, cudaStream_t st) {
  const int tm = pair_tile_m(shape.M, Ext::kLightEpilogue);
  if (Ext::kLightEpilogue && shape.N > kPairTile && pair_tile_m(2 * kPairTile, true) != kPairTile) {
    // 128 x 256: one MMA of N = 256 per product and step (grad-weight at C3: 0.212 -> 0.201 ms)
    shape.tiles_m = (shape.M + kPairTile - 1) / kPairTile;
    shape.tiles_n = (shape.N + 2 * kPairTile - 1) / (2 * kPairTile);
    return launch_pair_umma256<A_MN, B_MN, Ext, true>(mah, mal, mbh, mbl, out, shape, ext, st);
  }
  shape.tiles_m = (shape.M + tm - 1) / tm;
  if (tm == kP2TileM) return launch_pair_umma256<A_MN, B_MN>(mah, mal, mbh, mbl, out, shape, ext, st);
  return launch_pair_umma<A_MN, B_MN>(mah, mal, mbh, mbl, out, shape, ext, st);
}

static int pair_tn_splits(int M, int N, long long R) {
  if (M <= 0 || N <= 0 || R <= 0) return 1;
  const int tm = pair_tile_m(M, true);  // the split products have light epilogues
  const long long tiles = (long long)((M + tm - 1) / tm) * ((N + kPairTile - 1) / kPairTile);
  const long long max_splits = (R + 8 * kPairBK - 1) / (8 * kPairBK);
  const long long sms = sm_count();
  int best = 1;
  double best_cost = 1e30;
  for (int sp = 1; sp <= 64 && sp <= max_splits; ++sp) {
    const long long waves = (tiles * sp + sms - 1) / sms;
    const double cost = (double)waves / sp + 0.002 * sp;
    if (cost < best_cost - 1e-12) {
      best_cost = cost;
      best = sp;
    }
  }
  return best;
}

// row groups of the log-softmax backward: each CTA streams a contiguous group of rows for
// one chunk of 1024 columns; about eight CTAs per SM over all chunks
// threads per CTA of that kernel: one per 4-column vector, whole warps, at most 256
static int lsm_threads(int C) {
  const int nvec = C / 4;
  return nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
}
static int colsum_groups(long long rows, int C) {
  const int th = lsm_threads(C);
  const long long chunks = ((long long)C / 4 + th - 1) / th;
  long long want = ((long long)sm_count() * 8 + chunks - 1) / chunks;
  const long long cap = (rows + 3) / 4;  // at least four rows per group
  want = want < cap ? want : cap;
  return (int)(want < 1 ? 1 : want);
}

// Offsets (bytes) of everything the operator keeps: `saved` lives from forward to
// backward, the two scratch areas only during one call.
struct PjlLayout {
  size_t M, Cp;
  int tiles_n, splits, cs_ctas;
  size_t act_hi, act_lo, logits, lse, wt_hi, wt_lo, scales, saved_bytes;
  size_t w_hi, w_lo, stats, pxb, pyb, amax_part, fwd_bytes;
  size_t g_hi, g_lo, gz, rowinfo, gmax_part, dw_part, cs_part, jg, bwd_bytes;
};

static PjlLayout pjl_layout(int B, int T, int R, int S1, int C, int D) {
  PjlLayout L;
  const size_t M = (size_t)B * T * R;
  // row pitch of the planes whose rows have C entries: whole 128-byte lines, so that the
  // 128-byte row segments TMA fetches never straddle one more 32-byte sector
  const size_t Cp = (size_t)(C + 63) / 64 * 64;
  L.M = M;
  L.Cp = Cp;
  L.tiles_n = (C + kPairTile - 1) / kPairTile;
  L.splits = pair_tn_splits(C, D, (long long)M);
  L.cs_ctas = colsum_groups((long long)M, C);
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t r = o;
    o += up256(bytes);
    return r;
  };
  L.act_hi = take(M * D * 2);
  L.act_lo = take(M * D * 2);
  L.logits = take(M * C * 4);
  L.lse = take(M * 4);
  L.wt_hi = take((size_t)D * Cp * 2);
  L.wt_lo = take((size_t)D * Cp * 2);
  L.scales = take(16 * 4);
  L.saved_bytes = o;
  o = 0;
  L.w_hi = take((size_t)C * D * 2);
  L.w_lo = take((size_t)C * D * 2);
  L.stats = take(M * L.tiles_n * 8);
  L.pxb = take(M * 4);
  L.pyb = take(M * 4);
  L.amax_part = take(kMaxParts * 4);
  L.fwd_bytes = o;
  o = 0;
  L.g_hi = take(M * Cp * 2);
  L.g_lo = take(M * Cp * 2);
  L.gz = take(M * D * 4);
  L.rowinfo = take(M * 16);
  L.gmax_part = take(kMaxParts * 4);
  L.dw_part = take(L.splits > 1 ? (size_t)L.splits * C * D * 4 : 0);
  L.cs_part = take((size_t)L.cs_ctas * C * 4);
  L.jg = take(frnnt_joiner_input_grads_scratch_bytes(B, T, D));
  L.bwd_bytes = o;
  (void)S1;
  return L;
}

// ---- small reductions ---------------------------------------------------------------------
// max over part[0..n), computed by warp 0 and handed to every thread of the block
__device__ float block_max_of_partials(const float *__restrict__ part, int n, float *slot) {
  if (threadIdx.x < 32) {
    float m = 0.f;
    for (int i = threadIdx.x; i < n; i += 32) m = fmaxf(m, part[i]);
    m = warp_max(m);
    if (threadIdx.x == 0) *slot = m;
  }
  __syncthreads();
  return *slot;
}

__global__ void __launch_bounds__(256)
absmax_partial_kernel(const float *__restrict__ x, long long n, float *__restrict__ part) {
  __shared__ float s[8];
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256)
    m = fmaxf(m, fabsf(x[i]));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s[w]);
    part[blockIdx.x] = m;
  }
}

// W [C][D] -> planes in both orientations: w [C][D] (forward: B operand, K = D) and
// wt [D][Cp] (grad-input: B operand, K = C)
__global__ void __launch_bounds__(256)
split_weights_kernel(const float *__restrict__ W, int C, int D, int Cp, const float *__restrict__ part,
                     int nparts, __half *__restrict__ w_hi, __half *__restrict__ w_lo,
                     __half *__restrict__ wt_hi, __half *__restrict__ wt_lo, float *__restrict__ scales) {
  __shared__ float slot;
  const float scale = fp16_pair_scale(block_max_of_partials(part, nparts, &slot));
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[kScaleW] = 1.f / scale;
  const long long n = (long long)C * D;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const int c = (int)(i / D), d = (int)(i - (long long)c * D);
    __half hi, lo;
    fp16_pair(W[i], scale, hi, lo);
    w_hi[i] = hi;
    w_lo[i] = lo;
    wt_hi[(size_t)d * Cp + c] = hi;
    wt_lo[(size_t)d * Cp + c] = lo;
  }
}

// act[b][t][k][:] = tanh(enc[b][t][:] + dec[b][ranges[b][t][k]][:]) as planes; one warp per
// row, eight columns per lane
// eight consecutive inputs starting at element 8 * v of a row, as float32
__device__ __forceinline__ void in_load8(const float *row, int v, float (&x)[8]) {
  const float4 a = reinterpret_cast<const float4 *>(row)[2 * v], b = reinterpret_cast<const float4 *>(row)[2 * v + 1];
  x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
}
template <typename T16>
__device__ __forceinline__ void in_load8(const T16 *row, int v, float (&x)[8]) {
  const float4 a = in_load4(row, 2 * v), b = in_load4(row, 2 * v + 1);
  x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
}

template <typename TIn>
__global__ void __launch_bounds__(256)
pruned_tanh_pairs_kernel(const TIn *__restrict__ enc, const TIn *__restrict__ dec,
                         const int64_t *__restrict__ ranges, __half *__restrict__ act_hi,
                         __half *__restrict__ act_lo, long long frames, int R, int T, int S1, int D,
                         float *__restrict__ scales) {
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[kScaleAct] = 1.f / kActScale;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int d8 = D / 8;
  // one warp per frame (b, t): its encoder row is read once and stays in registers for the R
  // rows of the band (the kernel moves about 1 GB through the L2 for 0.33 GB of planes
  // otherwise, which is what bounds it, not HBM)
  for (long long bt = warp0; bt < frames; bt += nwarps) {
    const long long b = div_rows(bt, T);
    const TIn *e = enc + (size_t)bt * D;
    const int64_t *rg = ranges + (size_t)bt * R;
    for (int v0 = 0; v0 < d8; v0 += 64) {  // 16 columns per lane and pass
      const int va = v0 + lane, vb = v0 + 32 + lane;
      float xa[8], xb[8];
      if (va < d8) in_load8(e, va, xa);
      if (vb < d8) in_load8(e, vb, xb);
      for (int k = 0; k < R; ++k) {
        long long s = rg[k];
        s = s < 0 ? 0 : (s >= S1 ? S1 - 1 : s);
        const TIn *d = dec + ((size_t)b * S1 + s) * D;
        const size_t row = (size_t)bt * R + k;
        uint4 *oh = reinterpret_cast<uint4 *>(act_hi + row * D);
        uint4 *ol = reinterpret_cast<uint4 *>(act_lo + row * D);
        float ya[8], yb[8];
        if (va < d8) in_load8(d, va, ya);
        if (vb < d8) in_load8(d, vb, yb);
        auto emit = [&](const float (&x)[8], const float (&y)[8], int v) {
          const float t0[4] = {tanhf(x[0] + y[0]), tanhf(x[1] + y[1]), tanhf(x[2] + y[2]), tanhf(x[3] + y[3])};
          const float t1[4] = {tanhf(x[4] + y[4]), tanhf(x[5] + y[5]), tanhf(x[6] + y[6]), tanhf(x[7] + y[7])};
          uint2 h0, l0, h1, l1;
          fp16_pair4(t0, kActScale, h0, l0);
          fp16_pair4(t1, kActScale, h1, l1);
          oh[v] = make_uint4(h0.x, h0.y, h1.x, h1.y);
          ol[v] = make_uint4(l0.x, l0.y, l1.x, l1.y);
        };
        if (va < d8) emit(xa, ya, va);
        if (vb < d8) emit(xb, yb, vb);
      }
    }
  }
}

// ---- epilogues of the three products ----------------------------------------------------------
// logits = acc * (1/scales) + bias, and per row and tile (max, sum exp(logit - max))
struct PjlFwdExt {
  static constexpr bool kBatched = false, kCustomStore = false, kLightEpilogue = false;
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
  const float *bias;
  float2 *stats;
  const float *scales;
  int N, tiles_n;
  struct Row {
    float sc, mx, sum;
  };
  __device__ void row_begin(Row &r, int, int, int) const {
    r.sc = scales[kScaleAct] * scales[kScaleW];
    r.mx = -INFINITY;
    r.sum = 0.f;
  }
  __device__ void prefetch(Row &, int, int, int) const {}
  __device__ void finish(Row &r, int, int, int n, float (&v)[16], int) const {
    float cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const bool in = n + i < N;
      v[i] = v[i] * r.sc + ((bias != nullptr && in) ? bias[n + i] : 0.f);
      cm = in ? fmaxf(cm, v[i]) : cm;
    }
    if (cm > r.mx) {
      r.sum *= __expf(r.mx - cm);
      r.mx = cm;
    }
    const float base = (r.mx - r.mx != 0.f) ? 0.f : r.mx;  // an infinite maximum: as torch.logsumexp
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (n + i < N) r.sum += __expf(v[i] - base);
  }
  __device__ void row_end(Row &r, int, int m, int n0) const {
    stats[(size_t)m * tiles_n + n0 / kPairTile] = make_float2(r.mx, r.sum);
  }
};

// gz = acc * (1/scales) * (1 - act^2): the gradient with respect to enc + dec
struct PjlGradInExt {
  static constexpr bool kBatched = false, kCustomStore = false, kLightEpilogue = false;
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
  const __half *act_hi, *act_lo;
  const float *scales;
  int N;  // = D
  struct Row {
    float sc;
    uint4 h[4], l[4];  // the 32 activations (two planes) of the columns that come next
  };
  __device__ void row_begin(Row &r, int, int, int) const { r.sc = scales[kScaleG] * scales[kScaleW]; }
  __device__ void prefetch(Row &r, int, int m, int n) const {
    if (n + 32 <= N) {
      const uint4 *h = reinterpret_cast<const uint4 *>(act_hi + (size_t)m * N + n);
      const uint4 *l = reinterpret_cast<const uint4 *>(act_lo + (size_t)m * N + n);
#pragma unroll
      for (int i = 0; i < 4; ++i) r.h[i] = h[i], r.l[i] = l[i];
    }
  }
  __device__ void finish(Row &r, int, int m, int n, float (&v)[16], int half) const {
    const int n32 = n - 16 * half;
    if (n32 + 32 <= N) {
      __align__(16) __half hh[16], ll[16];
      *reinterpret_cast<uint4 *>(hh) = r.h[2 * half];
      *reinterpret_cast<uint4 *>(hh + 8) = r.h[2 * half + 1];
      *reinterpret_cast<uint4 *>(ll) = r.l[2 * half];
      *reinterpret_cast<uint4 *>(ll + 8) = r.l[2 * half + 1];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = (__half2float(hh[i]) + __half2float(ll[i])) * (1.f / kActScale);
        v[i] = v[i] * r.sc * (1.f - a * a);
      }
    } else {
      const __half *h = act_hi + (size_t)m * N + n, *l = act_lo + (size_t)m * N + n;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (n + i < N) {
          const float a = (__half2float(h[i]) + __half2float(l[i])) * (1.f / kActScale);
          v[i] = v[i] * r.sc * (1.f - a * a);
        }
      }
    }
  }
  __device__ void row_end(Row &, int, int, int) const {}
};

// W_grad partial sums: acc * (1/scales)
struct PjlGradWExt {
  static constexpr bool kBatched = false, kCustomStore = false, kLightEpilogue = true;
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
  const float *scales;
  struct Row {
    float sc;
  };
  __device__ void row_begin(Row &r, int, int, int) const { r.sc = scales[kScaleG] * scales[kScaleAct]; }
  __device__ void prefetch(Row &, int, int, int) const {}
  __device__ void finish(Row &r, int, int, int, float (&v)[16], int) const {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] *= r.sc;
  }
  __device__ void row_end(Row &, int, int, int) const {}
};

// out[i] = sum over z of partial[z][i], z in order
__global__ void ordered_sum_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                   long long n, int parts) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0;
  for (int z = 0; z < parts; ++z) acc += partial[(size_t)z * n + i];
  out[i] = acc;
}

// column sums per row group -> bias gradient.  The partials are stored column-major,
// partial[c][g]: one warp per column reads them as contiguous lines, every lane adds the
// groups g = lane, lane + 32, ... in order and the lanes are combined by a fixed shuffle
// tree -- the same order on every run.
__global__ void __launch_bounds__(256)
ordered_sum_cols_kernel(const float *__restrict__ partial, float *__restrict__ out, int n, int groups) {
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (c >= n) return;
  const float *src = partial + (size_t)c * groups;
  float acc = 0.f;
  for (int g = lane; g < groups; g += 32) acc += src[g];
  acc = warp_sum(acc);
  if (lane == 0) out[c] = acc;
}

// ---- bands ------------------------------------------------------------------------------------
// per row (b, t, k): lse from the per-tile (max, sum) pairs, logit[symbol] - lse, logit[blank] - lse
__global__ void __launch_bounds__(256)
joiner_band_kernel(const float *__restrict__ logits, const float2 *__restrict__ stats,
                   const int64_t *__restrict__ symbols, const int64_t *__restrict__ ranges,
                   float *__restrict__ lse, float *__restrict__ pxb, float *__restrict__ pyb,
                   long long rows, int T, int R, int S, int C, int blank, int tiles_n) {
  const long long row = (long long)blockIdx.x * 256 + threadIdx.x;
  if (row >= rows) return;
  const float2 *st = stats + (size_t)row * tiles_n;
  float m = -INFINITY;
  for (int j = 0; j < tiles_n; ++j) m = fmaxf(m, st[j].x);
  const float m0 = (m - m != 0.f) ? 0.f : m;
  float sum = 0.f;
  for (int j = 0; j < tiles_n; ++j) {
    const float2 q = st[j];
    const float base = (q.x - q.x != 0.f) ? 0.f : q.x;  // what the tile's sum was taken against
    sum += q.y * __expf(base - m0);
  }
  const float l = logf(sum) + m0;
  const long long bt = div_rows(row, R);
  const int k = mod_rows(row, R), b = (int)div_rows(bt, T);
  const int y = band_symbol(symbols, ranges, b, (size_t)row, k, S, blank, C);
  const float *x = logits + (size_t)row * C;
  lse[row] = l;
  pxb[row] = x[y] - l;
  pyb[row] = x[blank] - l;
}

// per row (b, t, k): what the log-softmax backward needs of it in one 16-byte entry -- the
// gradients that reach its two band entries from the lattices (the inverse of
// band_to_lattice_kernel), its log-sum-exp and its symbol -- and the largest |gx| + |gy|
// of each CTA's rows
__global__ void __launch_bounds__(256)
band_grad_kernel(const float *__restrict__ g_px, const float *__restrict__ g_py,
                 const int64_t *__restrict__ symbols, const int64_t *__restrict__ ranges,
                 const int64_t *__restrict__ boundary, const float *__restrict__ lse,
                 float4 *__restrict__ rowinfo, float *__restrict__ part, long long rows, int T, int R,
                 int S, int C, int blank, int rnnt_type) {
  __shared__ float sm[8];
  const int S1 = S + 1;
  const int T1 = (rnnt_type == FRNNT_REGULAR) ? T + 1 : T;
  float mx = 0.f;
  for (long long row = (long long)blockIdx.x * 256 + threadIdx.x; row < rows; row += (long long)gridDim.x * 256) {
    const long long bt = div_rows(row, R);
    const int k = mod_rows(row, R);
    const int b = (int)div_rows(bt, T), t = mod_rows(bt, T);
    const int s = band_row(ranges, (size_t)bt, R, k, S1);
    float gx = 0.f, gy = g_py[((size_t)b * S1 + s) * T + t];
    const bool masked = rnnt_type == FRNNT_REGULAR && boundary != nullptr &&
                        (long long)t == (long long)boundary[4 * b + 3];
    if (s < S && !masked) gx = g_px[((size_t)b * S + s) * T1 + t];
    if (rnnt_type == FRNNT_CONSTRAINED && s >= 1) gy += g_px[((size_t)b * S + s - 1) * T1 + t];
    const int y = band_symbol(symbols, ranges, b, (size_t)row, k, S, blank, C);
    rowinfo[row] = make_float4(gx, gy, lse[row], __int_as_float(y));
    mx = fmaxf(mx, fabsf(gx) + fabsf(gy));
  }
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, sm[w]);
    part[blockIdx.x] = mx;
  }
}

// g[row][c] = -(gx + gy) * exp(logit - lse) + gx * [c == symbol] + gy * [c == blank], written
// as planes (|g| <= |gx| + |gy|, whose maximum sets the scale).  Thread <-> four columns,
// CTA <-> a contiguous group of rows x a chunk of up to 1024 columns: the loads of four rows are
// in flight together, and the column sums of g (the bias gradient) stay in registers across
// the whole group -> one partial per group, added in a fixed order afterwards (no atomics).
constexpr int kLsmRowsInFlight = 4;
__global__ void __launch_bounds__(256)
lsm_backward_pairs_kernel(const float *__restrict__ logits, const float4 *__restrict__ rowinfo,
                          const float *__restrict__ gmax_part, int nparts, __half *__restrict__ g_hi,
                          __half *__restrict__ g_lo, float *__restrict__ cs_part,
                          float *__restrict__ scales, long long rows, int C, int Cp, int blank, int groups) {
  __shared__ float slot;
  const float scale = fp16_pair_scale(block_max_of_partials(gmax_part, nparts, &slot));
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) scales[kScaleG] = 1.f / scale;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;  // this thread's 4-column vector
  const bool col_ok = v < C / 4;
  const long long per = (rows + groups - 1) / groups;
  const long long r0 = (long long)blockIdx.y * per;
  const long long r1 = r0 + per < rows ? r0 + per : rows;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int c0 = 4 * v;
  for (long long row = r0; row < r1; row += kLsmRowsInFlight) {
    float4 q[kLsmRowsInFlight], info[kLsmRowsInFlight];
#pragma unroll
    for (int u = 0; u < kLsmRowsInFlight; ++u) {
      const long long r = row + u < r1 ? row + u : r1 - 1;
      info[u] = rowinfo[r];
      q[u] = col_ok ? reinterpret_cast<const float4 *>(logits + (size_t)r * C)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (!col_ok) continue;
#pragma unroll
    for (int u = 0; u < kLsmRowsInFlight; ++u) {
      if (row + u >= r1) break;
      const float gx = info[u].x, gy = info[u].y, l = info[u].z;
      const int y = __float_as_int(info[u].w);
      const float neg = -(gx + gy);
      const float x[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
      float g[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float gg = neg * __expf(x[e] - l);
        if (c0 + e == y) gg += gx;
        if (c0 + e == blank) gg += gy;
        g[e] = gg;
      }
      uint2 hi, lo;
      fp16_pair4(g, scale, hi, lo);
      reinterpret_cast<uint2 *>(g_hi + (size_t)(row + u) * Cp)[v] = hi;
      reinterpret_cast<uint2 *>(g_lo + (size_t)(row + u) * Cp)[v] = lo;
      acc.x += g[0], acc.y += g[1], acc.z += g[2], acc.w += g[3];
    }
  }
  if (col_ok) {  // column-major: partial[c][group]
    float *dst = cs_part + (size_t)c0 * groups + blockIdx.y;
    dst[0] = acc.x;
    dst[(size_t)groups] = acc.y;
    dst[(size_t)2 * groups] = acc.z;
    dst[(size_t)3 * groups] = acc.w;
  }
}

// ---- plain products on planes (the engine without the joiner around it) -------------------------
// D = acc * inv_scale_a * inv_scale_b (+ bias[n])
struct PlainPairExt {
  static constexpr bool kBatched = false, kCustomStore = false, kLightEpilogue = true;
  template <class R> __device__ void store_box(R &, int, int, int, int, float (&)[16], float (&)[16], const uint8_t *) const {}
  __device__ void tile_begin(int, int, uint8_t *, int) const {}
  const float *bias, *inv_a, *inv_b;
  int N;
  struct Row {
    float sc;
  };
  __device__ void row_begin(Row &r, int, int, int) const { r.sc = *inv_a * *inv_b; }
  __device__ void prefetch(Row &, int, int, int) const {}
  __device__ void finish(Row &r, int, int, int n, float (&v)[16], int) const {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = v[i] * r.sc + ((bias != nullptr && n + i < N) ? bias[n + i] : 0.f);
  }
  __device__ void row_end(Row &, int, int, int) const {}
};

// x [rows][cols] -> planes [rows][pitch], scaled by the power of two that the largest
// magnitude (from the per-CTA partial maxima) asks for
__global__ void __launch_bounds__(256)
split_matrix_kernel(const float *__restrict__ x, long long rows, int cols, long long pitch,
                    const float *__restrict__ part, int nparts, __half *__restrict__ hi,
                    __half *__restrict__ lo, float *__restrict__ inv_scale) {
  __shared__ float slot;
  const float scale = fp16_pair_scale(block_max_of_partials(part, nparts, &slot));
  if (blockIdx.x == 0 && threadIdx.x == 0) *inv_scale = 1.f / scale;
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    __half h, l;
    fp16_pair(x[i], scale, h, l);
    hi[r * pitch + c] = h;
    lo[r * pitch + c] = l;
  }
}

static int pjl_check(int B, int T, int R, int S, int C, int D, int blank, int rnnt_type) {
  FRNNT_REQUIRE(B >= 0 && T >= 0 && R >= 1 && S >= 0 && C >= 1 && D >= 1, FRNNT_EINVAL,
                "bad sizes B=%d T=%d R=%d S=%d C=%d D=%d", B, T, R, S, C, D);
  FRNNT_REQUIRE(R <= S + 1, FRNNT_EINVAL, "band width R=%d exceeds S+1=%d", R, S + 1);
  FRNNT_REQUIRE(blank >= 0 && blank < C, FRNNT_EINVAL, "blank=%d outside [0,%d)", blank, C);
  FRNNT_REQUIRE(rnnt_type >= 0 && rnnt_type <= 2, FRNNT_EINVAL, "bad rnnt_type %d", rnnt_type);
  FRNNT_REQUIRE(D % 8 == 0 && C % 4 == 0, FRNNT_EUNSUPPORTED,
                "the fused joiner needs D (=%d) to be a multiple of 8 and C (=%d) a multiple of 4", D, C);
  FRNNT_REQUIRE(S + 1 <= 65535 && B <= 65535, FRNNT_EUNSUPPORTED, "S or B too large for the grid");
  FRNNT_REQUIRE((long long)B * T * R < (1LL << 31) - 256, FRNNT_EUNSUPPORTED,
                "more than 2^31 joiner rows");
  return FRNNT_OK;
}

static int parts_for(long long n) {
  long long want = (n + 255) / 256;
  return (int)(want < 1 ? 1 : (want < kMaxParts ? want : kMaxParts));
}

}  // namespace frnnt

using namespace frnnt;

extern "C" size_t frnnt_pruned_joiner_saved_bytes(int B, int T, int R, int S, int C, int D) {
  if (B <= 0 || T <= 0 || R <= 0 || C <= 0 || D <= 0) return 0;
  return pjl_layout(B, T, R, S + 1, C, D).saved_bytes;
}
extern "C" size_t frnnt_pruned_joiner_forward_scratch_bytes(int B, int T, int R, int S, int C, int D) {
  if (B <= 0 || T <= 0 || R <= 0 || C <= 0 || D <= 0) return 0;
  return pjl_layout(B, T, R, S + 1, C, D).fwd_bytes;
}
extern "C" size_t frnnt_pruned_joiner_backward_scratch_bytes(int B, int T, int R, int S, int C, int D) {
  if (B <= 0 || T <= 0 || R <= 0 || C <= 0 || D <= 0) return 0;
  return pjl_layout(B, T, R, S + 1, C, D).bwd_bytes;
}

// parts of a forward / backward call (bit mask); the diagnostic entry points re-launch one
enum { kPartPlanes = 1, kPartProduct = 2, kPartRest = 4, kPartProduct2 = 8, kPartInputGrads = 16 };

static int pjl_forward(int input_dtype, const void *enc, const void *dec, const int64_t *ranges, const float *weight,
                       const float *bias, const int64_t *symbols, const int64_t *boundary, float *px,
                       float *py, void *saved, void *scratch, int B, int T, int R, int S, int C, int D,
                       int blank, int rnnt_type, double delay_penalty, void *stream, unsigned parts) {
  int rc = pjl_check(B, T, R, S, C, D, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0 || T == 0) return FRNNT_OK;
  FRNNT_REQUIRE(enc && dec && ranges && weight && px && py && saved && scratch && (symbols || S == 0),
                FRNNT_EINVAL, "NULL argument");
  FRNNT_REQUIRE((uintptr_t)enc % 16 == 0 && (uintptr_t)dec % 16 == 0 && (uintptr_t)saved % 256 == 0 &&
                    (uintptr_t)scratch % 256 == 0,
                FRNNT_EINVAL, "enc / dec must be 16-byte aligned, saved / scratch 256-byte aligned");
  const PjlLayout L = pjl_layout(B, T, R, S + 1, C, D);
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t *sv = (uint8_t *)saved, *sc = (uint8_t *)scratch;
  __half *act_hi = (__half *)(sv + L.act_hi), *act_lo = (__half *)(sv + L.act_lo);
  __half *wt_hi = (__half *)(sv + L.wt_hi), *wt_lo = (__half *)(sv + L.wt_lo);
  __half *w_hi = (__half *)(sc + L.w_hi), *w_lo = (__half *)(sc + L.w_lo);
  float *logits = (float *)(sv + L.logits), *lse = (float *)(sv + L.lse), *scales = (float *)(sv + L.scales);
  float2 *stats = (float2 *)(sc + L.stats);
  float *pxb = (float *)(sc + L.pxb), *pyb = (float *)(sc + L.pyb), *amax = (float *)(sc + L.amax_part);
  const long long rows = (long long)L.M;
  const int M = (int)rows;

  // tensor maps first: nothing has been launched if one of them is refused
  CUtensorMap mah, mal, mbh, mbl;
  rc = make_pair_map(&mah, act_hi, M, D, D, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mal, act_lo, M, D, D, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbh, w_hi, C, D, D, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbl, w_lo, C, D, D, false);
  if (rc != FRNNT_OK) return rc;

  if (parts & kPartPlanes) {
    const long long nW = (long long)C * D;
    const int wparts = parts_for(nW);
    FRNNT_KERNEL(absmax_partial_kernel<<<wparts, 256, 0, st>>>(weight, nW, amax));
    FRNNT_KERNEL(split_weights_kernel<<<wparts, 256, 0, st>>>(weight, C, D, (int)L.Cp, amax, wparts, w_hi, w_lo,
                                                             wt_hi, wt_lo, scales));
    long long want = (rows + 7) / 8;
    const int grid = (int)(want < (long long)sm_count() * 32 ? want : (long long)sm_count() * 32);
    if (input_dtype == FRNNT_F16) {
      FRNNT_KERNEL(pruned_tanh_pairs_kernel<__half><<<grid, 256, 0, st>>>(
          (const __half *)enc, (const __half *)dec, ranges, act_hi, act_lo, (long long)B * T, R, T, S + 1, D, scales));
    } else if (input_dtype == FRNNT_BF16) {
      FRNNT_KERNEL(pruned_tanh_pairs_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          (const __nv_bfloat16 *)enc, (const __nv_bfloat16 *)dec, ranges, act_hi, act_lo, (long long)B * T, R, T, S + 1, D,
          scales));
    } else {
      FRNNT_KERNEL(pruned_tanh_pairs_kernel<float><<<grid, 256, 0, st>>>(
          (const float *)enc, (const float *)dec, ranges, act_hi, act_lo, (long long)B * T, R, T, S + 1, D, scales));
    }
    FRNNT_CUDA(cudaGetLastError());
  }
  if (parts & kPartProduct) {
    const int mt = (M + kPairTile - 1) / kPairTile;
    const LinShape shape{M, C, D, ((D + kPairBK - 1) / kPairBK) * kPairBK, mt, L.tiles_n, 1};
    rc = launch_pair<false, false>(mah, mal, mbh, mbl, logits, shape,
                                   PjlFwdExt{bias, stats, scales, C, L.tiles_n}, st);
    if (rc != FRNNT_OK) return rc;
  }
  if (parts & kPartRest) {
    FRNNT_KERNEL(joiner_band_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(
        logits, stats, symbols, ranges, lse, pxb, pyb, rows, T, R, S, C, blank, L.tiles_n));
    dim3 grid2((unsigned)((T + 1 + 127) / 128), (unsigned)(S + 1), (unsigned)B);
    FRNNT_KERNEL(band_to_lattice_kernel<float><<<grid2, 128, 0, st>>>(pxb, pyb, ranges, boundary, px, py, S, T, R,
                                                                     rnnt_type, delay_penalty));
    FRNNT_CUDA(cudaGetLastError());
  }
  return FRNNT_OK;
}

extern "C" int frnnt_pruned_joiner_logprobs_forward(int input_dtype, const void *enc, const void *dec,
                                                    const int64_t *ranges, const float *weight,
                                                    const float *bias, const int64_t *symbols,
                                                    const int64_t *boundary, float *px, float *py,
                                                    void *saved, void *scratch, int B, int T, int R,
                                                    int S, int C, int D, int blank, int rnnt_type,
                                                    double delay_penalty, void *stream) {
  FRNNT_REQUIRE(input_dtype == FRNNT_F32 || is_half_input(input_dtype), FRNNT_EINVAL,
                "input_dtype must be FRNNT_F32, FRNNT_F16 or FRNNT_BF16");
  return pjl_forward(input_dtype, enc, dec, ranges, weight, bias, symbols, boundary, px, py, saved, scratch, B, T, R,
                     S, C, D, blank, rnnt_type, delay_penalty, stream, ~0u);
}

extern "C" int frnnt_pruned_joiner_logprobs_forward_part(int part, const float *enc, const float *dec,
                                                         const int64_t *ranges, const float *weight,
                                                         const float *bias, const int64_t *symbols,
                                                         const int64_t *boundary, float *px, float *py,
                                                         void *saved, void *scratch, int B, int T, int R,
                                                         int S, int C, int D, int blank, int rnnt_type,
                                                         void *stream) {
  FRNNT_REQUIRE(part >= 0 && part <= 2, FRNNT_EINVAL, "part must be 0 (planes), 1 (product) or 2 (lattices)");
  return pjl_forward(FRNNT_F32, enc, dec, ranges, weight, bias, symbols, boundary, px, py, saved, scratch, B, T, R,
                     S, C, D, blank, rnnt_type, 0.0, stream, 1u << part);
}

static int pjl_backward(const float *px_grad, const float *py_grad, const int64_t *ranges,
                        const int64_t *symbols, const int64_t *boundary, void *saved, void *scratch,
                        float *enc_grad, float *dec_grad, float *weight_grad, float *bias_grad, int B, int T,
                        int R, int S, int C, int D, int blank, int rnnt_type, void *stream, unsigned parts) {
  int rc = pjl_check(B, T, R, S, C, D, blank, rnnt_type);
  if (rc != FRNNT_OK) return rc;
  if (B == 0 || T == 0) return FRNNT_OK;
  FRNNT_REQUIRE(py_grad && ranges && saved && scratch && (px_grad || S == 0) && (symbols || S == 0),
                FRNNT_EINVAL, "NULL argument");
  FRNNT_REQUIRE((enc_grad == nullptr) == (dec_grad == nullptr), FRNNT_EINVAL,
                "enc_grad and dec_grad are computed together: pass both or neither");
  FRNNT_REQUIRE((uintptr_t)saved % 256 == 0 && (uintptr_t)scratch % 256 == 0 &&
                    (uintptr_t)enc_grad % 16 == 0 && (uintptr_t)dec_grad % 16 == 0 &&
                    (uintptr_t)weight_grad % 16 == 0,
                FRNNT_EINVAL, "misaligned buffer");
  const PjlLayout L = pjl_layout(B, T, R, S + 1, C, D);
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t *sv = (uint8_t *)saved, *sc = (uint8_t *)scratch;
  const __half *act_hi = (const __half *)(sv + L.act_hi), *act_lo = (const __half *)(sv + L.act_lo);
  const __half *wt_hi = (const __half *)(sv + L.wt_hi), *wt_lo = (const __half *)(sv + L.wt_lo);
  const float *logits = (const float *)(sv + L.logits), *lse = (const float *)(sv + L.lse);
  float *scales = (float *)(sv + L.scales);  // slot kScaleG is written here
  __half *g_hi = (__half *)(sc + L.g_hi), *g_lo = (__half *)(sc + L.g_lo);
  float *gz = (float *)(sc + L.gz);
  float4 *rowinfo = (float4 *)(sc + L.rowinfo);
  float *gmax = (float *)(sc + L.gmax_part), *dw_part = (float *)(sc + L.dw_part);
  float *cs_part = (float *)(sc + L.cs_part);
  const long long rows = (long long)L.M;
  const int M = (int)rows, Cp = (int)L.Cp;

  CUtensorMap gih, gil, wth, wtl, gwh, gwl, ach, acl;
  rc = make_pair_map(&gih, g_hi, M, C, Cp, false);                    // grad-input: A = g, K = C
  if (rc == FRNNT_OK) rc = make_pair_map(&gil, g_lo, M, C, Cp, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&wth, wt_hi, D, C, Cp, false);   // B = W^T planes [D][C]
  if (rc == FRNNT_OK) rc = make_pair_map(&wtl, wt_lo, D, C, Cp, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&gwh, g_hi, M, C, Cp, true);     // grad-weight: K = rows
  if (rc == FRNNT_OK) rc = make_pair_map(&gwl, g_lo, M, C, Cp, true);
  if (rc == FRNNT_OK) rc = make_pair_map(&ach, act_hi, M, D, D, true);
  if (rc == FRNNT_OK) rc = make_pair_map(&acl, act_lo, M, D, D, true);
  if (rc != FRNNT_OK) return rc;

  const int gparts = parts_for(rows);
  if (parts & kPartPlanes) {
    FRNNT_KERNEL(band_grad_kernel<<<gparts, 256, 0, st>>>(px_grad, py_grad, symbols, ranges, boundary, lse, rowinfo,
                                                         gmax, rows, T, R, S, C, blank, rnnt_type));
    const int th = lsm_threads(C);
    dim3 grid((unsigned)((C / 4 + th - 1) / th), (unsigned)L.cs_ctas);
    FRNNT_KERNEL(lsm_backward_pairs_kernel<<<grid, th, 0, st>>>(logits, rowinfo, gmax, gparts, g_hi, g_lo, cs_part,
                                                               scales, rows, C, Cp, blank, L.cs_ctas));
    FRNNT_CUDA(cudaGetLastError());
    if (bias_grad != nullptr) {
      FRNNT_KERNEL(ordered_sum_cols_kernel<<<(unsigned)((C + 7) / 8), 256, 0, st>>>(cs_part, bias_grad, C, L.cs_ctas));
      FRNNT_CUDA(cudaGetLastError());
    }
  }
  const int mt = (M + kPairTile - 1) / kPairTile;
  if (enc_grad != nullptr && (parts & kPartProduct)) {
    const LinShape shape{M, D, C, ((C + kPairBK - 1) / kPairBK) * kPairBK, mt, (D + kPairTile - 1) / kPairTile, 1};
    rc = launch_pair<false, false>(gih, gil, wth, wtl, gz, shape, PjlGradInExt{act_hi, act_lo, scales, D}, st);
    if (rc != FRNNT_OK) return rc;
  }
  if (enc_grad != nullptr && (parts & kPartInputGrads)) {
    if (D % 4 == 0 && D <= 3200) {
      rc = frnnt_joiner_input_grads(gz, ranges, enc_grad, dec_grad, sc + L.jg, B, S + 1, T, R, D, stream);
    } else {
      rc = frnnt_sum_over_range(FRNNT_F32, gz, enc_grad, (long long)B * T, R, D, stream);
      if (rc == FRNNT_OK)
        rc = frnnt_prune_gather_backward(FRNNT_F32, gz, ranges, dec_grad, B, S + 1, T, R, D, stream);
    }
    if (rc != FRNNT_OK) return rc;
  }
  if (weight_grad != nullptr && (parts & kPartProduct2)) {
    const int splits = L.splits;
    const long long kblocks = (rows + kPairBK - 1) / kPairBK;
    const int k_per_split = (int)((kblocks + splits - 1) / splits) * kPairBK;
    const LinShape shape{C, D, M, k_per_split, (C + kPairTile - 1) / kPairTile, (D + kPairTile - 1) / kPairTile,
                         splits};
    float *out = splits == 1 ? weight_grad : dw_part;
    rc = launch_pair<true, true>(gwh, gwl, ach, acl, out, shape, PjlGradWExt{scales}, st);
    if (rc != FRNNT_OK) return rc;
    if (splits > 1) {
      const long long n = (long long)C * D;
      FRNNT_KERNEL(ordered_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dw_part, weight_grad, n, splits));
      FRNNT_CUDA(cudaGetLastError());
    }
  }
  return FRNNT_OK;
}

extern "C" int frnnt_pruned_joiner_logprobs_backward(const float *px_grad, const float *py_grad,
                                                     const int64_t *ranges, const int64_t *symbols,
                                                     const int64_t *boundary, void *saved,
                                                     void *scratch, float *enc_grad, float *dec_grad,
                                                     float *weight_grad, float *bias_grad, int B, int T,
                                                     int R, int S, int C, int D, int blank, int rnnt_type,
                                                     void *stream) {
  return pjl_backward(px_grad, py_grad, ranges, symbols, boundary, saved, scratch, enc_grad, dec_grad, weight_grad,
                      bias_grad, B, T, R, S, C, D, blank, rnnt_type, stream, ~0u);
}

extern "C" int frnnt_pruned_joiner_logprobs_backward_part(int part, const float *px_grad, const float *py_grad,
                                                          const int64_t *ranges, const int64_t *symbols,
                                                          const int64_t *boundary, void *saved, void *scratch,
                                                          float *enc_grad, float *dec_grad, float *weight_grad,
                                                          float *bias_grad, int B, int T, int R, int S, int C,
                                                          int D, int blank, int rnnt_type, void *stream) {
  FRNNT_REQUIRE(part == 0 || part == 1 || part == 3 || part == 4, FRNNT_EINVAL,
                "part must be 0 (planes of g), 1 (grad-input product), 3 (grad-weight product) or 4 (input gradients)");
  return pjl_backward(px_grad, py_grad, ranges, symbols, boundary, saved, scratch, enc_grad, dec_grad, weight_grad,
                      bias_grad, B, T, R, S, C, D, blank, rnnt_type, stream, 1u << part);
}

// ---- plain products on planes ---------------------------------------------------------------------
extern "C" size_t frnnt_pairs_scratch_floats(void) { return kMaxParts; }

extern "C" int frnnt_pairs_from_f32(const float *x, long long rows, int cols, long long pitch, void *hi,
                                    void *lo, float *inv_scale, float *scratch, void *stream) {
  FRNNT_REQUIRE(rows >= 0 && cols >= 0 && pitch >= cols && pitch % 8 == 0, FRNNT_EINVAL,
                "bad sizes rows=%lld cols=%d pitch=%lld (the pitch must be a multiple of 8)", rows, cols, pitch);
  if (rows == 0 || cols == 0) return FRNNT_OK;
  FRNNT_REQUIRE(x && hi && lo && inv_scale && scratch, FRNNT_EINVAL, "NULL argument");
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = rows * cols;
  const int parts = parts_for(n);
  const int grid = (int)std::min<long long>((n + 255) / 256, (long long)sm_count() * 16);
  FRNNT_KERNEL(absmax_partial_kernel<<<parts, 256, 0, st>>>(x, n, scratch));
  FRNNT_KERNEL(split_matrix_kernel<<<grid, 256, 0, st>>>(x, rows, cols, pitch, scratch, parts, (__half *)hi,
                                                        (__half *)lo, inv_scale));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_pair_matmul_nt(const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
                                    const float *inv_scale_a, const float *inv_scale_b, const float *bias,
                                    float *d, int M, int N, int K, long long pitch_a, long long pitch_b,
                                    void *stream) {
  FRNNT_REQUIRE(M >= 0 && N >= 0 && K > 0, FRNNT_EINVAL, "bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0 || N == 0) return FRNNT_OK;
  FRNNT_REQUIRE(a_hi && a_lo && b_hi && b_lo && inv_scale_a && inv_scale_b && d, FRNNT_EINVAL, "NULL argument");
  FRNNT_REQUIRE((uintptr_t)d % 16 == 0, FRNNT_EINVAL, "d is misaligned");
  CUtensorMap mah, mal, mbh, mbl;
  int rc = make_pair_map(&mah, a_hi, M, K, pitch_a, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mal, a_lo, M, K, pitch_a, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbh, b_hi, N, K, pitch_b, false);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbl, b_lo, N, K, pitch_b, false);
  if (rc != FRNNT_OK) return rc;
  const LinShape shape{M, N, K, ((K + kPairBK - 1) / kPairBK) * kPairBK, (M + kPairTile - 1) / kPairTile,
                       (N + kPairTile - 1) / kPairTile, 1};
  return launch_pair<false, false>(mah, mal, mbh, mbl, d, shape,
                                        PlainPairExt{bias, inv_scale_a, inv_scale_b, N}, (cudaStream_t)stream);
}

extern "C" int frnnt_pair_matmul_tn_splits(int M, int N, long long R) { return pair_tn_splits(M, N, R); }

extern "C" int frnnt_pair_matmul_tn(const void *a_hi, const void *a_lo, const void *b_hi, const void *b_lo,
                                    const float *inv_scale_a, const float *inv_scale_b, float *d,
                                    float *partials, int M, int N, long long R, long long pitch_a,
                                    long long pitch_b, void *stream) {
  FRNNT_REQUIRE(M >= 0 && N >= 0 && R > 0 && R < (1LL << 31) - 256, FRNNT_EINVAL,
                "bad sizes M=%d N=%d R=%lld", M, N, R);
  if (M == 0 || N == 0) return FRNNT_OK;
  FRNNT_REQUIRE(a_hi && a_lo && b_hi && b_lo && inv_scale_a && inv_scale_b && d, FRNNT_EINVAL, "NULL argument");
  const int splits = pair_tn_splits(M, N, R);
  FRNNT_REQUIRE(splits == 1 || partials != nullptr, FRNNT_EINVAL,
                "a scratch of frnnt_pair_matmul_tn_splits() * M * N floats is required");
  FRNNT_REQUIRE((uintptr_t)d % 16 == 0 && (uintptr_t)partials % 16 == 0, FRNNT_EINVAL, "misaligned buffer");
  CUtensorMap mah, mal, mbh, mbl;
  int rc = make_pair_map(&mah, a_hi, (int)R, M, pitch_a, true);
  if (rc == FRNNT_OK) rc = make_pair_map(&mal, a_lo, (int)R, M, pitch_a, true);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbh, b_hi, (int)R, N, pitch_b, true);
  if (rc == FRNNT_OK) rc = make_pair_map(&mbl, b_lo, (int)R, N, pitch_b, true);
  if (rc != FRNNT_OK) return rc;
  const long long kblocks = (R + kPairBK - 1) / kPairBK;
  const int k_per_split = (int)((kblocks + splits - 1) / splits) * kPairBK;
  const LinShape shape{M, N, (int)R, k_per_split, (M + kPairTile - 1) / kPairTile,
                       (N + kPairTile - 1) / kPairTile, splits};
  cudaStream_t st = (cudaStream_t)stream;
  float *out = splits == 1 ? d : partials;
  rc = launch_pair<true, true>(mah, mal, mbh, mbl, out, shape,
                                    PlainPairExt{nullptr, inv_scale_a, inv_scale_b, N}, st);
  if (rc != FRNNT_OK) return rc;
  if (splits > 1) {
    const long long n = (long long)M * N;
    FRNNT_KERNEL(ordered_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partials, d, n, splits));
    FRNNT_CUDA(cudaGetLastError());
  }
  return FRNNT_OK;
}
