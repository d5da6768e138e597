// Mutual-information recursion on sm_100a: anti-diagonal wavefront kernels.
//
// What is computed (semantics of the reference's CPU implementation,
// fast_rnnt/csrc/mutual_information_cpu.cu:50-256):
//   forward   p[s0][t0] = 0
//             p[s][t]   = LogAdd(p[s-1][t+o] + px[s-1][t+o], p[s][t-1] + py[s][t-1])
//             (o = 0 regular, -1 modified; out-of-range terms are -inf)
//   backward  d1 = exp(p[s-1][t+o] + px[s-1][t+o] - p[s][t]),  d2 = 1 - d1
//             px_grad[s-1][t+o] = d1 * g[s][t],  py_grad[s][t-1] = d2 * g[s][t]
//             g[s][t] = (x-gradient arriving from row s+1) + (y-gradient from column t+1)
//
// How it is mapped to the GPU (not the reference's tile-per-launch scheme):
//   * one CTA per utterance, ONE launch per sweep;
//   * thread i owns lattice row s0+i; at step k it works on anti-diagonal k
//     (cell (i, k-i)), so the "row above" value arrives by a warp shuffle and the
//     "column before" value stays in a register;
//   * between the last lane of a warp and the first lane of the next the value
//     travels through shared memory.  float: a 64-bit word {step tag, value} per
//     step that the consumer polls (bounded), so the warps run as a pipeline and
//     never meet at a per-step barrier.  double: a value ring plus one named
//     barrier per step among the compute warps;
//   * px / py are re-laid by dedicated loader warps into a skewed shared-memory
//     ring (row i, diagonal k), 32 diagonals per chunk, double buffered: global
//     reads are contiguous row segments, ring reads by the diagonal are
//     bank-conflict free (pitch 33);
//   * the forward sweep stores, by anti-diagonal in a scratch ("lattice", fully
//     coalesced), the exponent of the backward weight of every cell,
//     p[s-1][t+o] + px[s-1][t+o] - p[s][t], which it has in registers anyway.  In
//     the backward sweep the helper warps turn it into the weights d1 (the only
//     exp() of the backward) one chunk ahead of the compute warps, whose
//     dependent chain per step is shuffle + add + multiply;
//   * gradients leave through the same kind of skewed ring, written back as
//     contiguous row segments by the helper warps, which also write the exact
//     zeros outside the boundary box.
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace frnnt {

constexpr int kChunk = 32;      // anti-diagonals staged per chunk
constexpr int kPitch = 33;      // ring row pitch in elements
constexpr int kIoWarps = 4;     // loader warps per CTA of the forward sweep
// helper warps per CTA of the backward sweep (they do the exp()): as many as the register
// file allows next to NCW compute warps
__host__ __device__ constexpr int bwd_io_warps(int ncw) { return ncw <= 4 ? 16 : 8; }
constexpr int kHandRing = 64;   // hand-off slots per warp (two chunks deep)
constexpr int kSpinLimit = 1 << 22;

struct MiBox {
  int s0, t0, sb, tb;  // origin and extents (s_end - s_begin, t_end - t_begin)
};

__device__ __forceinline__ MiBox load_box(const int64_t *boundary, int b, int S, int T) {
  MiBox box{0, 0, S, T};
  if (boundary != nullptr) {
    // clamped so that a malformed row can never index outside the tensors
    int s0 = (int)boundary[4 * b + 0], t0 = (int)boundary[4 * b + 1];
    int s1 = (int)boundary[4 * b + 2], t1 = (int)boundary[4 * b + 3];
    s0 = max(0, min(s0, S));
    t0 = max(0, min(t0, T));
    s1 = max(s0, min(s1, S));
    t1 = max(t0, min(t1, T));
    box = MiBox{s0, t0, s1 - s0, t1 - t0};
  }
  return box;
}

// lattice scratch: the weight exponents by anti-diagonal, [B][S+T+1][pitch]
__host__ __device__ inline int lattice_pitch(int S) { return (S + 1 + 31) & ~31; }
// followed, per utterance, by two vectors of edge_elems() values: when the lattice has
// more rows than one CTA holds it is swept in row blocks (one launch per block); the
// forward sweep passes p of a block's last row, the backward sweep the x-gradients of
// a block's first row, to the next launch through them
__host__ __device__ inline size_t edge_elems(int S, int T) { return (size_t)(S + T + 1 + 2 * kChunk); }
__host__ __device__ inline size_t lattice_elems_per_utt(int S, int T) {
  return (size_t)(S + T + 1) * lattice_pitch(S) + 2 * edge_elems(S, T);
}

__device__ __forceinline__ void bar_sync_named(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- asynchronous global -> shared copies of single elements ---------------------
// (the loader warps keep dozens of these in flight; a plain load + store loop
// would wait a full memory latency per element)
template <typename real>
__device__ __forceinline__ void async_copy_or_zero(real *smem_dst, const real *gsrc, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int src_bytes = valid ? (int)sizeof(real) : 0;  // 0 -> the destination is zero-filled
  if (sizeof(real) == 4)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(gsrc), "r"(src_bytes)
                 : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(gsrc), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void async_copy_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// The chunk barrier releases all compute warps at the same instant, so a consumer warp
// would ask for its neighbour's value of the previous step just before it becomes
// visible -- at every step, since both run at the same pace -- and pay a poll each time.
// Starting each warp a little after the one it depends on keeps the producer ahead.
constexpr int kStaggerCycles = 96;
__device__ __forceinline__ void stagger(int lag) {
  if (lag <= 0) return;
  const long long t0 = clock64();
  while (clock64() - t0 < (long long)lag * kStaggerCycles) {
  }
}

// ---- hand-off between neighbouring warps --------------------------------------
// float: tagged 64-bit slots, polled.  double: plain slots + a barrier per step.
template <typename real> struct Hand;

template <> struct Hand<float> {
  static constexpr bool kBarrier = false;
  using slot_t = unsigned long long;
  static constexpr int kSlotsPerWarp = kHandRing;
  __device__ static void init(volatile slot_t *q, int n, float) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) q[j] = ~0ull;
  }
  __device__ static void put(volatile slot_t *q, int warp, int step, float v) {
    q[warp * kHandRing + (step & (kHandRing - 1))] =
        ((unsigned long long)(unsigned)step << 32) | (unsigned long long)__float_as_uint(v);
  }
  // raw slot of `step`, read early: the consumer issues this one step before it needs
  // the value, so that the shared-memory latency is off its dependent chain
  __device__ static slot_t peek(volatile slot_t *q, int warp, int step) {
    return q[warp * kHandRing + (step & (kHandRing - 1))];
  }
  // value the neighbour published at `step`, starting from an early read of the slot;
  // polls (at most kSpinLimit times) only if that read came too early.
  // Called by ALL lanes of the consumer warp (one broadcast read, no divergence);
  // the neighbour normally runs a step ahead, so the early read succeeds.
  __device__ static float get(volatile slot_t *q, int warp, int step, volatile int *failed,
                              slot_t early) {
    volatile slot_t *slot = q + warp * kHandRing + (step & (kHandRing - 1));
    unsigned long long v = early;
    int spins = 0;
    while ((unsigned)(v >> 32) != (unsigned)step) {
      // one wait that runs out ends all later ones at their first miss
      if (*failed || ++spins > kSpinLimit) {
        *failed = 1;
        break;
      }
      v = *slot;
    }
    return __uint_as_float((unsigned)v);
  }
};

template <> struct Hand<double> {
  static constexpr bool kBarrier = true;
  using slot_t = double;
  static constexpr int kSlotsPerWarp = 4;
  __device__ static void init(volatile slot_t *q, int n, double fill) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) q[j] = fill;
  }
  __device__ static void put(volatile slot_t *q, int warp, int step, double v) {
    q[warp * 4 + (step & 3)] = v;
  }
  __device__ static slot_t peek(volatile slot_t *, int, int) { return 0; }
  __device__ static double get(volatile slot_t *q, int warp, int step, volatile int *, slot_t) {
    return q[warp * 4 + (step & 3)];
  }
};

template <typename real, int NCW>
__host__ __device__ constexpr size_t hand_bytes() {
  return (size_t)NCW * Hand<real>::kSlotsPerWarp * sizeof(typename Hand<real>::slot_t);
}

// -----------------------------------------------------------------------------
// forward
// -----------------------------------------------------------------------------
// BLOCKED: the launch covers lattice rows [row0, row0 + ROWS) only; p of the row above
// the block is read back from the edge vector where the previous launch left it.
template <typename real, int NCW, bool MODIFIED, bool WRITE_P, bool BLOCKED>
__global__ void __launch_bounds__((NCW + kIoWarps) * 32)
mi_forward_kernel(const real *__restrict__ px, const real *__restrict__ py,
                  const int64_t *__restrict__ boundary, real *__restrict__ p,
                  real *__restrict__ ans, real *__restrict__ lattice, int S, int T, int row0_arg) {
  constexpr int ROWS = NCW * 32;
  using H = Hand<real>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  real *ringx = reinterpret_cast<real *>(smem_raw);  // [2][ROWS][kPitch]
  real *ringy = ringx + 2 * ROWS * kPitch;           // [2][ROWS][kPitch]
  real *ringu = ringy + 2 * ROWS * kPitch;           // [2][kPitch]  p of the row above the block
  volatile typename H::slot_t *hand =
      reinterpret_cast<volatile typename H::slot_t *>(ringu + 2 * kPitch);
  __shared__ int failed;
  const int row0 = BLOCKED ? row0_arg : 0;

  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T1 = MODIFIED ? T : T + 1;
  constexpr int off = MODIFIED ? -1 : 0;
  const MiBox box = load_box(boundary, b, S, T);
  // rows of this launch: local row i <-> lattice row row0 + i, i <= ib; local diagonal
  // k = i + t', lattice diagonal row0 + k
  const int ib = min(ROWS - 1, box.sb - row0);
  const int nd = ib >= 0 ? ib + box.tb + 1 : 0;  // anti-diagonals of this launch
  const int nchunks = (nd + kChunk - 1) / kChunk;
  const real *X = px + (size_t)b * S * T1;
  const real *Y = py + (size_t)b * (S + 1) * T;
  real *P = WRITE_P ? p + (size_t)b * (S + 1) * (T + 1) : nullptr;
  const int lpitch = lattice_pitch(S);
  const bool is_io = warp >= NCW;
  const real ninf = neg_inf<real>();
  // edge vectors behind the lattice, indexed by lattice diagonal: this block writes one
  // (p of its last row), the next block reads it
  real *edge = lattice ? lattice + (size_t)b * lattice_elems_per_utt(S, T) + (size_t)(S + T + 1) * lpitch
                       : nullptr;
  const int blk = row0 / ROWS;
  real *edge_out = edge ? edge + (size_t)(blk & 1) * edge_elems(S, T) : nullptr;
  const real *edge_in = edge ? edge + (size_t)((blk + 1) & 1) * edge_elems(S, T) : nullptr;

  H::init(hand, NCW * H::kSlotsPerWarp, ninf);
  if (threadIdx.x == 0) failed = 0;

  // ring[slot][i][j] holds, for consumer cell (row i, diagonal 32c+j):
  //   x = px[s0+i-1][t0+t'+o]   and   y = py[s0+i][t0+t'-1],   t' = 32c+j-i
  auto load_chunk = [&](int c) {
    const int slot = c & 1;
    const int k = c * kChunk + lane;
    for (int i = warp - NCW; i <= ib; i += kIoWarps) {
      const int tp = k - i;
      const bool in_box = tp >= 0 && tp <= box.tb;
      const bool vx = in_box && row0 + i >= 1 && tp + off >= 0;
      const bool vy = in_box && tp >= 1;
      async_copy_or_zero(&ringx[(slot * ROWS + i) * kPitch + lane],
                         vx ? X + (size_t)(box.s0 + row0 + i - 1) * T1 + (box.t0 + tp + off) : X, vx);
      async_copy_or_zero(&ringy[(slot * ROWS + i) * kPitch + lane],
                         vy ? Y + (size_t)(box.s0 + row0 + i) * T + box.t0 + tp - 1 : Y, vy);
    }
    if (BLOCKED && row0 > 0 && warp == NCW) {
      // p of cell (row0 - 1, k + o) of the block above, by lattice diagonal
      const bool v = k + off >= 0 && k + off <= box.tb;
      async_copy_or_zero(&ringu[slot * kPitch + lane], v ? edge_in + (row0 + k - 1 + off) : edge_in, v);
    }
    async_copy_wait_all();
  };

  if (is_io) load_chunk(0);
  __syncthreads();

  const int i = threadIdx.x;          // local lattice row (compute threads only)
  const bool row_ok = i <= ib;
  const bool top_row = row0 + i == 0;
  const int k_first = i, k_last = i + box.tb;  // this row is active for k in [k_first, k_last]
  // this row's cells at t'-1 and t'-2.  Regular recursion: row 0 starts from 0 instead
  // of -inf, so its first cell comes out as LogAdd(-inf, 0 + 0) = 0, the origin, without
  // a special case in the loop (the modified recursion also reads the value of two steps
  // back, where the fake start would leak into row 1, so it keeps the special case).
  real p_cur = (!MODIFIED && top_row) ? (real)0 : ninf, p_old = ninf;
  real p_last = ninf;                 // the last active value (the answer for row sb)
  typename H::slot_t early = 0;       // the neighbour's slot for the next step, read ahead
  real *L = lattice ? lattice + (size_t)b * lattice_elems_per_utt(S, T) + (size_t)row0 * lpitch +
                          row0 + i
                    : nullptr;

  for (int c = 0; c < nchunks; ++c) {
    if (is_io) {
      if (c + 1 < nchunks) load_chunk(c + 1);
    } else {
      if (!H::kBarrier && NCW > 1) stagger(warp);
      const real *rx = ringx + ((c & 1) * ROWS + i) * kPitch;
      const real *ry = ringy + ((c & 1) * ROWS + i) * kPitch;
      const real *ru = ringu + (c & 1) * kPitch;
#pragma unroll 1
      for (int j0 = 0; j0 < kChunk; j0 += 8) {
        real xv[8], yv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          xv[u] = rx[j0 + u];
          yv[u] = ry[j0 + u];
        }
        // the results of the eight steps leave for memory after the batch, so that no
        // store sits between two steps of the dependent chain
        real dlv[8], pv[8];
        unsigned act_mask = 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = c * kChunk + j0 + u;
          // p of the row above: one step back (regular) or two (modified)
          const real hist = MODIFIED ? p_old : p_cur;
          real up = __shfl_up_sync(0xffffffffu, hist, 1);
          if (NCW > 1 && warp > 0) {  // warp-uniform: every lane reads the neighbour's slot
            const int src = k - 1 + off;
            const real nb = src >= 0 ? H::get(hand, warp - 1, src, &failed, early) : ninf;
            if (lane == 0) up = nb;
          }
          if (BLOCKED && row0 > 0 && i == 0) up = k + off >= 0 ? ru[j0 + u] : ninf;
          const bool active = row_ok && k >= k_first && k <= k_last;
          const real a = top_row ? ninf : up + xv[u];
          const real bb = p_cur + yv[u];
          real pn = log_add(a, bb);
          if (MODIFIED && k == 0 && top_row) pn = 0;
          if (!active) pn = ninf;
          p_last = active ? pn : p_last;
          act_mask |= active ? 1u << u : 0u;
          dlv[u] = a - pn;   // exponent of this cell's backward weight
          pv[u] = pn;
          p_old = p_cur;
          p_cur = pn;
          if (NCW > 1) {
            if (lane == 31 && warp + 1 < NCW) H::put(hand, warp, k, pn);
            if (!H::kBarrier && warp > 0) early = H::peek(hand, warp - 1, k + off);  // for step k+1
            if (H::kBarrier) bar_sync_named(1, NCW * 32);
          }
        }
        if (L != nullptr) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (act_mask >> u & 1u) L[(size_t)u * lpitch] = dlv[u];
          L += (size_t)8 * lpitch;
        }
        if (BLOCKED && i == ROWS - 1) {
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (act_mask >> u & 1u) edge_out[row0 + c * kChunk + j0 + u] = pv[u];
        }
        if (WRITE_P) {
          real *prow = P + (size_t)(box.s0 + row0 + i) * (T + 1) + box.t0 + (c * kChunk + j0 - i);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (act_mask >> u & 1u) prow[u] = pv[u];
        }
      }
    }
    __syncthreads();
  }
  if (!is_io && row0 + i == box.sb) ans[b] = failed ? (real)NAN : p_last;
  // a hand-off that ran out in a block that does not hold the last row: NaN in the row
  // it passes down, so that every later block and finally ans[b] turn NaN as well
  if (BLOCKED && failed && edge_out != nullptr)
    for (int k = threadIdx.x; k < nd; k += blockDim.x) edge_out[row0 + k] = (real)NAN;
}

// -----------------------------------------------------------------------------
// backward (from the diagonal-major lattice)
// -----------------------------------------------------------------------------
// px is not read: the lattice holds everything the sweep needs.
// BLOCKED: the launch covers lattice rows [row0, row0 + ROWS) only, blocks run from the
// last to the first.  The x-gradients that the first row of a block sends to the row
// above are left, by lattice diagonal, in one of the two edge vectors behind the
// lattice (alternating from block to block); the next launch stages them for its last row.
template <typename real, int NCW, bool MODIFIED, bool BLOCKED>
__global__ void __launch_bounds__((NCW + bwd_io_warps(NCW)) * 32)
mi_backward_kernel(const real *__restrict__ px, real *__restrict__ lattice,
                   const int64_t *__restrict__ boundary, const real *__restrict__ ans_grad,
                   real *__restrict__ px_grad, real *__restrict__ py_grad,
                   real *__restrict__ origin_grad, int S, int T, int row0_arg) {
  constexpr int ROWS = NCW * 32;
  constexpr int NIO = bwd_io_warps(NCW);
  using H = Hand<real>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  real *ringd = reinterpret_cast<real *>(smem_raw);  // [2][ROWS][kPitch]  px, then d1
  real *ringx = ringd + 2 * ROWS * kPitch;           // [2][ROWS][kPitch]  d/dpx
  real *ringy = ringx + 2 * ROWS * kPitch;           // [2][ROWS][kPitch]  d/dpy
  real *ringb = ringy + 2 * ROWS * kPitch;           // [2][kPitch]  x-gradients from the block below
  volatile typename H::slot_t *hand =
      reinterpret_cast<volatile typename H::slot_t *>(ringb + 2 * kPitch);
  __shared__ int failed;
  const int row0 = BLOCKED ? row0_arg : 0;

  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T1 = MODIFIED ? T : T + 1;
  constexpr int off = MODIFIED ? -1 : 0;
  constexpr int tp_min_x = MODIFIED ? 1 : 0;  // first t' whose cell has an x-predecessor
  const MiBox box = load_box(boundary, b, S, T);
  const int ib = min(ROWS - 1, box.sb - row0);  // last local row of this launch
  const int nd = ib >= 0 ? ib + box.tb + 1 : 0;
  const int nchunks = (nd + kChunk - 1) / kChunk;
  (void)px;
  real *GX = px_grad + (size_t)b * S * T1;
  real *GY = py_grad + (size_t)b * (S + 1) * T;
  const int lpitch = lattice_pitch(S);
  const real *LT = lattice + (size_t)b * lattice_elems_per_utt(S, T);
  // edge vectors, indexed by lattice diagonal: this block writes one, reads the other
  real *edge = lattice + (size_t)b * lattice_elems_per_utt(S, T) + (size_t)(S + T + 1) * lpitch;
  const int blk = row0 / ROWS;
  real *edge_out = edge + (size_t)(blk & 1) * edge_elems(S, T);
  const real *edge_in = edge + (size_t)((blk + 1) & 1) * edge_elems(S, T);
  const bool block_below = BLOCKED && row0 + ROWS <= box.sb;
  const bool is_io = warp >= NCW;

  H::init(hand, NCW * H::kSlotsPerWarp, (real)0);
  if (threadIdx.x == 0) failed = 0;

  // helper warps: weights of chunk c.  lane = row, the weight exponents are read by
  // diagonal (contiguous), all loads of this warp's diagonals in flight before the
  // first exp
  auto weights_chunk = [&](int c) {
    const int slot = c & 1;
    const int iw = warp - NCW;
    if (BLOCKED && iw == 0) {
      // what cell (row0 + ROWS, t' - o) of the block below sent up to the last row's
      // cell (row0 + ROWS - 1, t'), t' = k - (ROWS - 1)
      const int k = c * kChunk + lane;
      const int ts = k - (ROWS - 1) - off;
      const bool v = block_below && ts >= 0 && ts <= box.tb;
      async_copy_or_zero(&ringb[slot * kPitch + lane], v ? edge_in + (row0 + k + 1 - off) : edge_in, v);
      async_copy_wait_all();
    }
    constexpr int NJ = kChunk / NIO;   // diagonals per helper warp
    constexpr int NM = NCW;                 // 32-row blocks
    real dl[NJ][NM];
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      const int k = c * kChunk + iw + jj * NIO;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const int i = lane + 32 * m;
        const int tp = k - i;
        const bool v = row0 + i >= 1 && i <= ib && tp >= 1 && tp <= box.tb;
        dl[jj][m] = v ? LT[(size_t)(row0 + k) * lpitch + row0 + i] : (real)0;
      }
    }
    // the slot still holds gradients that other helper warps are writing out
    // (drain_chunk of two chunks back): wait for all of them, loads in flight
    bar_sync_named(2, NIO * 32);
    // weights of every cell of the chunk, special cases resolved here so that the
    // compute warps only multiply: d1 (share of the x-predecessor) into ringd,
    // d2 (share of the y-predecessor) into the slot of ringx they will overwrite
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      const int j = iw + jj * NIO;
      const int k = c * kChunk + j;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const int i = lane + 32 * m;
        if (i > ib) continue;
        const int tp = k - i;
        real d1 = 0, d2 = 0;
        if (tp >= 0 && tp <= box.tb) {
          if (row0 + i == 0) {     // first row: only a y-predecessor
            d2 = 1;
          } else if (tp == 0) {    // first column: only an x-predecessor (regular) or none
            d1 = MODIFIED ? 0 : 1;
          } else {
            // an unreachable cell has a non-finite exponent; it gets no gradient
            const real w = exp_r(dl[jj][m]);
            if (w - w == 0) {
              d1 = w;
              d2 = (real)1 - w;
            }
          }
        }
        ringd[(slot * ROWS + i) * kPitch + j] = d1;
        ringx[(slot * ROWS + i) * kPitch + j] = d2;
      }
    }
  };

  // cells (row i, diagonal 32c+j) -> px_grad[s0+i-1][t0+t'+o], py_grad[s0+i][t0+t'-1]
  auto drain_chunk = [&](int c) {
    const int slot = c & 1;
    const int k = c * kChunk + lane;
#pragma unroll 4
    for (int i = warp - NCW; i <= ib; i += NIO) {
      const int tp = k - i;
      if (tp <= box.tb) {
        if (row0 + i >= 1 && tp >= tp_min_x)
          GX[(size_t)(box.s0 + row0 + i - 1) * T1 + (box.t0 + tp + off)] =
              ringx[(slot * ROWS + i) * kPitch + lane];
        if (tp >= 1)
          GY[(size_t)(box.s0 + row0 + i) * T + box.t0 + tp - 1] =
              ringy[(slot * ROWS + i) * kPitch + lane];
      }
    }
  };

  if (is_io && nchunks > 0) weights_chunk(nchunks - 1);
  __syncthreads();

  if (is_io && row0 == 0) {
    // exact zeros outside the boundary box (mutual_information_cpu.cu:161-166);
    // overlaps with the compute warps' first chunk
    const int lw = warp - NCW;
    const int cx_lo = box.t0, cx_hi = box.t0 + box.tb + off;  // inclusive, in-box columns of px_grad
    for (int r = lw; r < S; r += NIO) {
      const bool in_rows = r >= box.s0 && r < box.s0 + box.sb;
      for (int col = lane; col < T1; col += 32)
        if (!in_rows || col < cx_lo || col > cx_hi) GX[(size_t)r * T1 + col] = 0;
    }
    const int cy_lo = box.t0, cy_hi = box.t0 + box.tb - 1;
    for (int r = lw; r <= S; r += NIO) {
      const bool in_rows = r >= box.s0 && r <= box.s0 + box.sb;
      for (int col = lane; col < T; col += 32)
        if (!in_rows || col < cy_lo || col > cy_hi) GY[(size_t)r * T + col] = 0;
    }
  }

  const int i = threadIdx.x;
  const bool row_ok = i <= ib;
  real g1_cur = 0, g1_old = 0;  // x-gradients this row sent up at the last two steps
  real g2_cur = 0;              // y-gradient this row sent left at the last step
  real g_last = 0;              // gradient of the cell handled last (the origin for row 0)
  const real g_end = ans_grad[b];
  // local diagonal where the incoming gradient enters (cell (sb, tb))
  const int k_inject = row0 + i == box.sb ? i + box.tb : -1;
  const int k_top = nchunks * kChunk - 1;          // first diagonal the sweep visits
  const bool has_below = NCW > 1 && warp + 1 < NCW;
  typename H::slot_t early = 0;       // the neighbour's slot for the next step, read ahead

  for (int c = nchunks - 1; c >= 0; --c) {
    if (is_io) {
      if (c + 1 < nchunks) drain_chunk(c + 1);
      if (c >= 1) weights_chunk(c - 1);
    } else {
      if (!H::kBarrier && NCW > 1) stagger(NCW - 1 - warp);
      const real *rd = ringd + ((c & 1) * ROWS + i) * kPitch;
      real *rx = ringx + ((c & 1) * ROWS + i) * kPitch;
      real *ry = ringy + ((c & 1) * ROWS + i) * kPitch;
      const real *rb = ringb + (c & 1) * kPitch;
#pragma unroll 1
      for (int j0 = kChunk - 8; j0 >= 0; j0 -= 8) {
        real d1v[8], d2v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          d1v[u] = row_ok ? rd[j0 + u] : (real)0;
          d2v[u] = row_ok ? rx[j0 + u] : (real)0;
        }
#pragma unroll
        for (int u = 7; u >= 0; --u) {
          const int k = c * kChunk + j0 + u;
          const real hist = MODIFIED ? g1_old : g1_cur;
          real below = __shfl_down_sync(0xffffffffu, hist, 1);
          if (has_below) {  // warp-uniform: every lane reads the neighbour's slot
            const int src = k + 1 - off;
            const real nb = src <= k_top ? H::get(hand, warp + 1, src, &failed, early) : (real)0;
            if (lane == 31) below = nb;
          } else if (lane == 31) {
            below = BLOCKED ? rb[j0 + u] : (real)0;
          }
          real g = below + g2_cur;
          if (k == k_inject) g = g_end;
          const real g1 = d1v[u] * g, g2 = d2v[u] * g;
          rx[j0 + u] = g1;
          ry[j0 + u] = g2;
          g_last = g;
          g1_old = g1_cur;
          g1_cur = g1;
          g2_cur = g2;
          if (BLOCKED && row0 > 0 && i == 0 && k < nd) edge_out[row0 + k] = g1;
          if (NCW > 1) {
            if (lane == 0 && warp > 0) H::put(hand, warp, k, g1);
            if (!H::kBarrier && has_below) early = H::peek(hand, warp + 1, k - off);  // for step k-1
            if (H::kBarrier) bar_sync_named(1, NCW * 32);
          }
        }
      }
    }
    __syncthreads();
  }
  if (!is_io && row0 + i == 0 && origin_grad != nullptr) origin_grad[b] = g_last;
  if (is_io && nchunks > 0) drain_chunk(0);
  __syncthreads();
  // a hand-off that ran out: the gradients of this launch are wrong.  Say so in an
  // output that every caller has -- NaN in the first gradient entry of this launch's
  // rows inside the box -- and in origin_grad when it was asked for; the gradients a
  // block passes up turn NaN too, so that the launch that holds row 0 (the last one,
  // which writes origin_grad) sees the failure of an earlier one
  if (BLOCKED && failed && row0 > 0)
    for (int k = threadIdx.x; k < nd; k += blockDim.x) edge_out[row0 + k] = (real)NAN;
  if (failed && threadIdx.x == 0) {
    if (ib >= 0 && box.tb >= 1)
      GY[(size_t)(box.s0 + row0) * T + box.t0] = (real)NAN;
    else if (ib >= 0 && row0 < box.sb)
      GX[(size_t)(box.s0 + row0) * T1 + box.t0] = (real)NAN;
    if (origin_grad != nullptr) origin_grad[b] = (real)NAN;
  }
}

// -----------------------------------------------------------------------------
// Backward sweep with four rows per thread (float, lattices of 33 .. 128 rows)
// -----------------------------------------------------------------------------
// The same reverse sweep with ONE compute warp: lane l owns lattice rows 4l .. 4l+3.  A
// step then advances four cells per thread -- independent of each other, so their
// multiply-add chains overlap in the pipeline -- and the only neighbour value that has to
// travel is the one between a thread's outer rows, one warp shuffle per step.  No value
// crosses a warp boundary, so the tagged shared-memory hand-off of the row-per-thread
// kernel (a third of its step time) is gone: 88 -> 68 us on a 64 x (100, 500) batch.  The
// arithmetic per cell is unchanged, so results are bit-identical to that kernel.  (The
// forward sweep does not profit: a LogAdd is ~100 instructions, so four per thread make one
// warp issue-bound at ~750 cycles per step against ~370 for the row-per-thread kernel:
// 0.24 ms instead of 0.12 ms, measured; its variant was dropped.)
constexpr int kRpt = 4;
constexpr int kRptRows = 32 * kRpt;
constexpr int kRptBatch = 4;  // steps whose weights are fetched together

template <bool MODIFIED>
__global__ void __launch_bounds__((1 + bwd_io_warps(kRpt)) * 32)
mi_backward_rpt_kernel(float *__restrict__ lattice, const int64_t *__restrict__ boundary,
                       const float *__restrict__ ans_grad, float *__restrict__ px_grad,
                       float *__restrict__ py_grad, float *__restrict__ origin_grad, int S, int T) {
  constexpr int ROWS = kRptRows;
  constexpr int NIO = bwd_io_warps(kRpt);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float *ringd = reinterpret_cast<float *>(smem_raw);  // [2][ROWS][kPitch]  d1
  float *ringx = ringd + 2 * ROWS * kPitch;            // [2][ROWS][kPitch]  d2, then d/dpx
  float *ringy = ringx + 2 * ROWS * kPitch;            // [2][ROWS][kPitch]  d/dpy

  const int b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int T1 = MODIFIED ? T : T + 1;
  constexpr int off = MODIFIED ? -1 : 0;
  constexpr int tp_min_x = MODIFIED ? 1 : 0;
  const MiBox box = load_box(boundary, b, S, T);
  const int ib = min(ROWS - 1, box.sb);
  const int nd = ib + box.tb + 1;
  const int nchunks = (nd + kChunk - 1) / kChunk;
  float *GX = px_grad + (size_t)b * S * T1;
  float *GY = py_grad + (size_t)b * (S + 1) * T;
  const int lpitch = lattice_pitch(S);
  const float *LT = lattice + (size_t)b * lattice_elems_per_utt(S, T);
  const bool is_io = warp >= 1;

  // helper warps: weights of chunk c (lane = row within a block of 32, diagonals by warp)
  auto weights_chunk = [&](int c) {
    const int slot = c & 1;
    const int iw = warp - 1;
    constexpr int NJ = kChunk / NIO;
    constexpr int NM = kRpt;
    float dl[NJ][NM];
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      const int k = c * kChunk + iw + jj * NIO;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const int i = lane + 32 * m;
        const int tp = k - i;
        const bool v = i >= 1 && i <= ib && tp >= 1 && tp <= box.tb;
        dl[jj][m] = v ? LT[(size_t)k * lpitch + i] : 0.f;
      }
    }
    bar_sync_named(2, NIO * 32);
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) {
      const int j = iw + jj * NIO;
      const int k = c * kChunk + j;
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const int i = lane + 32 * m;
        if (i > ib) continue;
        const int tp = k - i;
        float d1 = 0, d2 = 0;
        if (tp >= 0 && tp <= box.tb) {
          if (i == 0) {
            d2 = 1;
          } else if (tp == 0) {
            d1 = MODIFIED ? 0 : 1;
          } else {
            const float w = exp_r(dl[jj][m]);
            if (w - w == 0) {
              d1 = w;
              d2 = 1.f - w;
            }
          }
        }
        ringd[(slot * ROWS + i) * kPitch + j] = d1;
        ringx[(slot * ROWS + i) * kPitch + j] = d2;
      }
    }
  };

  auto drain_chunk = [&](int c) {
    const int slot = c & 1;
    const int k = c * kChunk + lane;
#pragma unroll 4
    for (int i = warp - 1; i <= ib; i += NIO) {
      const int tp = k - i;
      if (tp <= box.tb) {
        if (i >= 1 && tp >= tp_min_x)
          GX[(size_t)(box.s0 + i - 1) * T1 + (box.t0 + tp + off)] = ringx[(slot * ROWS + i) * kPitch + lane];
        if (tp >= 1) GY[(size_t)(box.s0 + i) * T + box.t0 + tp - 1] = ringy[(slot * ROWS + i) * kPitch + lane];
      }
    }
  };

  if (is_io && nchunks > 0) weights_chunk(nchunks - 1);
  __syncthreads();

  if (is_io) {
    // exact zeros outside the boundary box (mutual_information_cpu.cu:161-166)
    const int lw = warp - 1;
    const int cx_lo = box.t0, cx_hi = box.t0 + box.tb + off;
    for (int r = lw; r < S; r += NIO) {
      const bool in_rows = r >= box.s0 && r < box.s0 + box.sb;
      for (int col = lane; col < T1; col += 32)
        if (!in_rows || col < cx_lo || col > cx_hi) GX[(size_t)r * T1 + col] = 0;
    }
    const int cy_lo = box.t0, cy_hi = box.t0 + box.tb - 1;
    for (int r = lw; r <= S; r += NIO) {
      const bool in_rows = r >= box.s0 && r <= box.s0 + box.sb;
      for (int col = lane; col < T; col += 32)
        if (!in_rows || col < cy_lo || col > cy_hi) GY[(size_t)r * T + col] = 0;
    }
  }

  const int i0 = lane * kRpt;
  float g1_cur[kRpt], g1_old[kRpt], g2_cur[kRpt];
  int k_inject[kRpt];
#pragma unroll
  for (int j = 0; j < kRpt; ++j) {
    g1_cur[j] = g1_old[j] = g2_cur[j] = 0.f;
    k_inject[j] = i0 + j == box.sb ? i0 + j + box.tb : -1;
  }
  float g_last = 0;  // gradient of row 0's last cell: what reaches the origin
  const float g_end = ans_grad[b];

  for (int c = nchunks - 1; c >= 0; --c) {
    if (is_io) {
      if (c + 1 < nchunks) drain_chunk(c + 1);
      if (c >= 1) weights_chunk(c - 1);
    } else {
#pragma unroll 1
      for (int j0 = kChunk - kRptBatch; j0 >= 0; j0 -= kRptBatch) {
        float d1v[kRpt][kRptBatch], d2v[kRpt][kRptBatch];
#pragma unroll
        for (int j = 0; j < kRpt; ++j) {
          const bool row_ok = i0 + j <= ib;
          const float *rd = ringd + ((c & 1) * ROWS + i0 + j) * kPitch + j0;
          const float *rx = ringx + ((c & 1) * ROWS + i0 + j) * kPitch + j0;
#pragma unroll
          for (int u = 0; u < kRptBatch; ++u) {
            d1v[j][u] = row_ok ? rd[u] : 0.f;
            d2v[j][u] = row_ok ? rx[u] : 0.f;
          }
        }
#pragma unroll
        for (int u = kRptBatch - 1; u >= 0; --u) {
          const int k = c * kChunk + j0 + u;
          float hist[kRpt];
#pragma unroll
          for (int j = 0; j < kRpt; ++j) hist[j] = MODIFIED ? g1_old[j] : g1_cur[j];
          float from_below = __shfl_down_sync(0xffffffffu, hist[0], 1);
          if (lane == 31) from_below = 0.f;
          float n1[kRpt], n2[kRpt];
#pragma unroll
          for (int j = 0; j < kRpt; ++j) {
            const float below = j == kRpt - 1 ? from_below : hist[j + 1];
            float g = below + g2_cur[j];
            if (k == k_inject[j]) g = g_end;
            n1[j] = d1v[j][u] * g;
            n2[j] = d2v[j][u] * g;
            if (j == 0 && lane == 0) g_last = g;
          }
#pragma unroll
          for (int j = 0; j < kRpt; ++j) {
            ringx[((c & 1) * ROWS + i0 + j) * kPitch + j0 + u] = n1[j];
            ringy[((c & 1) * ROWS + i0 + j) * kPitch + j0 + u] = n2[j];
            g1_old[j] = g1_cur[j];
            g1_cur[j] = n1[j];
            g2_cur[j] = n2[j];
          }
        }
      }
    }
    __syncthreads();
  }
  if (!is_io && lane == 0 && origin_grad != nullptr) origin_grad[b] = g_last;
  if (is_io && nchunks > 0) drain_chunk(0);
}

// p in the reference's [B][S+1][T+1] layout -> the weight exponents
// p[s-1][t+o] + px[s-1][t+o] - p[s][t] in the diagonal-major scratch
template <typename real>
__global__ void mi_lattice_from_p_kernel(const real *__restrict__ p, const real *__restrict__ px,
                                         const int64_t *__restrict__ boundary,
                                         real *__restrict__ lattice, int S, int T, int modified) {
  const int b = blockIdx.y;
  const MiBox box = load_box(boundary, b, S, T);
  const int T1 = modified ? T : T + 1, off = modified ? -1 : 0;
  const real *P = p + (size_t)b * (S + 1) * (T + 1);
  const real *X = px + (size_t)b * S * T1;
  const int lpitch = lattice_pitch(S);
  real *LT = lattice + (size_t)b * lattice_elems_per_utt(S, T);
  const int ncell = (box.sb + 1) * (box.tb + 1);
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < ncell;
       idx += gridDim.x * blockDim.x) {
    const int i = idx / (box.tb + 1), tp = idx % (box.tb + 1);
    real d = 0;  // first row / first column: the weights are fixed by position
    if (i >= 1 && tp >= 1) {
      const size_t up = (size_t)(box.s0 + i - 1);
      d = P[up * (T + 1) + box.t0 + tp + off] + X[up * T1 + box.t0 + tp + off] -
          P[(size_t)(box.s0 + i) * (T + 1) + box.t0 + tp];
    }
    LT[(size_t)(i + tp) * lpitch + i] = d;
  }
}

// -----------------------------------------------------------------------------
// host side
// -----------------------------------------------------------------------------
template <typename real, int NCW>
static size_t mi_smem_bytes(int rings) {
  return (size_t)(rings * 2 * NCW * 32 + 2) * kPitch * sizeof(real) + hand_bytes<real, NCW>();
}

// lattice rows one CTA holds: 8 warps of float rows, 4 of double (the three rings of
// the backward sweep fill shared memory beyond that)
static int mi_rows_per_block(int dtype) { return (dtype == FRNNT_F64 ? 4 : 8) * 32; }

template <typename real, int NCW, bool MODIFIED, bool WRITE_P, bool BLOCKED>
static int launch_forward_p(const void *px, const void *py, const int64_t *boundary, void *p,
                            void *ans, void *lattice, int B, int S, int T, int row0,
                            cudaStream_t st) {
  auto kern = mi_forward_kernel<real, NCW, MODIFIED, WRITE_P, BLOCKED>;
  const size_t smem = mi_smem_bytes<real, NCW>(2);
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  FRNNT_KERNEL(kern<<<B, (NCW + kIoWarps) * 32, smem, st>>>((const real *)px, (const real *)py,
                                                            boundary, (real *)p, (real *)ans,
                                                            (real *)lattice, S, T, row0));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

template <typename real, int NCW, bool MODIFIED>
static int launch_forward(const void *px, const void *py, const int64_t *boundary, void *p,
                          void *ans, void *lattice, int B, int S, int T, cudaStream_t st) {
  if (p != nullptr)
    return launch_forward_p<real, NCW, MODIFIED, true, false>(px, py, boundary, p, ans, lattice, B,
                                                              S, T, 0, st);
  return launch_forward_p<real, NCW, MODIFIED, false, false>(px, py, boundary, p, ans, lattice, B,
                                                             S, T, 0, st);
}

// more rows than one CTA holds: one launch per block of rows, top to bottom
template <typename real, bool MODIFIED>
static int launch_forward_blocked(const void *px, const void *py, const int64_t *boundary, void *p,
                                  void *ans, void *lattice, int B, int S, int T, cudaStream_t st) {
  constexpr int NCW = sizeof(real) == 8 ? 4 : 8;
  for (int row0 = 0; row0 <= S; row0 += NCW * 32) {
    const int rc = p != nullptr
                       ? launch_forward_p<real, NCW, MODIFIED, true, true>(
                             px, py, boundary, p, ans, lattice, B, S, T, row0, st)
                       : launch_forward_p<real, NCW, MODIFIED, false, true>(
                             px, py, boundary, p, ans, lattice, B, S, T, row0, st);
    if (rc != FRNNT_OK) return rc;
  }
  return FRNNT_OK;
}

template <typename real, int NCW, bool MODIFIED, bool BLOCKED>
static int launch_backward_b(const void *px, void *lattice, const int64_t *boundary,
                             const void *ans_grad, void *px_grad, void *py_grad,
                             void *origin_grad, int B, int S, int T, int row0, cudaStream_t st) {
  auto kern = mi_backward_kernel<real, NCW, MODIFIED, BLOCKED>;
  const size_t smem = mi_smem_bytes<real, NCW>(3);
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  FRNNT_KERNEL(kern<<<B, (NCW + bwd_io_warps(NCW)) * 32, smem, st>>>(
      (const real *)px, (real *)lattice, boundary, (const real *)ans_grad, (real *)px_grad,
      (real *)py_grad, (real *)origin_grad, S, T, row0));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

template <typename real, int NCW, bool MODIFIED>
static int launch_backward(const void *px, void *lattice, const int64_t *boundary,
                           const void *ans_grad, void *px_grad, void *py_grad, void *origin_grad,
                           int B, int S, int T, cudaStream_t st) {
  return launch_backward_b<real, NCW, MODIFIED, false>(px, lattice, boundary, ans_grad, px_grad,
                                                       py_grad, origin_grad, B, S, T, 0, st);
}

// one launch per block of rows, bottom to top
template <typename real, bool MODIFIED>
static int launch_backward_blocked(const void *px, void *lattice, const int64_t *boundary,
                                   const void *ans_grad, void *px_grad, void *py_grad,
                                   void *origin_grad, int B, int S, int T, cudaStream_t st) {
  constexpr int NCW = sizeof(real) == 8 ? 4 : 8;
  constexpr int ROWS = NCW * 32;
  for (int row0 = (S / ROWS) * ROWS; row0 >= 0; row0 -= ROWS) {
    const int rc = launch_backward_b<real, NCW, MODIFIED, true>(
        px, lattice, boundary, ans_grad, px_grad, py_grad, origin_grad, B, S, T, row0, st);
    if (rc != FRNNT_OK) return rc;
  }
  return FRNNT_OK;
}

// float lattices of 33 .. 128 rows: the four-rows-per-thread reverse sweep
template <bool MODIFIED>
static int launch_backward_rpt(const void *px, void *lattice, const int64_t *boundary, const void *ans_grad,
                               void *px_grad, void *py_grad, void *origin_grad, int B, int S, int T,
                               cudaStream_t st) {
  (void)px;
  auto kern = mi_backward_rpt_kernel<MODIFIED>;
  const size_t smem = (size_t)(3 * 2 * kRptRows) * kPitch * sizeof(float);
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  FRNNT_KERNEL(kern<<<B, (1 + bwd_io_warps(kRpt)) * 32, smem, st>>>((float *)lattice, boundary,
                                                                   (const float *)ans_grad, (float *)px_grad,
                                                                   (float *)py_grad, (float *)origin_grad, S, T));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

static bool mi_use_rpt(int dtype, int ncw) {
  if (dtype != FRNNT_F32 || ncw < 2 || ncw > kRpt) return false;
  const char *mode = getenv("FRNNT_MI");
  return !(mode != nullptr && strcmp(mode, "row_per_thread") == 0);
}

#define MI_DISPATCH_NCW(FN, real, MOD, ncw, ...)                          \
  switch (ncw) {                                                          \
    case 1: return FN<real, 1, MOD>(__VA_ARGS__);                         \
    case 2: return FN<real, 2, MOD>(__VA_ARGS__);                         \
    case 3: return FN<real, 3, MOD>(__VA_ARGS__);                         \
    case 4: return FN<real, 4, MOD>(__VA_ARGS__);                         \
    case 5: return FN<real, 5, MOD>(__VA_ARGS__);                         \
    case 6: return FN<real, 6, MOD>(__VA_ARGS__);                         \
    case 7: return FN<real, 7, MOD>(__VA_ARGS__);                         \
    case 8: return FN<real, 8, MOD>(__VA_ARGS__);                         \
    default: return FN##_blocked<real, MOD>(__VA_ARGS__);                 \
  }

#define MI_DISPATCH_NCW_F64(FN, MOD, ncw, ...)                            \
  switch (ncw) {                                                          \
    case 1: return FN<double, 1, MOD>(__VA_ARGS__);                       \
    case 2: return FN<double, 2, MOD>(__VA_ARGS__);                       \
    case 3: return FN<double, 3, MOD>(__VA_ARGS__);                       \
    case 4: return FN<double, 4, MOD>(__VA_ARGS__);                       \
    default: return FN##_blocked<double, MOD>(__VA_ARGS__);               \
  }

#define MI_DISPATCH(FN, dtype, modified, ncw, ...)                        \
  do {                                                                    \
    if ((dtype) == FRNNT_F32) {                                           \
      if (modified) { MI_DISPATCH_NCW(FN, float, true, ncw, __VA_ARGS__) }  \
      else { MI_DISPATCH_NCW(FN, float, false, ncw, __VA_ARGS__) }          \
    } else {                                                              \
      if (modified) { MI_DISPATCH_NCW_F64(FN, true, ncw, __VA_ARGS__) }   \
      else { MI_DISPATCH_NCW_F64(FN, false, ncw, __VA_ARGS__) }           \
    }                                                                     \
  } while (0)

// *ncw = compute warps of the single launch that holds the whole lattice, or 0 when
// the lattice has more rows than that and is swept in row blocks
static int mi_check_sizes(int dtype, int B, int S, int T, int modified, int *ncw) {
  FRNNT_REQUIRE(check_dtype(dtype), FRNNT_EINVAL, "dtype must be FRNNT_F32 or FRNNT_F64, got %d",
                dtype);
  FRNNT_REQUIRE(B >= 0 && S >= 0 && T >= 0, FRNNT_EINVAL, "negative size B=%d S=%d T=%d", B, S, T);
  FRNNT_REQUIRE(modified == 0 || modified == 1, FRNNT_EINVAL, "modified must be 0 or 1");
  *ncw = S + 1 <= mi_rows_per_block(dtype) ? (S + 1 + 31) / 32 : 0;
  return FRNNT_OK;
}

// -----------------------------------------------------------------------------
// scratch for the entry point that allocates nothing
// -----------------------------------------------------------------------------
// A fixed region of device memory that belongs to the library image: it exists
// on every GPU whose context loads the library, from load until the process
// ends.  Host code may not use the symbol as a pointer (on the host it is only
// a stand-in); its device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_mi_static_scratch[FRNNT_MI_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void *g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the CURRENT device (looked up on the
// first call per device, with that device current).
static int static_scratch_address(void **out) {
  int dev = -1;
  FRNNT_CUDA(cudaGetDevice(&dev));
  FRNNT_REQUIRE(dev >= 0 && dev < kMaxDevices, FRNNT_EUNSUPPORTED, "device index %d too large", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void *ptr = nullptr;
    FRNNT_CUDA(cudaGetSymbolAddress(&ptr, g_mi_static_scratch));
    FRNNT_REQUIRE(ptr != nullptr, FRNNT_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return FRNNT_OK;
}

}  // namespace frnnt

using namespace frnnt;

extern "C" int frnnt_mi_rows_per_block(int dtype) {
  return check_dtype(dtype) ? mi_rows_per_block(dtype) : 0;
}

extern "C" size_t frnnt_mi_lattice_bytes(int dtype, int B, int S, int T) {
  if (!check_dtype(dtype) || B < 0 || S < 0 || T < 0) return 0;
  return (size_t)B * lattice_elems_per_utt(S, T) * dtype_size(dtype);
}

extern "C" int frnnt_mi_forward(int dtype, const void *px, const void *py,
                                const int64_t *boundary, void *p, void *ans, void *lattice, int B,
                                int S, int T, int modified, void *stream) {
  int ncw = 0;
  int rc = mi_check_sizes(dtype, B, S, T, modified, &ncw);
  if (rc != FRNNT_OK) return rc;
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(ans != nullptr, FRNNT_EINVAL, "ans is NULL");
  FRNNT_REQUIRE((px != nullptr || S == 0 || (modified && T == 0)) && (py != nullptr || T == 0),
                FRNNT_EINVAL, "px or py is NULL");
  FRNNT_REQUIRE(ncw != 0 || lattice != nullptr, FRNNT_EINVAL,
                "S+1=%d exceeds frnnt_mi_rows_per_block(): the sweep runs in row blocks and needs "
                "the lattice scratch",
                S + 1);
  cudaStream_t st = (cudaStream_t)stream;
  MI_DISPATCH(launch_forward, dtype, modified, ncw, px, py, boundary, p, ans, lattice, B, S, T, st);
  return FRNNT_OK;
}

extern "C" int frnnt_mi_backward_from_lattice(int dtype, const void *px, void *lattice,
                                              const int64_t *boundary, const void *ans_grad,
                                              void *px_grad, void *py_grad, void *origin_grad,
                                              int B, int S, int T, int modified, void *stream) {
  int ncw = 0;
  int rc = mi_check_sizes(dtype, B, S, T, modified, &ncw);
  if (rc != FRNNT_OK) return rc;
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(lattice != nullptr && ans_grad != nullptr, FRNNT_EINVAL,
                "lattice or ans_grad is NULL");
  FRNNT_REQUIRE((px_grad != nullptr || S == 0 || (modified && T == 0)) &&
                    (py_grad != nullptr || T == 0),
                FRNNT_EINVAL, "px_grad or py_grad is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (mi_use_rpt(dtype, ncw))
    return modified ? launch_backward_rpt<true>(px, lattice, boundary, ans_grad, px_grad, py_grad, origin_grad,
                                                B, S, T, st)
                    : launch_backward_rpt<false>(px, lattice, boundary, ans_grad, px_grad, py_grad, origin_grad,
                                                 B, S, T, st);
  MI_DISPATCH(launch_backward, dtype, modified, ncw, px, lattice, boundary, ans_grad, px_grad,
              py_grad, origin_grad, B, S, T, st);
  return FRNNT_OK;
}

extern "C" int frnnt_mi_backward(int dtype, const void *px, const void *py,
                                 const int64_t *boundary, const void *p, const void *ans_grad,
                                 void *px_grad, void *py_grad, void *origin_grad, void *lattice,
                                 int B, int S, int T, int modified, void *stream) {
  (void)py;
  int ncw = 0;
  int rc = mi_check_sizes(dtype, B, S, T, modified, &ncw);
  if (rc != FRNNT_OK) return rc;
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(p != nullptr && lattice != nullptr, FRNNT_EINVAL, "p or lattice is NULL");
  FRNNT_REQUIRE(px != nullptr || S == 0 || (modified && T == 0), FRNNT_EINVAL, "px is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)min(64, ((S + 1) * (T + 1) + 255) / 256), (unsigned)B);
  if (dtype == FRNNT_F32)
    FRNNT_KERNEL(mi_lattice_from_p_kernel<float><<<grid, 256, 0, st>>>(
        (const float *)p, (const float *)px, boundary, (float *)lattice, S, T, modified));
  else
    FRNNT_KERNEL(mi_lattice_from_p_kernel<double><<<grid, 256, 0, st>>>(
        (const double *)p, (const double *)px, boundary, (double *)lattice, S, T, modified));
  FRNNT_CUDA(cudaGetLastError());
  return frnnt_mi_backward_from_lattice(dtype, px, lattice, boundary, ans_grad, px_grad, py_grad,
                                        origin_grad, B, S, T, modified, stream);
}

extern "C" int frnnt_mi_fwd_bwd_noalloc(int dtype, const void *px, const void *py,
                                        const int64_t *boundary, const void *ans_grad, void *ans,
                                        void *px_grad, void *py_grad, int B, int S, int T,
                                        int modified, void *stream) {
  int ncw = 0;
  int rc = mi_check_sizes(dtype, B, S, T, modified, &ncw);
  if (rc != FRNNT_OK) return rc;
  const size_t need = frnnt_mi_lattice_bytes(dtype, B, S, T);
  FRNNT_REQUIRE(need <= (size_t)FRNNT_MI_NOALLOC_SCRATCH_BYTES, FRNNT_EUNSUPPORTED,
                "lattice B=%d S=%d T=%d needs %zu bytes of scratch, the built-in region holds %zu; "
                "use frnnt_mi_forward + frnnt_mi_backward_from_lattice with your own buffer",
                B, S, T, need, (size_t)FRNNT_MI_NOALLOC_SCRATCH_BYTES);
  if (B == 0) return FRNNT_OK;
  FRNNT_REQUIRE(ans != nullptr && ans_grad != nullptr, FRNNT_EINVAL, "ans or ans_grad is NULL");
  // everything either sweep would refuse is refused here, before the first launch
  FRNNT_REQUIRE((px != nullptr || S == 0 || (modified && T == 0)) && (py != nullptr || T == 0),
                FRNNT_EINVAL, "px or py is NULL");
  FRNNT_REQUIRE((px_grad != nullptr || S == 0 || (modified && T == 0)) &&
                    (py_grad != nullptr || T == 0),
                FRNNT_EINVAL, "px_grad or py_grad is NULL");
  void *scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != FRNNT_OK) return rc;
  // Nothing in the region has to start at zero: the forward sweep writes every
  // lattice value that the backward sweep reads, so the previous call's contents
  // are simply overwritten.
  rc = frnnt_mi_forward(dtype, px, py, boundary, nullptr, ans, scratch, B, S, T, modified, stream);
  if (rc != FRNNT_OK) return rc;
  return frnnt_mi_backward_from_lattice(dtype, px, scratch, boundary, ans_grad, px_grad, py_grad,
                                        nullptr, B, S, T, modified, stream);
}
