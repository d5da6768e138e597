// The second tensor-core product engine of this library (sm_100a): D = A * B^T-like
// products whose operands are already stored as PAIRS OF HALF-PRECISION PLANES,
// x * 2^e ~= hi + lo with hi = fp16(x * 2^e) and lo = fp16(x * 2^e - hi).  An fp16 value
// carries an 11-bit significand like a tf32 value, so hi*hi + hi*lo + lo*hi has the
// accuracy of the 3xTF32 scheme (22 bits per operand) -- but kind::f16 MMAs run at twice
// the tf32 rate on half the operand bytes, and because the producers of the operands
// (the tanh kernel, the log-softmax backward, a small pass over the weights) write the
// planes themselves, nothing has to be split inside this kernel: it is a pure
// TMA -> tcgen05.mma pipeline with both operands read from shared memory.
//
// fp16 has a 5-bit exponent; the power-of-two scale 2^e of every operand is chosen by
// its producer so that the largest magnitude lands in [2^14, 2^15).  Values down to
// 2^-18 of the largest keep all 22 bits, smaller ones an absolute error of 2^-40 of the
// largest (see fp16_pair()).  The scales are undone in the epilogue (exactly).
//
// Kernel structure (one 128x128 output tile per work item, 10 warps, one persistent CTA
// per SM):
//   warp 0   : TMA producer.  Per 64-wide K slice four 16 KB boxes (A hi, A lo, B hi, B lo)
//              land in 128-byte-swizzled tiles; 3-stage ring; rows / columns outside the
//              matrices arrive as zeros.  K-major operands (rows = M or N index): one box
//              of 64 k x 128 rows.  Operands that are contiguous along M / N (rows = k
//              index): two boxes of 64 values x 64 k rows.
//   warp 1   : one thread issues, per K = 16 step, hi*hi, hi*lo, lo*hi into a 128x128 fp32
//              accumulator in tensor memory.  The tensor core adds into its accumulator
//              with truncation, so every 128-wide K group gets a fresh accumulator (two
//              alternate) and
//   warps 2-9: two sets of four fold / epilogue warps, one set per tile in turn.  A set
//              folds the finished groups of its tile into its own running sum in tensor
//              memory with round-to-nearest adds (tcgen05.ld / add / tcgen05.st), which
//              frees the accumulator at once, and then runs the epilogue from the running
//              sum -- policy, 32x32 boxes staged in shared memory, TMA stores -- while the
//              other set already folds the next tile: the epilogue has a whole tile's
//              time and never holds an accumulator.
// One CTA per SM, every load is a plain per-CTA TMA load.  Every wait is bounded; a timeout poisons the tile with NaN.
//
// Policy ("Ext") interface, all __device__:
//   static constexpr bool kBatched;                the work-item index z is a batch index (the
//                                                  outer coordinate of every tensor map) instead
//                                                  of a split of the reduction
//   static constexpr bool kCustomStore;            the policy writes the result itself:
//                                                  store_box() is called instead of finish(),
//                                                  staging and the TMA store, for the 32-column
//                                                  boxes of a tile from the last to the first
//   struct Row;                                    per-row state across one tile's columns
//   void row_begin(Row &, int z, int m, int n0) const;
//   void prefetch(Row &, int z, int m, int n) const;      columns n..n+31 come next: loads
//                                                  the policy needs for them may start
//   void finish(Row &, int z, int m, int n, float (&v)[16], int half) const;   columns
//                                                  n..n+15 of row m (half = 0 / 1 of the
//                                                  prefetched 32), in place; only columns
//                                                  below N count
//   void row_end(Row &, int z, int m, int n0) const;
//   void tile_begin(int z, int n0, uint8_t *box, int lane) const;   (kCustomStore) called by
//                                                  all lanes of a fold warp when it takes a
//                                                  tile: 4 KB of shared memory per warp for
//                                                  per-column data
//   void store_box(Row &, int z, int m, int n0, int c0, float (&v0)[16], float (&v1)[16],
//                  const uint8_t *box) const;      (kCustomStore) columns n0+c0..n0+c0+31 of row m < M
// The result goes out through a tensor map of the output (rows beyond M and columns
// beyond N are clipped by the TMA store).
#pragma once
#include <cuda_fp16.h>

#include "umma_linear.cuh"

namespace frnnt {

constexpr int kPairThreads = 320;  // TMA warp, MMA warp, 2 x 4 fold / epilogue warps
constexpr int kPairFolders = 4;    // warps of one set
constexpr int kPairTile = 128;
constexpr int kPairBK = 64;        // K slice: 128 bytes of fp16 per row
constexpr int kPairStages = 3;
constexpr int kPairGroup = 2;      // K slices per accumulator group (128 values of K)
constexpr uint32_t kPairOpBytes = kPairTile * 128;       // one plane of one operand tile
constexpr uint32_t kPairStageBytes = 4 * kPairOpBytes;   // A hi, A lo, B hi, B lo
constexpr uint32_t kPairBoxBytes = 32 * 128;             // a 32 x 32 float box of the output
constexpr size_t kPairSmemBytes = (size_t)kPairStages * kPairStageBytes + 8 * kPairBoxBytes + 1024;
// tensor-memory columns: two group accumulators, one running sum per fold set
constexpr uint32_t kPairCols = 512, kPairAcc1 = 128, kPairRun = 256;

// x * scale as a pair of fp16 values.  |x * scale| must stay below 65504.  hi has 11
// significant bits; lo = fp16(x * scale - hi) is exact to 11 more bits while it is a
// normal fp16 number (|x * scale| >= 2^-3), below that to half a subnormal step, 2^-25.
__device__ __forceinline__ void fp16_pair(float x, float scale, __half &hi, __half &lo) {
  const float xs = x * scale;
  hi = __float2half_rn(xs);
  lo = __float2half_rn(xs - __half2float(hi));
}

// two values at once, same results: the conversions to fp16 are packed (one instruction per
// pair instead of one per value; the unpacked conversion shares the special-function pipe,
// a quarter of the issue rate, with exp and tanh)
__device__ __forceinline__ void fp16_pair2(float x0, float x1, float scale, __half2 &hi, __half2 &lo) {
  const float a = x0 * scale, b = x1 * scale;
  hi = __floats2half2_rn(a, b);
  const float2 h = __half22float2(hi);
  lo = __floats2half2_rn(a - h.x, b - h.y);
}
// four values -> the 8 bytes of each plane
__device__ __forceinline__ void fp16_pair4(const float (&x)[4], float scale, uint2 &hi, uint2 &lo) {
  __half2 h0, l0, h1, l1;
  fp16_pair2(x[0], x[1], scale, h0, l0);
  fp16_pair2(x[2], x[3], scale, h1, l1);
  hi = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
  lo = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
}

// power-of-two scale that brings a largest magnitude `amax` into [2^14, 2^15); 1 when
// amax is zero or not finite (then the data decides the result anyway)
__device__ __forceinline__ float fp16_pair_scale(float amax) {
  if (!(amax > 0.f) || amax - amax != 0.f) return 1.f;
  int e;
  frexpf(amax, &e);  // amax = m * 2^e, m in [0.5, 1)
  e = 15 - e;        // amax * 2^(15 - e) in [2^14, 2^15)
  e = e > 100 ? 100 : (e < -100 ? -100 : e);
  return ldexpf(1.f, e);
}

__host__ __device__ inline uint32_t idesc_f16(int M, int N, bool a_mn_major, bool b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;  // D format: F32; A and B formats: 0 = F16
  d |= (a_mn_major ? 1u : 0u) << 15;
  d |= (b_mn_major ? 1u : 0u) << 16;
  d |= (uint32_t)(N >> 3) << 17;
  d |= (uint32_t)(M >> 4) << 24;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem], fp16 operands, fp32 accumulation; issued by ONE thread
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// box in shared memory -> global, clipped at the tensor's edges; completion is tracked
// by the issuing thread's bulk groups
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"((uint64_t)map), "r"(smem_src), "r"(x), "r"(y), "r"(z)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// until the stores issued by this thread have READ their shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// mbar_wait that also gives up as soon as another role of the CTA has given up
__device__ __forceinline__ bool mbar_wait_watch(uint64_t *bar, uint32_t parity, volatile int *failed) {
  for (int it = 0; it < kWaitLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63) == 63 && *failed) return false;
  }
  return false;
}

struct PairTile {
  int m0, n0, z, KB, k_begin;
};
// work item w -> (z, m tile, n tile); the n tiles of one m tile are neighbours, so the
// CTAs that run at the same time share their A rows in L2
template <bool BATCHED>
__device__ __forceinline__ PairTile pair_tile(const LinShape &p, int w) {
  PairTile t;
  const int per_z = p.tiles_m * p.tiles_n;
  t.z = w / per_z;
  const int r = w - t.z * per_z;
  t.m0 = (r / p.tiles_n) * kPairTile;
  t.n0 = (r % p.tiles_n) * kPairTile;
  t.k_begin = BATCHED ? 0 : t.z * p.k_per_split;
  const int k_end = BATCHED ? p.K : min(p.K, t.k_begin + p.k_per_split);
  t.KB = k_end > t.k_begin ? (k_end - t.k_begin + kPairBK - 1) / kPairBK : 0;
  return t;
}

template <bool A_MN, bool B_MN, class Ext>
__global__ void __launch_bounds__(kPairThreads, 1)
pair_umma_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                 const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
                 const __grid_constant__ CUtensorMap map_out, LinShape p, Ext ext) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kPairStages];   // TMA bytes have landed
  __shared__ __align__(8) uint64_t bar_empty[kPairStages];  // the MMAs are done with the stage
  // a group's accumulator is complete: one barrier per (fold set, accumulator), because a
  // parity wait can only tell the current phase from the one before it -- a set must find
  // nothing but its own tiles' groups on the barriers it waits on
  __shared__ __align__(8) uint64_t bar_grp[2][2];
  __shared__ __align__(8) uint64_t bar_fold[2];             // ... and has been folded away
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.tiles_m * p.tiles_n * p.nz;
  const uint32_t tiles = (smem_u32(smem_dyn) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&bar_grp[0][r], 1);
      mbar_init(&bar_grp[1][r], 1);
      mbar_init(&bar_fold[r], kPairFolders);
    }
    failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, kPairCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_slot;
  volatile int *vfailed = &failed;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // K slices issued so far, over all items
      for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
        const PairTile t = pair_tile<Ext::kBatched>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kPairStages;
          if (it >= kPairStages && !mbar_wait_watch(&bar_empty[s], (uint32_t)((it / kPairStages - 1) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          const int k0 = t.k_begin + kb * kPairBK;
          const uint32_t st = tiles + (uint32_t)s * kPairStageBytes;
          mbar_expect_tx(&bar_full[s], kPairStageBytes);
          const int zc = Ext::kBatched ? t.z : 0;  // outer coordinate of the operand maps
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              tma_load_3d(st + j * 8192, &map_ahi, t.m0 + 64 * j, k0, zc, &bar_full[s]);
              tma_load_3d(st + kPairOpBytes + j * 8192, &map_alo, t.m0 + 64 * j, k0, zc, &bar_full[s]);
            }
          } else {
            tma_load_3d(st, &map_ahi, k0, t.m0, zc, &bar_full[s]);
            tma_load_3d(st + kPairOpBytes, &map_alo, k0, t.m0, zc, &bar_full[s]);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              tma_load_3d(st + 2 * kPairOpBytes + j * 8192, &map_bhi, t.n0 + 64 * j, k0, zc, &bar_full[s]);
              tma_load_3d(st + 3 * kPairOpBytes + j * 8192, &map_blo, t.n0 + 64 * j, k0, zc, &bar_full[s]);
            }
          } else {
            tma_load_3d(st + 2 * kPairOpBytes, &map_bhi, k0, t.n0, zc, &bar_full[s]);
            tma_load_3d(st + 3 * kPairOpBytes, &map_blo, k0, t.n0, zc, &bar_full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_f16(kPairTile, kPairTile, A_MN, B_MN);
      // a K = 16 step inside a tile: 32 bytes along a K-major row, or two 8-row atoms
      // (2048 bytes) of a tile whose rows run along M / N; LBO = next block of 64
      // M / N values (only the latter layout uses it), SBO = next group of 8 rows
      constexpr uint32_t a_step = A_MN ? 2048u : 32u, b_step = B_MN ? 2048u : 32u;
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
      int it = 0, gg = 0, item = 0;  // K slices, accumulator groups and items so far
      for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x, ++item) {
        const PairTile t = pair_tile<Ext::kBatched>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kPairStages;
          const bool group_start = kb % kPairGroup == 0;
          // this accumulator was last used two groups ago: it must have been folded away
          if (group_start && gg >= 2 && !mbar_wait_watch(&bar_fold[gg & 1], (uint32_t)(((gg - 2) >> 1) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          if (!mbar_wait_watch(&bar_full[s], (uint32_t)((it / kPairStages) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t acc = tmem_d + ((gg & 1) ? kPairAcc1 : 0u);
          const uint32_t st = tiles + (uint32_t)s * kPairStageBytes;
#pragma unroll
          for (int ks = 0; ks < kPairBK / 16; ++ks) {
            const uint64_t dah = smem_desc_sw128(st + ks * a_step, a_lbo, 1024u);
            const uint64_t dal = smem_desc_sw128(st + kPairOpBytes + ks * a_step, a_lbo, 1024u);
            const uint64_t dbh = smem_desc_sw128(st + 2 * kPairOpBytes + ks * b_step, b_lbo, 1024u);
            const uint64_t dbl = smem_desc_sw128(st + 3 * kPairOpBytes + ks * b_step, b_lbo, 1024u);
            mma_f16_ss(acc, dah, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
            mma_f16_ss(acc, dah, dbl, idesc, 1u);
            mma_f16_ss(acc, dal, dbh, idesc, 1u);
          }
          mma_commit(&bar_empty[s]);
          if (kb % kPairGroup == kPairGroup - 1 || kb == t.KB - 1) {
            mma_commit(&bar_grp[item & 1][gg & 1]);
            ++gg;
          }
        }
      }
    }
  } else {
    // ---- fold finished groups into the set's running sum, then the epilogue --------------------
    const int set = (warp - 2) >> 2;  // which of the two sets; tiles alternate between them
    const int quarter = warp & 3;     // tensor-memory lanes 32*quarter..
    const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
    const uint32_t run = tmem_d + lane_base + kPairRun + 128u * (uint32_t)set;
    const uint32_t box = tiles + (uint32_t)kPairStages * kPairStageBytes + (uint32_t)(warp - 2) * kPairBoxBytes;
    uint8_t *box_ptr = smem_dyn + (box - smem_u32(smem_dyn));
    bool ok = true;
    int gg = 0, item = 0;
    int seen[2] = {0, 0};  // phases this set has consumed on its two barriers
    for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++item) {
      const PairTile t = pair_tile<Ext::kBatched>(p, w);
      const int NG = (t.KB + kPairGroup - 1) / kPairGroup;
      if ((item & 1) != set) {  // the other set's tile
        gg += NG;
        continue;
      }
      const int m = t.m0 + 32 * quarter + lane;
      const bool row_ok = m < p.M;
      typename Ext::Row rs;
      if (Ext::kCustomStore) {
        // whole warp: per-column data of the tile into the warp's (otherwise unused) box
        ext.tile_begin(t.z, t.n0, box_ptr, lane);
        __syncwarp();
      }
      if (row_ok) {
        ext.row_begin(rs, t.z, m, t.n0);
        ext.prefetch(rs, t.z, m, t.n0);
      }
      for (int g = 0; g < NG && ok; ++g, ++gg) {
        bool got = mbar_wait_watch(&bar_grp[set][gg & 1], (uint32_t)(seen[gg & 1] & 1), vfailed);
        ++seen[gg & 1];
        got = __all_sync(0xffffffffu, got);
        if (!got) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem_d + lane_base + ((gg & 1) ? kPairAcc1 : 0u);
        // 32 columns at a time: both loads in flight, one wait; the stores drain behind
        for (int c = 0; c < kPairTile; c += 32) {
          float pv[32], rv[32];
          tmem_ld32_nowait(acc + c, pv);
          if (g > 0) tmem_ld32_nowait(run + c, rv);
          tmem_ld_wait();
          if (g > 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i) pv[i] = rv[i] + pv[i];
          }
          tmem_st32_nowait(run + c, pv);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_fold[gg & 1]);
      }
      ok = __all_sync(0xffffffffu, ok) && !*vfailed;
      if (!ok) *vfailed = 1;
      if (Ext::kCustomStore) {
        // the policy stores the tile itself, boxes from the last to the first
        for (int c0 = kPairTile - 32; c0 >= 0; c0 -= 32) {
          if (t.n0 + c0 >= p.N) continue;
          float pv[32];
          if (ok && t.KB > 0) {
            tmem_ld32_nowait(run + c0, pv);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) pv[i] = ok ? 0.f : NAN;
          }
          float v0[16], v1[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v0[i] = pv[i], v1[i] = pv[16 + i];
          if (row_ok) ext.store_box(rs, t.z, m, t.n0, c0, v0, v1, box_ptr);
        }
      } else {
      // epilogue from the running sum: 32 columns -> policy -> swizzled 32 x 32 box -> TMA store
      for (int c0 = 0; c0 < kPairTile && t.n0 + c0 < p.N; c0 += 32) {
        float pv[32];
        if (ok && t.KB > 0) {
          tmem_ld32_nowait(run + c0, pv);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) pv[i] = 0.f;
        }
        const int n = t.n0 + c0;
        float v0[16], v1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v0[i] = pv[i], v1[i] = pv[16 + i];
        if (row_ok) {
          ext.finish(rs, t.z, m, n, v0, 0);
          if (n + 16 < p.N) ext.finish(rs, t.z, m, n + 16, v1, 1);
          if (c0 + 32 < kPairTile && n + 32 < p.N) ext.prefetch(rs, t.z, m, n + 32);
        }
        if (!ok) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v0[i] = v1[i] = NAN;
        }
        // the store of the previous box must have read the staging buffer
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          *reinterpret_cast<float4 *>(box_ptr + sw128_offset(lane, j)) =
              make_float4(v0[4 * j], v0[4 * j + 1], v0[4 * j + 2], v0[4 * j + 3]);
          *reinterpret_cast<float4 *>(box_ptr + sw128_offset(lane, 4 + j)) =
              make_float4(v1[4 * j], v1[4 * j + 1], v1[4 * j + 2], v1[4 * j + 3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) tma_store_3d(&map_out, box, n, t.m0 + 32 * quarter, t.z);
      }
      }
      if (row_ok) ext.row_end(rs, t.z, m, t.n0);
      tc_fence_before_sync();
    }
    if (lane == 0) tma_store_wait_read();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, kPairCols);
}

// ---- host -----------------------------------------------------------------------------------
// map of `batch` row-major fp16 matrices [rows][cols] whose rows are `pitch` halves apart and
// which follow each other every `batch_stride` halves (batch <= 1: one matrix); box =
// box_cols x box_rows x 1, 128-byte swizzle.  Elements outside [rows][cols] read as zeros.
inline int make_map_f16(CUtensorMap *map, const void *base, int rows, int cols, long long pitch, int batch,
                        long long batch_stride, int box_cols, int box_rows) {
  auto enc = tensor_map_encoder();
  FRNNT_REQUIRE(enc != nullptr, FRNNT_ECUDA, "cuTensorMapEncodeTiled is not available");
  if (batch <= 1) {
    batch = 1;
    batch_stride = (long long)rows * pitch;
  }
  FRNNT_REQUIRE((uintptr_t)base % 16 == 0 && pitch % 8 == 0 && batch_stride % 8 == 0, FRNNT_EUNSUPPORTED,
                "TMA needs a 16-byte aligned base and row / matrix strides that are multiples of 8 halves");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)pitch * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FRNNT_REQUIRE(r == CUDA_SUCCESS, FRNNT_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return FRNNT_OK;
}
// operand plane for the engine: K-major ([M or N rows][K cols], box 64 k x 128 rows) or
// contiguous along M / N ([K rows][M or N cols], boxes of 64 values x 64 k rows)
inline int make_pair_map(CUtensorMap *map, const void *base, int rows, int cols, long long pitch,
                         bool mn_major, int batch = 0, long long batch_stride = 0) {
  return mn_major ? make_map_f16(map, base, rows, cols, pitch, batch, batch_stride, 64, kPairBK)
                  : make_map_f16(map, base, rows, cols, pitch, batch, batch_stride, kPairBK, kPairTile);
}

// map of the float32 output [nz][M][N] (row pitch N floats): boxes of 32 x 32, stored from
// a 128-byte-swizzled staging buffer
inline int make_out_map(CUtensorMap *map, const float *base, int nz, int M, int N) {
  auto enc = tensor_map_encoder();
  FRNNT_REQUIRE(enc != nullptr, FRNNT_ECUDA, "cuTensorMapEncodeTiled is not available");
  FRNNT_REQUIRE((uintptr_t)base % 16 == 0 && N % 4 == 0, FRNNT_EUNSUPPORTED,
                "the output needs a 16-byte aligned base and a row length that is a multiple of 4 floats");
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)(nz > 0 ? nz : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)N * 4, (cuuint64_t)N * 4 * (cuuint64_t)M};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FRNNT_REQUIRE(r == CUDA_SUCCESS, FRNNT_ECUDA, "cuTensorMapEncodeTiled (output) failed with %d", (int)r);
  return FRNNT_OK;
}

// out = [shape.nz][shape.M][shape.N] floats
template <bool A_MN, bool B_MN, class Ext>
int launch_pair_umma(const CUtensorMap &mah, const CUtensorMap &mal, const CUtensorMap &mbh,
                     const CUtensorMap &mbl, float *out, const LinShape &shape, const Ext &ext,
                     cudaStream_t st) {
  CUtensorMap mo;
  // a policy that stores the result itself never uses the map, which still has to be valid
  int rc = Ext::kCustomStore ? make_out_map(&mo, out, 1, 4, 4) : make_out_map(&mo, out, shape.nz, shape.M, shape.N);
  if (rc != FRNNT_OK) return rc;
  auto kern = pair_umma_kernel<A_MN, B_MN, Ext>;
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmemBytes));
  int ctas = 0;
  rc = lin_grid((long long)shape.tiles_m * shape.tiles_n * shape.nz, &ctas);
  if (rc != FRNNT_OK) return rc;
  if (ctas == 0) return FRNNT_OK;
  FRNNT_KERNEL(kern<<<ctas, kPairThreads, kPairSmemBytes, st>>>(mah, mal, mbh, mbl, mo, shape, ext));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

}  // namespace frnnt
