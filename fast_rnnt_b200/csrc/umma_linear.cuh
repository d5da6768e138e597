// The 3xTF32 tensor-core product engine of this library (sm_100a): a persistent,
// TMA-fed kernel for D = A * B^T-like products of row-major float matrices with
// fp32-level accuracy, parameterised by a small policy ("Ext") that says
//   * whether the product is batched (a third tensor-map dimension),
//   * whether the B operand is exponentiated on its way to the tensor core
//     (exp(x - shift[k]): the softmax numerators of the lattice gradients), and
//   * what the epilogue does with a finished row segment.
//
// Kernel structure (one 128x128 output tile per work item, 14 warps, one CTA per SM
// that walks a list of work items):
//   warp 0   : TMA producer.  cp.async.bulk.tensor loads the raw fp32 operand
//              tiles of a 32-wide K slice into the 128-byte-swizzled layouts
//              (K-major: swizzle 128B; operands that are contiguous along M/N:
//              swizzle 128B with 32-byte atoms), completion on an mbarrier;
//              4-stage ring.  Out-of-range rows / columns arrive as zeros.
//   warps 2-9: split every landed value x into hi + lo in tf32.  A: hi = tf32(x) and
//              lo = tf32(x - hi), both rounded to nearest.  B: hi is the landed word
//              itself (the tensor core drops its low 13 bits), lo = tf32(x - trunc(x))
//              goes to a second buffer (an element-wise pass that does not care about
//              the tile layout).  A goes to TENSOR MEMORY: thread <-> row
//              of the tile, tcgen05.st of its 16 k values (hi and lo), a ring of
//              two K slices.  The tensor core then reads only B from shared
//              memory, whose bandwidth is what bounds a 3xTF32 product whose
//              operands both live there.
//   warp 1   : one thread issues hi*hi, hi*lo, lo*hi tcgen05.mma per K=8 step
//              (A from tensor memory) into a 128x128 fp32 accumulator in tensor
//              memory; tcgen05.commit hands the stage back to the producer and
//              the A slot back to the split warps.  The tensor core adds into
//              its accumulator with truncation (a bias of ~half an ulp per
//              step), so every 128-wide K group gets a fresh accumulator and
//   warps 10-13 fold finished groups into a running sum with round-to-nearest
//              adds (tcgen05.ld / add / tcgen05.st), one group behind the MMAs,
//              and run the epilogue (tcgen05.ld -> policy -> 64-byte row
//              segments) while the other warps are already on the next item.
// One CTA per SM, every load is a plain per-CTA TMA load.  Every wait is bounded; a timeout poisons the tile.
//
// Policy interface (all __device__, called with z = batch or split index):
//   static constexpr bool kBatched;   tensor maps are 3-D, z is their outer coordinate
//   static constexpr bool kExpB;      B := exp(B - b_shift(z)[k]), 0 for k >= K (needs B_MN)
//   const float *b_shift(int z) const;
//   const float *pre_row(int z, int m) const;   row m of a matrix [..][N] the epilogue
//                                     combines with the result (or nullptr); the engine
//                                     loads it early and hands it to finish()
//   void finish(int z, int m, int n, float (&v)[16], const float (&x)[16]) const;
//                                     columns n..n+15 of row m, in place
//   float *out_row(int z, int m) const;         where row m of the result goes
//   static constexpr bool kColSumA;   also sum the A operand over k (per row m of the tile):
//   float *a_colsum(int z, int half) const;     [M] partial sums of work-item slice z, one per
//                                     half of the split warps (they share a K slice 16 / 16)
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"
#include "umma.cuh"

namespace frnnt {
using namespace umma;

constexpr int kLinThreads = 448;   // TMA warp, MMA warp, 8 split warps, 4 fold / epilogue warps
constexpr int kLinWorkers = 8;
constexpr int kLinFolders = 4;
constexpr int kLinTile = 128;
constexpr int kLinBK = 32;
constexpr int kLinStages = 4;
constexpr int kLinASlots = 2;  // K slices of the A operand held in tensor memory
constexpr int kLinGroup = 4;   // K slices per accumulator group
constexpr uint32_t kLinOpBytes = kLinTile * 128;          // one operand tile
constexpr uint32_t kLinStageBytes = 3 * kLinOpBytes;      // A_raw, B_raw -> B_hi, B_lo
constexpr size_t kLinSmemBytes = (size_t)kLinStages * kLinStageBytes + 1024;
// tensor-memory columns: two group accumulators, the running sum, the A ring (hi | lo per slot)
constexpr uint32_t kLinCols = 512, kLinAcc1 = 128, kLinRun = 256, kLinAop = 384;

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// tiled TMA loads: box at (x = innermost coordinate, y[, z]) -> shared memory, bytes counted on bar
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap *map, int x, int y,
                                            int z, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void *p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

struct LinShape {
  int M, N, K;         // K = reduction length
  int k_per_split;     // multiple of kLinBK (the whole of K when batched)
  int tiles_m, tiles_n, nz;   // nz = splits or batch size
};

// work item w -> (z, m tile, n tile); the n tiles of one m tile are neighbours, so
// the CTAs that run at the same time share their A rows in L2
struct LinTile {
  int m0, n0, z, KB, k_begin;
};
template <bool BATCHED>
__device__ __forceinline__ LinTile lin_tile(const LinShape &p, int w) {
  LinTile t;
  const int per_z = p.tiles_m * p.tiles_n;
  t.z = w / per_z;
  const int r = w - t.z * per_z;
  t.m0 = (r / p.tiles_n) * kLinTile;
  t.n0 = (r % p.tiles_n) * kLinTile;
  t.k_begin = BATCHED ? 0 : t.z * p.k_per_split;
  const int k_end = min(p.K, t.k_begin + p.k_per_split);
  t.KB = k_end > t.k_begin ? (k_end - t.k_begin + kLinBK - 1) / kLinBK : 0;
  return t;
}

// Persistent: CTA c works on items c, c + gridDim.x, ...; every role walks the same
// list, and the ring / accumulator indices run on across items, so the TMA producer,
// the split warps and the MMAs of the next tile start while the fold warps still
// write the previous tile out.
template <bool A_MN, bool B_MN, class Ext>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   LinShape p, Ext ext) {
  static_assert(!Ext::kExpB || B_MN, "the exponentiated operand must be contiguous along N");
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kLinStages];   // TMA bytes have landed
  __shared__ __align__(8) uint64_t bar_split[kLinStages];  // hi / lo are ready
  __shared__ __align__(8) uint64_t bar_empty[kLinStages];  // the MMAs are done with the stage
  __shared__ __align__(8) uint64_t bar_grp[2];             // a group's accumulator is complete
  __shared__ __align__(8) uint64_t bar_fold[2];            // ... and has been folded away
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  constexpr bool BATCHED = Ext::kBatched;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.tiles_m * p.tiles_n * p.nz;
  const uint32_t tiles = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  uint8_t *tiles_ptr = smem_dyn + (tiles - smem_u32(smem_dyn));

  if (tid == 0) {
    for (int s = 0; s < kLinStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_split[s], kLinWorkers);
      mbar_init(&bar_empty[s], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&bar_grp[r], 1);
      mbar_init(&bar_fold[r], kLinFolders);
    }
    failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&tmem_slot, kLinCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_slot;
  volatile int *vfailed = &failed;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // K slices issued so far, over all items
      for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
        const LinTile t = lin_tile<BATCHED>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kLinStages;
          if (it >= kLinStages && !mbar_wait(&bar_empty[s], (uint32_t)((it / kLinStages - 1) & 1))) {
            *vfailed = 1;
            break;
          }
          const int k0 = t.k_begin + kb * kLinBK;
          const uint32_t st = tiles + (uint32_t)s * kLinStageBytes;
          mbar_expect_tx(&bar_full[s], 2 * kLinOpBytes);
          auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y) {
            if (BATCHED)
              tma_load_3d(dst, map, x, y, t.z, &bar_full[s]);
            else
              tma_load_2d(dst, map, x, y, &bar_full[s]);
          };
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 4; ++j) load(st + j * 4096, &map_a, t.m0 + 32 * j, k0);
          } else {
            load(st, &map_a, k0, t.m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 4; ++j) load(st + kLinOpBytes + j * 4096, &map_b, t.n0 + 32 * j, k0);
          } else {
            load(st + kLinOpBytes, &map_b, k0, t.n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // A comes from tensor memory (always K-major there), B from shared memory
      const uint32_t idesc = idesc_tf32(kLinTile, kLinTile, false, B_MN);
      int it = 0, gg = 0;  // K slices and accumulator groups so far, over all items
      for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
        const LinTile t = lin_tile<BATCHED>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kLinStages;
          const bool group_start = kb % kLinGroup == 0;
          // this accumulator was last used two groups ago: it must have been folded away
          if (group_start && gg >= 2 && !mbar_wait(&bar_fold[gg & 1], (uint32_t)(((gg - 2) >> 1) & 1))) {
            *vfailed = 1;
            break;
          }
          if (!mbar_wait(&bar_split[s], (uint32_t)((it / kLinStages) & 1))) {
            *vfailed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t acc = tmem_d + ((gg & 1) ? kLinAcc1 : 0u);
          const uint32_t a_hi = tmem_d + kLinAop + (uint32_t)(it % kLinASlots) * 64u, a_lo = a_hi + 32u;
          const uint32_t st = tiles + (uint32_t)s * kLinStageBytes;
#pragma unroll
          for (int ks = 0; ks < kLinBK / 8; ++ks) {
            const uint32_t bo = B_MN ? ks * 1024u : ks * 32u;
            const uint32_t b_lbo = B_MN ? 4096u : 16u, b_sbo = B_MN ? 512u : 1024u;
            const uint32_t b_lt = B_MN ? 1u : 2u;
            const uint64_t dbh = smem_desc_sw128(st + kLinOpBytes + bo, b_lbo, b_sbo, b_lt);
            const uint64_t dbl = smem_desc_sw128(st + 2 * kLinOpBytes + bo, b_lbo, b_sbo, b_lt);
            mma_tf32_ts(acc, a_hi + 8u * ks, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
            mma_tf32_ts(acc, a_hi + 8u * ks, dbl, idesc, 1u);
            mma_tf32_ts(acc, a_lo + 8u * ks, dbh, idesc, 1u);
          }
          mma_commit(&bar_empty[s]);
          if (kb % kLinGroup == kLinGroup - 1 || kb == t.KB - 1) {
            mma_commit(&bar_grp[gg & 1]);
            ++gg;
          }
        }
      }
    }
  } else if (warp < 2 + kLinWorkers) {
    // ---- split pass ------------------------------------------------------------------------
    const int st_tid = tid - 64;  // 0..255
    const int quarter = warp & 3;          // tensor-memory lanes 32*quarter..
    const int half = (warp - 2) >> 2;      // which half of the K slice
    const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
    const int row = 32 * quarter + lane;   // row of the A tile this thread moves to tensor memory
    // B is contiguous along N when it is exponentiated: chunk c of the tile belongs to
    // k row (c >> 3) & 31, the same for all of this thread's chunks
    const int b_krow = (st_tid >> 3) & 31;
    int it = 0;
    for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
      const LinTile t = lin_tile<BATCHED>(p, w);
      const float *shift = Ext::kExpB ? ext.b_shift(t.z) : nullptr;
      float asum = 0.f;
      for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
        const int s = it % kLinStages;
        float sh = 0.f;
        bool k_ok = true;
        if (Ext::kExpB) {  // in flight while the slice lands
          const int k = t.k_begin + kb * kLinBK + b_krow;
          k_ok = k < p.K;
          sh = k_ok ? shift[k] : 0.f;
        }
        if (!mbar_wait(&bar_full[s], (uint32_t)((it / kLinStages) & 1))) {
          *vfailed = 1;
          break;
        }
        const uint8_t *araw = tiles_ptr + (size_t)s * kLinStageBytes;
        float4 *braw = reinterpret_cast<float4 *>(tiles_ptr + (size_t)s * kLinStageBytes + kLinOpBytes);
        float4 *blo = braw + kLinOpBytes / 16;
        // all shared-memory loads of the slice first
        constexpr int kChunksPerThread = (int)(kLinOpBytes / 16) / (32 * kLinWorkers);
        float4 x[kChunksPerThread];
        float av[16];
#pragma unroll
        for (int q = 0; q < kChunksPerThread; ++q) x[q] = braw[st_tid + q * 32 * kLinWorkers];
        if (A_MN) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            av[i] = *reinterpret_cast<const float *>(araw + mn_tile_offset(16 * half + i, row >> 2) +
                                                     4 * (row & 3));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 v = *reinterpret_cast<const float4 *>(araw + sw128_offset(row, 4 * half + j));
            av[4 * j] = v.x, av[4 * j + 1] = v.y, av[4 * j + 2] = v.z, av[4 * j + 3] = v.w;
          }
        }
        // B: hi and lo; an element-wise pass, the tile layout does not matter.  A plain B
        // stays where it landed: the tensor core reads the raw fp32 word as tf32, i.e. its
        // hi is the TRUNCATED value, and only lo = tf32(x - trunc(x)) is written.  The
        // one-sided remainder is harmless because A is split with rounding: the neglected
        // term lo_a * lo_b then has no preferred sign.  An exponentiated B is new data
        // and is written in full.
#pragma unroll
        for (int q = 0; q < kChunksPerThread; ++q) {
          if (Ext::kExpB) {
            x[q].x = k_ok ? expf(x[q].x - sh) : 0.f;
            x[q].y = k_ok ? expf(x[q].y - sh) : 0.f;
            x[q].z = k_ok ? expf(x[q].z - sh) : 0.f;
            x[q].w = k_ok ? expf(x[q].w - sh) : 0.f;
            float4 h, l;
            split_tf32(x[q], h, l);
            braw[st_tid + q * 32 * kLinWorkers] = h;
            blo[st_tid + q * 32 * kLinWorkers] = l;
          } else {
            float4 l;
            l.x = round_tf32(x[q].x - trunc_tf32(x[q].x));
            l.y = round_tf32(x[q].y - trunc_tf32(x[q].y));
            l.z = round_tf32(x[q].z - trunc_tf32(x[q].z));
            l.w = round_tf32(x[q].w - trunc_tf32(x[q].w));
            blo[st_tid + q * 32 * kLinWorkers] = l;
          }
        }
        // A: this thread's row, 16 of the 32 k values, hi and lo into tensor memory
        float hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) split_tf32(av[i], hi[i], lo[i]);
        if (Ext::kColSumA) {
#pragma unroll
          for (int i = 0; i < 16; ++i) asum += av[i];
        }
        // the slot was last read by the MMAs of K slice it - kLinASlots
        if (it >= kLinASlots) {
          const int ip = it - kLinASlots;
          if (!mbar_wait(&bar_empty[ip % kLinStages], (uint32_t)((ip / kLinStages) & 1))) {
            *vfailed = 1;
            break;
          }
          tc_fence_after_sync();
        }
        const uint32_t a_hi = tmem_d + lane_base + kLinAop + (uint32_t)(it % kLinASlots) * 64u + 16u * half;
        tmem_st16_nowait(a_hi, hi);
        tmem_st16_nowait(a_hi + 32u, lo);
        tmem_st_wait();
        fence_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_split[s]);
      }
      if (Ext::kColSumA && t.n0 == 0 && t.m0 + row < p.M) {
        float *cs = ext.a_colsum(t.z, half);
        if (cs != nullptr) cs[t.m0 + row] = asum;
      }
    }
  } else {
    // ---- fold finished groups into the running sum, then the epilogue -------------------------
    const int quarter = warp & 3;          // tensor-memory lanes 32*quarter..
    const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
    const uint32_t run = tmem_d + lane_base + kLinRun;
    const bool vec = (p.N % 4) == 0;
    bool ok = true;
    int gg = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
      const LinTile t = lin_tile<BATCHED>(p, w);
      const int NG = (t.KB + kLinGroup - 1) / kLinGroup;
      const int m = t.m0 + 32 * quarter + lane;
      const bool row_ok = m < p.M;
      float *out = row_ok ? ext.out_row(t.z, m) : nullptr;
      const float *pre = row_ok ? ext.pre_row(t.z, m) : nullptr;
      // the values the epilogue combines with come from DRAM: ask for them now, while the
      // tile is still being computed (these warps have nothing else to do yet)
      if (pre != nullptr) {
#pragma unroll
        for (int c = 0; c < kLinTile; c += 32)
          if (t.n0 + c < p.N) prefetch_l2(pre + t.n0 + c);
      }
      for (int g = 0; g < NG && ok; ++g, ++gg) {
        if (!mbar_wait(&bar_grp[gg & 1], (uint32_t)((gg >> 1) & 1))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem_d + lane_base + ((gg & 1) ? kLinAcc1 : 0u);
        // 16 columns at a time: both loads in flight, one wait; the stores drain behind
        for (int c = 0; c < kLinTile; c += 16) {
          float pv[16], rv[16];
          tmem_ld16_nowait(acc + c, pv);
          if (g > 0) tmem_ld16_nowait(run + c, rv);
          tmem_ld_wait();
          if (g > 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) pv[i] = rv[i] + pv[i];
          }
          tmem_st16_nowait(run + c, pv);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_fold[gg & 1]);
      }
      ok = __all_sync(0xffffffffu, ok) && !*vfailed;
      if (!ok) *vfailed = 1;
      tc_fence_after_sync();
      // 32 columns per round: the loads of the values the epilogue combines with are
      // issued before the first accumulator read, so their latency is paid four times
      // per tile, not once per 16 columns
      for (int c0 = 0; c0 < kLinTile; c0 += 32) {
        float4 tv[8];
        const bool pre_vec = pre != nullptr && vec && t.n0 + c0 + 32 <= p.N;
        if (pre_vec) {
          const float4 *a4 = reinterpret_cast<const float4 *>(pre + t.n0 + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) tv[i] = a4[i];
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int ch = c0 / 16 + cc;
          float v[16], x[16];
          if (ok && t.KB > 0) {
            tmem_ld16(run + (uint32_t)(ch * 16), v);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
          }
          const int n = t.n0 + ch * 16;
          if (row_ok && n < p.N) {
            if (pre_vec) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float4 tt = tv[4 * cc + i];
                x[4 * i] = tt.x, x[4 * i + 1] = tt.y, x[4 * i + 2] = tt.z, x[4 * i + 3] = tt.w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) x[i] = (pre != nullptr && n + i < p.N) ? pre[n + i] : 0.f;
            }
            ext.finish(t.z, m, n, v, x);
            if (!ok) {
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = NAN;
            }
            float *dst = out + n;
            if (vec && n + 16 <= p.N) {
#pragma unroll
              for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n + i < p.N) dst[i] = v[i];
            }
          }
        }
      }
      // the running sum is rewritten by the first fold of the next item, which these
      // same warps perform: no further hand-shake is needed
      tc_fence_before_sync();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, kLinCols);
}

// ---- host -----------------------------------------------------------------------------------
inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)ptr;
  }
  return fn;
}

// map of `batch` row-major float matrices [rows][cols] whose rows are `pitch` floats apart
// (pitch >= cols) and which follow each other every `batch_stride` floats; box = box_cols x
// box_rows (x 1).  batch == 0: a 2-D map of a single matrix.  Elements outside
// [rows][cols] read as zeros.
inline int make_map(CUtensorMap *map, const float *base, int rows, int cols, long long pitch,
                    long long batch_stride, int batch, int box_cols, int box_rows, bool atom32) {
  auto enc = tensor_map_encoder();
  FRNNT_REQUIRE(enc != nullptr, FRNNT_ECUDA, "cuTensorMapEncodeTiled is not available");
  FRNNT_REQUIRE((uintptr_t)base % 16 == 0 && pitch % 4 == 0 && batch_stride % 4 == 0, FRNNT_EUNSUPPORTED,
                "TMA needs a 16-byte aligned base and row / matrix strides that are multiples of 4 floats");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)pitch * sizeof(float), (cuuint64_t)batch_stride * sizeof(float)};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, batch > 0 ? 3 : 2, (void *)base, dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FRNNT_REQUIRE(r == CUDA_SUCCESS, FRNNT_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return FRNNT_OK;
}
// operand map for the engine: K-major (rows = M or N index, box 32 k x 128 rows) or
// contiguous along M/N (rows = k index, boxes of 32 values x 32 k rows, 32-byte swizzle atoms)
inline int make_operand_map(CUtensorMap *map, const float *base, int rows, int cols, long long pitch,
                            long long batch_stride, int batch, bool mn_major) {
  return mn_major ? make_map(map, base, rows, cols, pitch, batch_stride, batch, 32, kLinBK, true)
                  : make_map(map, base, rows, cols, pitch, batch_stride, batch, kLinBK, kLinTile, false);
}

// one persistent CTA per SM (shared memory and tensor memory allow no more), fewer when
// there are fewer work items
inline int lin_grid(long long items, int *ctas) {
  const int sms = sm_count();
  *ctas = (int)(items < sms ? items : sms);
  return FRNNT_OK;
}

template <bool A_MN, bool B_MN, class Ext>
int launch_linear_umma(const CUtensorMap &ma, const CUtensorMap &mb, const LinShape &shape, const Ext &ext,
                       cudaStream_t st) {
  auto kern = linear_umma_kernel<A_MN, B_MN, Ext>;
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemBytes));
  int ctas = 0;
  const int rc = lin_grid((long long)shape.tiles_m * shape.tiles_n * shape.nz, &ctas);
  if (rc != FRNNT_OK) return rc;
  if (ctas == 0) return FRNNT_OK;
  FRNNT_KERNEL(kern<<<ctas, kLinThreads, kLinSmemBytes, st>>>(ma, mb, shape, ext));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

}  // namespace frnnt
