// The fp16-pair engine (umma_pairs.cuh) with 256 x 128 output tiles per work item.
//
// Why: the 128 x 128 kernel keeps the tensor pipe about half busy: per 64-wide K slice it
// takes 64 KB of planes into shared memory (measured 37-48 bytes per clock and SM) while
// the MMAs read 96 KB of operands out of it.  A 256 x 128 tile shares every B slice between
// two row halves: 96 KB per slice for twice the flops, a quarter less traffic per flop, with
// plain per-CTA loads (no thread-block clusters).
//
// What changes against the 128 x 128 kernel:
//   * a stage holds A hi / lo for both row halves (4 x 16 KB) and B hi / lo (2 x 16 KB);
//     two stages (a stage is now 1536 cycles of MMA work, and one 96 KB stage in flight
//     covers the bandwidth-delay product of the feed);
//   * per K = 16 step six MMAs: the three products for each row half, into the
//     accumulator of that half: four 128-column accumulators (row half x group parity)
//     fill the 512 tensor-memory columns, so
//   * the running sums of the group folding live in REGISTERS: eight fold / epilogue
//     warps, warp <-> 32 rows of one half, thread <-> one row's 128 sums.  A fold is
//     tcgen05.ld of the finished accumulator + 128 round-to-nearest adds; the epilogue
//     (policy, staging box, TMA store) runs from the registers, with no tensor-memory
//     traffic.  The same warps serve every tile, so the epilogue of one tile overlaps only
//     the first two K groups of the next (enough: it is shorter than their 6000 cycles of
//     MMA).
// Policies are the ones of umma_pairs.cuh (custom-store policies are not supported here).
//
// WIDE = true turns the tile by ninety degrees: 128 rows x 256 columns, ONE MMA of N = 256 per
// product and K = 16 step instead of two of M = 128.  The stage is the same 96 KB (A hi / lo
// 2 x 16 KB, B hi / lo 2 x 32 KB), but the tensor core then reads 12 KB of operands out of
// shared memory per 128 cycles instead of 16 KB: shared memory serves the MMAs' operand reads
// (128 bytes per clock while an N = 128 MMA runs -- all there is) AND takes the TMA writes, and
// that, not the L2, is what holds the 128 x 128 kernel near half of the tensor pipe.  The fold
// warps are then warp <-> (32 rows, column half).
#pragma once
#include "umma_pairs.cuh"

namespace frnnt {

constexpr int kP2Threads = 320;   // TMA warp, MMA warp, 8 fold / epilogue warps
constexpr int kP2TileM = 256;
constexpr int kP2Stages = 2;
constexpr uint32_t kP2StageBytes = 6 * kPairOpBytes;  // A hi0, A lo0, A hi1, A lo1, B hi, B lo
constexpr size_t kP2SmemBytes = (size_t)kP2Stages * kP2StageBytes + 8 * kPairBoxBytes + 1024;

template <bool BATCHED, bool WIDE = false>
__device__ __forceinline__ PairTile pair_tile256(const LinShape &p, int w) {
  PairTile t;
  const int per_z = p.tiles_m * p.tiles_n;
  t.z = w / per_z;
  const int r = w - t.z * per_z;
  t.m0 = (r / p.tiles_n) * (WIDE ? kPairTile : kP2TileM);
  t.n0 = (r % p.tiles_n) * (WIDE ? 2 * kPairTile : kPairTile);
  t.k_begin = BATCHED ? 0 : t.z * p.k_per_split;
  const int k_end = BATCHED ? p.K : min(p.K, t.k_begin + p.k_per_split);
  t.KB = k_end > t.k_begin ? (k_end - t.k_begin + kPairBK - 1) / kPairBK : 0;
  return t;
}

// p.tiles_m counts 256-row tiles (WIDE: 128-row tiles, and p.tiles_n 256-column tiles)
template <bool A_MN, bool B_MN, class Ext, bool WIDE = false>
__global__ void __launch_bounds__(kP2Threads, 1)
pair_umma256_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                    const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
                    const __grid_constant__ CUtensorMap map_out, LinShape p, Ext ext) {
  static_assert(!Ext::kCustomStore, "custom-store policies run on the 128 x 128 kernel");
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kP2Stages];   // TMA bytes have landed
  __shared__ __align__(8) uint64_t bar_empty[kP2Stages];  // the MMAs are done with the stage
  __shared__ __align__(8) uint64_t bar_grp[2];            // a group's accumulators are complete
  __shared__ __align__(8) uint64_t bar_fold[2];           // ... and have been added to the sums
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.tiles_m * p.tiles_n * p.nz;
  const uint32_t tiles = (smem_u32(smem_dyn) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < kP2Stages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&bar_grp[r], 1);
      mbar_init(&bar_fold[r], 8);
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
        const PairTile t = pair_tile256<Ext::kBatched, WIDE>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kP2Stages;
          if (it >= kP2Stages && !mbar_wait_watch(&bar_empty[s], (uint32_t)((it / kP2Stages - 1) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          const int k0 = t.k_begin + kb * kPairBK;
          const uint32_t st = tiles + (uint32_t)s * kP2StageBytes;
          mbar_expect_tx(&bar_full[s], kP2StageBytes);
          const int zc = Ext::kBatched ? t.z : 0;
          if (WIDE) {
            // [A hi 16 KB][A lo 16 KB][B hi 32 KB][B lo 32 KB]
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
            const uint32_t sbw = st + 2 * kPairOpBytes;
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tma_load_3d(sbw + j * 8192, &map_bhi, t.n0 + 64 * j, k0, zc, &bar_full[s]);
                tma_load_3d(sbw + 2 * kPairOpBytes + j * 8192, &map_blo, t.n0 + 64 * j, k0, zc, &bar_full[s]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                tma_load_3d(sbw + j * kPairOpBytes, &map_bhi, k0, t.n0 + 128 * j, zc, &bar_full[s]);
                tma_load_3d(sbw + (2 + j) * kPairOpBytes, &map_blo, k0, t.n0 + 128 * j, zc, &bar_full[s]);
              }
            }
          } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t sa = st + (uint32_t)h * 2 * kPairOpBytes;
            const int mh = t.m0 + 128 * h;
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                tma_load_3d(sa + j * 8192, &map_ahi, mh + 64 * j, k0, zc, &bar_full[s]);
                tma_load_3d(sa + kPairOpBytes + j * 8192, &map_alo, mh + 64 * j, k0, zc, &bar_full[s]);
              }
            } else {
              tma_load_3d(sa, &map_ahi, k0, mh, zc, &bar_full[s]);
              tma_load_3d(sa + kPairOpBytes, &map_alo, k0, mh, zc, &bar_full[s]);
            }
          }
          const uint32_t sb = st + 4 * kPairOpBytes;
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              tma_load_3d(sb + j * 8192, &map_bhi, t.n0 + 64 * j, k0, zc, &bar_full[s]);
              tma_load_3d(sb + kPairOpBytes + j * 8192, &map_blo, t.n0 + 64 * j, k0, zc, &bar_full[s]);
            }
          } else {
            tma_load_3d(sb, &map_bhi, k0, t.n0, zc, &bar_full[s]);
            tma_load_3d(sb + kPairOpBytes, &map_blo, k0, t.n0, zc, &bar_full[s]);
          }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_f16(kPairTile, WIDE ? 2 * kPairTile : kPairTile, A_MN, B_MN);
      constexpr uint32_t a_step = A_MN ? 2048u : 32u, b_step = B_MN ? 2048u : 32u;
      constexpr uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
      int it = 0, gg = 0;  // K slices and accumulator groups so far, over all items
      for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
        const PairTile t = pair_tile256<Ext::kBatched, WIDE>(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kP2Stages;
          const bool group_start = kb % kPairGroup == 0;
          // these accumulators were last used two groups ago: they must have been folded away
          if (group_start && gg >= 2 && !mbar_wait_watch(&bar_fold[gg & 1], (uint32_t)(((gg - 2) >> 1) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          if (!mbar_wait_watch(&bar_full[s], (uint32_t)((it / kP2Stages) & 1), vfailed)) {
            *vfailed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t st = tiles + (uint32_t)s * kP2StageBytes;
          if (WIDE) {
            const uint32_t acc = tmem_d + (uint32_t)((gg & 1) * 256);
            const uint32_t sbw = st + 2 * kPairOpBytes;
#pragma unroll
            for (int ks = 0; ks < kPairBK / 16; ++ks) {
              const uint64_t dah = smem_desc_sw128(st + ks * a_step, a_lbo, 1024u);
              const uint64_t dal = smem_desc_sw128(st + kPairOpBytes + ks * a_step, a_lbo, 1024u);
              const uint64_t dbh = smem_desc_sw128(sbw + ks * b_step, b_lbo, 1024u);
              const uint64_t dbl = smem_desc_sw128(sbw + 2 * kPairOpBytes + ks * b_step, b_lbo, 1024u);
              mma_f16_ss(acc, dah, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
              mma_f16_ss(acc, dah, dbl, idesc, 1u);
              mma_f16_ss(acc, dal, dbh, idesc, 1u);
            }
          }
          const uint32_t sb = st + 4 * kPairOpBytes;
#pragma unroll
          for (int ks = 0; ks < (WIDE ? 0 : kPairBK / 16); ++ks) {
            const uint64_t dbh = smem_desc_sw128(sb + ks * b_step, b_lbo, 1024u);
            const uint64_t dbl = smem_desc_sw128(sb + kPairOpBytes + ks * b_step, b_lbo, 1024u);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t acc = tmem_d + (uint32_t)(((gg & 1) * 2 + h) * 128);
              const uint32_t sa = st + (uint32_t)h * 2 * kPairOpBytes;
              const uint64_t dah = smem_desc_sw128(sa + ks * a_step, a_lbo, 1024u);
              const uint64_t dal = smem_desc_sw128(sa + kPairOpBytes + ks * a_step, a_lbo, 1024u);
              mma_f16_ss(acc, dah, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
              mma_f16_ss(acc, dah, dbl, idesc, 1u);
              mma_f16_ss(acc, dal, dbh, idesc, 1u);
            }
          }
          mma_commit(&bar_empty[s]);
          if (kb % kPairGroup == kPairGroup - 1 || kb == t.KB - 1) {
            mma_commit(&bar_grp[gg & 1]);
            ++gg;
          }
        }
      }
    }
  } else {
    // ---- fold finished groups into the row's sums (registers), then the epilogue ---------------
    const int half = (warp - 2) >> 2;  // row half of the tile
    const int quarter = warp & 3;      // tensor-memory lanes 32*quarter..
    const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
    const uint32_t box = tiles + (uint32_t)kP2Stages * kP2StageBytes + (uint32_t)(warp - 2) * kPairBoxBytes;
    uint8_t *box_ptr = smem_dyn + (box - smem_u32(smem_dyn));
    bool ok = true;
    int gg = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
      const PairTile t = pair_tile256<Ext::kBatched, WIDE>(p, w);
      const int NG = (t.KB + kPairGroup - 1) / kPairGroup;
      // this warp's rows and first column (half = row half of the tile, or column half if WIDE)
      const int mw = t.m0 + (WIDE ? 0 : 128 * half) + 32 * quarter;
      const int nw = t.n0 + (WIDE ? 128 * half : 0);
      const int m = mw + lane;
      const bool row_ok = m < p.M && nw < p.N;
      typename Ext::Row rs;
      if (row_ok) {
        ext.row_begin(rs, t.z, m, nw);
        ext.prefetch(rs, t.z, m, nw);
      }
      float run[8][16];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 16; ++i) run[j][i] = 0.f;
      for (int g = 0; g < NG && ok; ++g, ++gg) {
        bool got = mbar_wait_watch(&bar_grp[gg & 1], (uint32_t)((gg >> 1) & 1), vfailed);
        got = __all_sync(0xffffffffu, got);
        if (!got) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // (WIDE: the same address -- columns 128 * half of accumulator (gg & 1) of 256 columns)
        const uint32_t acc = tmem_d + lane_base + (uint32_t)(((gg & 1) * 2 + half) * 128);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float pv[16];
          tmem_ld16_nowait(acc + 16 * j, pv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) run[j][i] += pv[i];
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_fold[gg & 1]);
      }
      ok = __all_sync(0xffffffffu, ok) && !*vfailed;
      if (!ok) *vfailed = 1;
      // epilogue from the registers: 32 columns -> policy -> swizzled 32 x 32 box -> TMA store
#pragma unroll
      for (int jb = 0; jb < 4; ++jb) {
        const int n = nw + 32 * jb;
        if (n < p.N) {  // warp-uniform
          if (row_ok) {
            ext.finish(rs, t.z, m, n, run[2 * jb], 0);
            if (n + 16 < p.N) ext.finish(rs, t.z, m, n + 16, run[2 * jb + 1], 1);
            if (jb < 3 && n + 32 < p.N) ext.prefetch(rs, t.z, m, n + 32);
          }
          if (!ok) {
#pragma unroll
            for (int i = 0; i < 16; ++i) run[2 * jb][i] = run[2 * jb + 1][i] = NAN;
          }
          // the store of the previous box must have read the staging buffer
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float4 *>(box_ptr + sw128_offset(lane, j)) =
                make_float4(run[2 * jb][4 * j], run[2 * jb][4 * j + 1], run[2 * jb][4 * j + 2], run[2 * jb][4 * j + 3]);
            *reinterpret_cast<float4 *>(box_ptr + sw128_offset(lane, 4 + j)) =
                make_float4(run[2 * jb + 1][4 * j], run[2 * jb + 1][4 * j + 1], run[2 * jb + 1][4 * j + 2],
                            run[2 * jb + 1][4 * j + 3]);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) tma_store_3d(&map_out, box, n, mw, t.z);
        }
      }
      if (row_ok) ext.row_end(rs, t.z, m, nw);
    }
    if (lane == 0) tma_store_wait_read();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, kPairCols);
}

// shape.tiles_m must count 256-row tiles (WIDE: 128-row tiles and shape.tiles_n 256-column
// tiles); out = [shape.nz][shape.M][shape.N] floats
template <bool A_MN, bool B_MN, class Ext, bool WIDE = false>
int launch_pair_umma256(const CUtensorMap &mah, const CUtensorMap &mal, const CUtensorMap &mbh,
                        const CUtensorMap &mbl, float *out, const LinShape &shape, const Ext &ext,
                        cudaStream_t st) {
  CUtensorMap mo;
  int rc = make_out_map(&mo, out, shape.nz, shape.M, shape.N);
  if (rc != FRNNT_OK) return rc;
  auto kern = pair_umma256_kernel<A_MN, B_MN, Ext, WIDE>;
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kP2SmemBytes));
  int ctas = 0;
  rc = lin_grid((long long)shape.tiles_m * shape.tiles_n * shape.nz, &ctas);
  if (rc != FRNNT_OK) return rc;
  if (ctas == 0) return FRNNT_OK;
  FRNNT_KERNEL(kern<<<ctas, kP2Threads, kP2SmemBytes, st>>>(mah, mal, mbh, mbl, mo, shape, ext));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

}  // namespace frnnt
