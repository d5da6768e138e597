// A batched 128x128-tile contraction on the sm_100a tensor cores with fp32
// accuracy (3xTF32) whose operands are produced on the fly:
//
//     D[m][n] = sum_k A(m,k) * B(n,k)
//
// A policy supplies, per operand, a function that returns four transformed
// values that are contiguous in memory -- along K ("K-major") or along M/N
// ("MN-major") -- and consumes the accumulator 16 columns at a time.  The
// kernel stages the values (split into tf32 hi + fp32 remainder) in the
// 128-byte-swizzled canonical layouts, issues tcgen05.mma from one thread with
// the accumulator in tensor memory, and keeps fp32 accuracy over long K by
// giving every 64-wide K group a fresh accumulator that is folded into a
// running sum with round-to-nearest adds (the tensor core itself adds with
// truncation).  All waits are bounded.
//
// Policy interface (all __device__):
//   static constexpr bool A_MN, B_MN;      operand is contiguous along M/N (true) or K (false)
//   void  init(int batch);                  select the batch
//   int   K() const;
//   Raw4  a_raw(int m, int k) const;        A_MN: (m..m+3, k)   else: (m, k..k+3): the loads only
//   float4 a_fix(const Raw4&) const;        the arithmetic on them (zeros outside the matrix)
//   Raw4  b_raw(int n, int k) const;  float4 b_fix(const Raw4&) const;      likewise
//     (split so that the loads of the next stage stay in flight across the
//      barrier and the MMA issue of the current one)
//   void  store(int m, int n0, const float (&acc)[16]);   columns n0..n0+15 of row m
//   void  poison(int m, int n0);            same footprint, called instead of store on a timeout
#pragma once
#include "umma.cuh"

namespace frnnt {
namespace umma {

constexpr int kGemmThreads = 256;
constexpr int kGemmTile = 128;   // M and N of a CTA tile
constexpr int kGemmBK = 32;      // K per stage
constexpr int kGemmStages = 2;
constexpr int kGemmGroup = 2;    // stages per accumulator group (K = 64)
// four raw values plus one per-row scalar (e.g. the row maximum an exp() needs)
struct Raw4 {
  float4 v;
  float aux;
};

constexpr size_t kGemmSmemBytes = (size_t)kGemmStages * 4 * kGemmTile * 128 + 1024;

template <class Pol>
__global__ void __launch_bounds__(kGemmThreads, 1) umma_gemm_kernel(Pol pol) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_mma[kGemmStages];
  __shared__ __align__(8) uint64_t bar_grp[2];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * kGemmTile, n0 = blockIdx.z * kGemmTile;
  pol.init(blockIdx.y);
  constexpr uint32_t kCols = 512, kAcc1 = 128, kRun = 256;
  const uint32_t idesc = idesc_tf32(kGemmTile, kGemmTile, Pol::A_MN, Pol::B_MN);

  const uint32_t tiles = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  constexpr uint32_t op_bytes = kGemmTile * 128;          // one operand tile (hi or lo)
  constexpr uint32_t stage_bytes = 4 * op_bytes;          // A_hi, A_lo, B_hi, B_lo
  uint8_t *tiles_ptr = smem_dyn + (tiles - smem_u32(smem_dyn));

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) mbar_init(&bar_mma[s], 1);
    mbar_init(&bar_grp[0], 1);
    mbar_init(&bar_grp[1], 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&tmem_slot, kCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  const int K = pol.K();
  const int KB = (K + kGemmBK - 1) / kGemmBK;
  const int NG = (KB + kGemmGroup - 1) / kGemmGroup;

  // staging assignment of this thread, four 16-byte chunks per operand and stage:
  //   K-major : rows (tid>>3) + 32q, k chunk (tid&7)
  //   MN-major: k rows (tid>>5) + 8q, mn chunk (tid&31)
  Raw4 ra[4], rb4[4];
  auto load_stage = [&](int kb) {
    const int k0 = kb * kGemmBK;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      ra[q] = Pol::A_MN ? pol.a_raw(m0 + 4 * (tid & 31), k0 + (tid >> 5) + 8 * q)
                        : pol.a_raw(m0 + (tid >> 3) + 32 * q, k0 + 4 * (tid & 7));
      rb4[q] = Pol::B_MN ? pol.b_raw(n0 + 4 * (tid & 31), k0 + (tid >> 5) + 8 * q)
                         : pol.b_raw(n0 + (tid >> 3) + 32 * q, k0 + 4 * (tid & 7));
    }
  };
  auto stage_offset = [&](bool mn, int q) -> uint32_t {
    return mn ? mn_tile_offset((tid >> 5) + 8 * q, tid & 31)
              : sw128_offset((tid >> 3) + 32 * q, tid & 7);
  };

  const int quarter = warp & 3, half = warp >> 2;
  constexpr int nchunks = kGemmTile / 16;
  const int ch_lo = half * (nchunks / 2), ch_hi = ch_lo + nchunks / 2;
  const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
  auto fold_group = [&](int g, bool first) {
    const uint32_t acc = tmem_base + lane_base + ((g & 1) ? kAcc1 : 0u);
    const uint32_t run = tmem_base + lane_base + kRun;
    for (int ch = ch_lo; ch < ch_hi; ++ch) {
      float p[16], r[16];
      tmem_ld16(acc + ch * 16, p);
      if (!first) {
        tmem_ld16(run + ch * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) p[i] = r[i] + p[i];
      }
      tmem_st16(run + ch * 16, p);
    }
  };

  load_stage(0);
  int failed = 0;
  for (int kb = 0; kb < KB; ++kb) {
    const int stage = kb % kGemmStages;
    const int g = kb / kGemmGroup;
    const bool group_start = kb % kGemmGroup == 0;
    if (kb >= kGemmStages && !mbar_wait(&bar_mma[stage], (uint32_t)((kb / kGemmStages - 1) & 1)))
      failed = 1;
    uint8_t *st = tiles_ptr + (size_t)stage * stage_bytes;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float4 hi, lo;
      split_tf32(pol.a_fix(ra[q]), hi, lo);
      uint32_t o = stage_offset(Pol::A_MN, q);
      *reinterpret_cast<float4 *>(st + o) = hi;
      *reinterpret_cast<float4 *>(st + op_bytes + o) = lo;
      split_tf32(pol.b_fix(rb4[q]), hi, lo);
      o = stage_offset(Pol::B_MN, q);
      *reinterpret_cast<float4 *>(st + 2 * op_bytes + o) = hi;
      *reinterpret_cast<float4 *>(st + 3 * op_bytes + o) = lo;
    }
    if (kb + 1 < KB) load_stage(kb + 1);
    if (group_start && g >= 2 && !failed) {
      if (mbar_wait(&bar_grp[g & 1], (uint32_t)(((g - 2) >> 1) & 1))) {
        tc_fence_after_sync();
        fold_group(g - 2, g == 2);
      } else {
        failed = 1;
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    failed = __syncthreads_or(failed);
    if (failed) break;
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t acc = tmem_base + ((g & 1) ? kAcc1 : 0u);
      const uint32_t sa = tiles + (uint32_t)stage * stage_bytes;
#pragma unroll
      for (int ks = 0; ks < kGemmBK / 8; ++ks) {
        // one K = 8 step: 32 bytes along the rows (K-major) or two 4-row atoms (MN-major)
        const uint32_t ao = Pol::A_MN ? ks * 1024u : ks * 32u;
        const uint32_t bo = Pol::B_MN ? ks * 1024u : ks * 32u;
        const uint32_t a_lbo = Pol::A_MN ? 4096u : 16u, b_lbo = Pol::B_MN ? 4096u : 16u;
        const uint32_t a_sbo = Pol::A_MN ? 512u : 1024u, b_sbo = Pol::B_MN ? 512u : 1024u;
        const uint32_t a_lt = Pol::A_MN ? 1u : 2u, b_lt = Pol::B_MN ? 1u : 2u;
        const uint64_t dah = smem_desc_sw128(sa + ao, a_lbo, a_sbo, a_lt);
        const uint64_t dal = smem_desc_sw128(sa + op_bytes + ao, a_lbo, a_sbo, a_lt);
        const uint64_t dbh = smem_desc_sw128(sa + 2 * op_bytes + bo, b_lbo, b_sbo, b_lt);
        const uint64_t dbl = smem_desc_sw128(sa + 3 * op_bytes + bo, b_lbo, b_sbo, b_lt);
        mma_tf32(acc, dah, dbh, idesc, (!group_start || ks > 0) ? 1u : 0u);
        mma_tf32(acc, dah, dbl, idesc, 1u);
        mma_tf32(acc, dal, dbh, idesc, 1u);
      }
      mma_commit(&bar_mma[stage]);
      if (kb % kGemmGroup == kGemmGroup - 1 || kb == KB - 1) mma_commit(&bar_grp[g & 1]);
    }
  }

  if (!failed && KB > 0) {
    if (NG >= 2 && !mbar_wait(&bar_grp[(NG - 2) & 1], (uint32_t)(((NG - 2) >> 1) & 1))) failed = 1;
    if (!mbar_wait(&bar_grp[(NG - 1) & 1], (uint32_t)(((NG - 1) >> 1) & 1))) failed = 1;
  }
  failed = __syncthreads_or(failed);
  tc_fence_after_sync();

  {
    const int m = m0 + 32 * quarter + lane;
    const uint32_t acc0 = tmem_base + lane_base, acc1 = acc0 + kAcc1, run = acc0 + kRun;
    for (int ch = ch_lo; ch < ch_hi; ++ch) {
      float v[16];
      if (failed) {
        pol.poison(m, n0 + ch * 16);
        continue;
      }
      if (NG >= 3) {
        float p[16];
        tmem_ld16(run + ch * 16, v);
        tmem_ld16(((NG - 2) & 1 ? acc1 : acc0) + ch * 16, p);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += p[i];
        tmem_ld16(((NG - 1) & 1 ? acc1 : acc0) + ch * 16, p);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += p[i];
      } else if (NG == 2) {
        float p[16];
        tmem_ld16(acc0 + ch * 16, v);
        tmem_ld16(acc1 + ch * 16, p);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += p[i];
      } else if (NG == 1) {
        tmem_ld16(acc0 + ch * 16, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      pol.store(m, n0 + ch * 16, v);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kCols);
}

}  // namespace umma
}  // namespace frnnt
