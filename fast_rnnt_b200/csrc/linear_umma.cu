// fp32-accurate (3xTF32) matrix products on the sm_100a tensor cores for plain
// row-major float matrices, fed by TMA.  Two entry points, the three products a
// linear layer needs (the joiner between do_rnnt_pruning and rnnt_loss_pruned):
//
//   frnnt_matmul_nt:  D[M][N] = A[M][K] * B[N][K]^T (+ bias[N])     forward, and
//                     grad_input = grad_out * W with B = W^T
//   frnnt_matmul_tn:  D[M][N] = A[R][M]^T * B[R][N]                 grad_weight,
//                     the long reduction over R is split over CTAs (partial sums
//                     in a caller scratch, added in a fixed order)
//
// Kernel structure (one 128x128 output tile per CTA, 14 warps):
//   warp 0   : TMA producer.  cp.async.bulk.tensor loads the raw fp32 operand
//              tiles of a 32-wide K slice into the 128-byte-swizzled layouts
//              (K-major: swizzle 128B; operands that are contiguous along M/N:
//              swizzle 128B with 32-byte atoms), completion on an mbarrier;
//              4-stage ring.
//   warps 2-9: split every landed value x into hi = tf32(x) and lo = tf32(x - hi),
//              both rounded to nearest.  B is split in shared memory (hi in place,
//              lo in a second buffer; an element-wise pass that does not care
//              about the tile layout).  A goes to TENSOR MEMORY: thread <-> row
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
//              and run the epilogue, tcgen05.ld -> (+bias) -> 64-byte row segments.
// No multicast, no clusters.  Every wait is bounded; a timeout poisons the tile.
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
// 2-D tiled TMA load: box at (x = innermost coordinate, y) -> shared memory, bytes counted on bar
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

struct LinParams {
  float *out;          // [splits][M][N] (splits == 1: the result itself)
  const float *bias;   // [N] or nullptr
  const float *tanh_out;  // [M][N] or nullptr: the result is multiplied by 1 - tanh_out^2
  int M, N, K;         // K = reduction length
  int k_per_split;     // multiple of kLinBK
  int tiles_m, tiles_n, splits;
};

// work item w -> (split, m tile, n tile); the n tiles of one m tile are neighbours, so
// the CTAs that run at the same time share their A rows in L2
struct LinTile {
  int m0, n0, z, KB, k_begin;
};
__device__ __forceinline__ LinTile lin_tile(const LinParams &p, int w) {
  LinTile t;
  const int per_split = p.tiles_m * p.tiles_n;
  t.z = w / per_split;
  const int r = w - t.z * per_split;
  t.m0 = (r / p.tiles_n) * kLinTile;
  t.n0 = (r % p.tiles_n) * kLinTile;
  t.k_begin = t.z * p.k_per_split;
  const int k_end = min(p.K, t.k_begin + p.k_per_split);
  t.KB = k_end > t.k_begin ? (k_end - t.k_begin + kLinBK - 1) / kLinBK : 0;
  return t;
}

// Persistent: CTA c works on items c, c + gridDim.x, ...; every role walks the same
// list, and the ring / accumulator indices run on across items, so the TMA producer,
// the split warps and the MMAs of the next tile start while the fold warps still
// write the previous tile out.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   LinParams p) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kLinStages];   // TMA bytes have landed
  __shared__ __align__(8) uint64_t bar_split[kLinStages];  // hi / lo are ready
  __shared__ __align__(8) uint64_t bar_empty[kLinStages];  // the MMAs are done with the stage
  __shared__ __align__(8) uint64_t bar_grp[2];             // a group's accumulator is complete
  __shared__ __align__(8) uint64_t bar_fold[2];            // ... and has been folded away
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = p.tiles_m * p.tiles_n * p.splits;
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
        const LinTile t = lin_tile(p, w);
        for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
          const int s = it % kLinStages;
          if (it >= kLinStages && !mbar_wait(&bar_empty[s], (uint32_t)((it / kLinStages - 1) & 1))) {
            *vfailed = 1;
            break;
          }
          const int k0 = t.k_begin + kb * kLinBK;
          const uint32_t st = tiles + (uint32_t)s * kLinStageBytes;
          mbar_expect_tx(&bar_full[s], 2 * kLinOpBytes);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_2d(st + j * 4096, &map_a, t.m0 + 32 * j, k0, &bar_full[s]);
          } else {
            tma_load_2d(st, &map_a, k0, t.m0, &bar_full[s]);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_2d(st + kLinOpBytes + j * 4096, &map_b, t.n0 + 32 * j, k0, &bar_full[s]);
          } else {
            tma_load_2d(st + kLinOpBytes, &map_b, k0, t.n0, &bar_full[s]);
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
        const LinTile t = lin_tile(p, w);
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
    int it = 0;
    for (int w = blockIdx.x; w < n_items && !*vfailed; w += gridDim.x) {
      const LinTile t = lin_tile(p, w);
      for (int kb = 0; kb < t.KB && !*vfailed; ++kb, ++it) {
        const int s = it % kLinStages;
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
        // B: split in place (hi) and into the second buffer (lo); the layout does not matter
#pragma unroll
        for (int q = 0; q < kChunksPerThread; ++q) {
          float4 h, l;
          split_tf32(x[q], h, l);
          braw[st_tid + q * 32 * kLinWorkers] = h;
          blo[st_tid + q * 32 * kLinWorkers] = l;
        }
        // A: this thread's row, 16 of the 32 k values, hi and lo into tensor memory
        float hi[16], lo[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) split_tf32(av[i], hi[i], lo[i]);
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
      const LinTile t = lin_tile(p, w);
      const int NG = (t.KB + kLinGroup - 1) / kLinGroup;
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
      const int m = t.m0 + 32 * quarter + lane;
      float *out = p.out + (size_t)t.z * p.M * p.N;
      const bool row_ok = m < p.M;
      // 32 columns per round: the loads of the tanh values of a whole round are issued
      // before the first accumulator read, so their latency is paid four times per
      // tile, not once per 16 columns
      for (int c0 = 0; c0 < kLinTile; c0 += 32) {
        float4 tv[8];
        const bool tanh_vec = p.tanh_out != nullptr && vec && row_ok && t.n0 + c0 + 32 <= p.N;
        if (tanh_vec) {
          const float4 *a4 = reinterpret_cast<const float4 *>(p.tanh_out + (size_t)m * p.N + t.n0 + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) tv[i] = a4[i];
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int ch = c0 / 16 + cc;
          float v[16];
          if (ok && t.KB > 0) {
            tmem_ld16(run + (uint32_t)(ch * 16), v);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = ok ? 0.f : NAN;
          }
          const int n = t.n0 + ch * 16;
          if (row_ok && n < p.N) {
            if (p.bias != nullptr) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n + i < p.N) v[i] += p.bias[n + i];
            }
            if (tanh_vec) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float4 tt = tv[4 * cc + i];
                v[4 * i] *= 1.f - tt.x * tt.x;
                v[4 * i + 1] *= 1.f - tt.y * tt.y;
                v[4 * i + 2] *= 1.f - tt.z * tt.z;
                v[4 * i + 3] *= 1.f - tt.w * tt.w;
              }
            } else if (p.tanh_out != nullptr) {
              const float *a = p.tanh_out + (size_t)m * p.N + n;
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n + i < p.N) v[i] *= 1.f - a[i] * a[i];
            }
            float *dst = out + (size_t)m * p.N + n;
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

// out[i] = sum over splits of partial[z][i], z in order
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                     long long n, int splits) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0;
  for (int z = 0; z < splits; ++z) acc += partial[(size_t)z * n + i];
  out[i] = acc;
}

// ---- host -----------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
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

// map of a row-major float matrix [rows][cols]; box = box_cols x box_rows
static int make_map(CUtensorMap *map, const float *base, int rows, int cols, int box_cols,
                    int box_rows, bool atom32) {
  auto enc = tensor_map_encoder();
  FRNNT_REQUIRE(enc != nullptr, FRNNT_ECUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FRNNT_REQUIRE(r == CUDA_SUCCESS, FRNNT_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return FRNNT_OK;
}

// one persistent CTA per SM (shared memory and tensor memory allow no more), fewer when
// there are fewer work items
static int lin_grid(long long items, int *ctas) {
  static int sm_count[64] = {0};
  int dev = 0;
  FRNNT_CUDA(cudaGetDevice(&dev));
  FRNNT_REQUIRE(dev >= 0 && dev < 64, FRNNT_EUNSUPPORTED, "device index %d too large", dev);
  if (sm_count[dev] == 0) {
    int n = 0;
    FRNNT_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    FRNNT_REQUIRE(n > 0, FRNNT_ECUDA, "no multiprocessors reported");
    sm_count[dev] = n;
  }
  *ctas = (int)(items < sm_count[dev] ? items : sm_count[dev]);
  return FRNNT_OK;
}

static int check_matrix(const void *p, int cols, const char *what) {
  FRNNT_REQUIRE(p != nullptr, FRNNT_EINVAL, "%s is NULL", what);
  FRNNT_REQUIRE((uintptr_t)p % 16 == 0 && cols % 4 == 0, FRNNT_EUNSUPPORTED,
                "%s: TMA needs a 16-byte aligned base and a row length that is a multiple of 4 floats",
                what);
  return FRNNT_OK;
}

}  // namespace frnnt

using namespace frnnt;

extern "C" int frnnt_matmul_nt(const float *a, const float *b, const float *bias,
                               const float *tanh_out, float *d, int M, int N, int K, void *stream) {
  FRNNT_REQUIRE(M >= 0 && N >= 0 && K >= 0, FRNNT_EINVAL, "negative size");
  if (M == 0 || N == 0) return FRNNT_OK;
  FRNNT_REQUIRE(K > 0, FRNNT_EINVAL, "K must be positive");
  int rc = check_matrix(a, K, "a");
  if (rc == FRNNT_OK) rc = check_matrix(b, K, "b");
  if (rc != FRNNT_OK) return rc;
  FRNNT_REQUIRE(d != nullptr && (uintptr_t)d % 16 == 0, FRNNT_EINVAL, "d is NULL or misaligned");
  CUtensorMap ma, mb;
  rc = make_map(&ma, a, M, K, kLinBK, kLinTile, false);
  if (rc == FRNNT_OK) rc = make_map(&mb, b, N, K, kLinBK, kLinTile, false);
  if (rc != FRNNT_OK) return rc;
  auto kern = linear_umma_kernel<false, false>;
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemBytes));
  const int mt = (M + kLinTile - 1) / kLinTile, nt = (N + kLinTile - 1) / kLinTile;
  LinParams p{d, bias, tanh_out, M, N, K, ((K + kLinBK - 1) / kLinBK) * kLinBK, mt, nt, 1};
  int ctas = 0;
  rc = lin_grid(mt * nt, &ctas);
  if (rc != FRNNT_OK) return rc;
  FRNNT_KERNEL(kern<<<ctas, kLinThreads, kLinSmemBytes, (cudaStream_t)stream>>>(ma, mb, p));
  FRNNT_CUDA(cudaGetLastError());
  return FRNNT_OK;
}

extern "C" int frnnt_matmul_tn_splits(int M, int N, int R) {
  if (M <= 0 || N <= 0 || R <= 0) return 1;
  const int tiles = ((M + kLinTile - 1) / kLinTile) * ((N + kLinTile - 1) / kLinTile);
  int splits = (2 * 148) / tiles;   // at most two CTAs per SM (one is resident at a time): two full waves
  const int max_splits = (R + 8 * kLinBK - 1) / (8 * kLinBK);  // at least 8 K slices per CTA
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  return splits;
}

extern "C" int frnnt_matmul_tn(const float *a, const float *b, float *d, float *partials, int M,
                               int N, int R, void *stream) {
  FRNNT_REQUIRE(M >= 0 && N >= 0 && R >= 0, FRNNT_EINVAL, "negative size");
  if (M == 0 || N == 0) return FRNNT_OK;
  FRNNT_REQUIRE(R > 0, FRNNT_EINVAL, "R must be positive");
  int rc = check_matrix(a, M, "a");
  if (rc == FRNNT_OK) rc = check_matrix(b, N, "b");
  if (rc != FRNNT_OK) return rc;
  FRNNT_REQUIRE(d != nullptr && (uintptr_t)d % 16 == 0, FRNNT_EINVAL, "d is NULL or misaligned");
  const int splits = frnnt_matmul_tn_splits(M, N, R);
  FRNNT_REQUIRE(splits == 1 || (partials != nullptr && (uintptr_t)partials % 16 == 0), FRNNT_EINVAL,
                "partials scratch of splits*M*N floats is required");
  CUtensorMap ma, mb;
  // operands contiguous along M / N: boxes of 32 values x 32 reduction rows, 32-byte swizzle atoms
  rc = make_map(&ma, a, R, M, 32, kLinBK, true);
  if (rc == FRNNT_OK) rc = make_map(&mb, b, R, N, 32, kLinBK, true);
  if (rc != FRNNT_OK) return rc;
  auto kern = linear_umma_kernel<true, true>;
  FRNNT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLinSmemBytes));
  const int mt = (M + kLinTile - 1) / kLinTile, nt = (N + kLinTile - 1) / kLinTile;
  const int kblocks = (R + kLinBK - 1) / kLinBK;
  const int k_per_split = ((kblocks + splits - 1) / splits) * kLinBK;
  LinParams p{splits == 1 ? d : partials, nullptr, nullptr, M, N, R, k_per_split, mt, nt, splits};
  cudaStream_t st = (cudaStream_t)stream;
  int ctas = 0;
  rc = lin_grid(mt * nt * splits, &ctas);
  if (rc != FRNNT_OK) return rc;
  FRNNT_KERNEL(kern<<<ctas, kLinThreads, kLinSmemBytes, st>>>(ma, mb, p));
  FRNNT_CUDA(cudaGetLastError());
  if (splits > 1) {
    const long long n = (long long)M * N;
    FRNNT_KERNEL(splitk_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partials, d, n, splits));
    FRNNT_CUDA(cudaGetLastError());
  }
  return FRNNT_OK;
}
