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
// Both run on the engine in umma_linear.cuh (persistent, TMA-fed, A operand through
// tensor memory, grouped accumulators); this file adds the epilogue of a linear layer.
#include "umma_linear.cuh"

namespace frnnt {

// (+ bias[n]) and, for the gradient that flows back through tanh, * (1 - tanh_out^2)
template <bool COLSUM>
struct PlainLinearExt {
  static constexpr bool kBatched = false, kExpB = false, kColSumA = COLSUM;
  float *out;             // [splits][M][N] (splits == 1: the result itself)
  const float *bias;      // [N] or nullptr
  const float *tanh_out;  // [M][N] or nullptr
  float *colsum;          // [splits][2][M] partial sums of A over its rows, or nullptr
  int M, N;
  __device__ float *a_colsum(int z, int half) const {
    return colsum != nullptr ? colsum + ((size_t)z * 2 + half) * M : nullptr;
  }
  __device__ const float *b_shift(int) const { return nullptr; }
  __device__ const float *pre_row(int, int m) const {
    return tanh_out != nullptr ? tanh_out + (size_t)m * N : nullptr;
  }
  __device__ float *out_row(int z, int m) const { return out + ((size_t)z * M + m) * N; }
  __device__ void finish(int, int, int n, float (&v)[16], const float (&x)[16]) const {
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (n + i < N) v[i] += bias[n + i];
    }
    if (tanh_out != nullptr) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] *= 1.f - x[i] * x[i];
    }
  }
};

// out[i] = sum over splits of partial[z][i], z in order
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ out,
                                     long long n, int splits) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0;
  for (int z = 0; z < splits; ++z) acc += partial[(size_t)z * n + i];
  out[i] = acc;
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
  rc = make_operand_map(&ma, a, M, K, K, 0, 0, false);
  if (rc == FRNNT_OK) rc = make_operand_map(&mb, b, N, K, K, 0, 0, false);
  if (rc != FRNNT_OK) return rc;
  const int mt = (M + kLinTile - 1) / kLinTile, nt = (N + kLinTile - 1) / kLinTile;
  const LinShape shape{M, N, K, ((K + kLinBK - 1) / kLinBK) * kLinBK, mt, nt, 1};
  const PlainLinearExt<false> ext{d, bias, tanh_out, nullptr, M, N};
  return launch_linear_umma<false, false>(ma, mb, shape, ext, (cudaStream_t)stream);
}

extern "C" int frnnt_matmul_tn_splits(int M, int N, int R) {
  if (M <= 0 || N <= 0 || R <= 0) return 1;
  // The persistent CTAs (one per SM) take the tiles x splits work items
  // round-robin, so the time is ceil(items / SMs) item lengths, an item being 1 / splits
  // of the reduction: pick the split count that minimises it, with a small price per
  // split for the partial sums, and at least 8 K slices per item.
  const long long tiles = (long long)((M + kLinTile - 1) / kLinTile) * ((N + kLinTile - 1) / kLinTile);
  const int max_splits = (R + 8 * kLinBK - 1) / (8 * kLinBK);
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

extern "C" size_t frnnt_matmul_tn_scratch_floats(int M, int N, int R) {
  if (M <= 0 || N <= 0 || R <= 0) return 0;
  const size_t splits = (size_t)frnnt_matmul_tn_splits(M, N, R);
  return (splits > 1 ? splits * M * N : 0) + 2 * splits * M;
}

extern "C" int frnnt_matmul_tn_colsum(const float *a, const float *b, float *d, float *a_colsum,
                                      float *scratch, int M, int N, int R, void *stream) {
  FRNNT_REQUIRE(M >= 0 && N >= 0 && R >= 0, FRNNT_EINVAL, "negative size");
  if (M == 0 || N == 0) return FRNNT_OK;
  FRNNT_REQUIRE(R > 0, FRNNT_EINVAL, "R must be positive");
  int rc = check_matrix(a, M, "a");
  if (rc == FRNNT_OK) rc = check_matrix(b, N, "b");
  if (rc != FRNNT_OK) return rc;
  FRNNT_REQUIRE(d != nullptr && (uintptr_t)d % 16 == 0, FRNNT_EINVAL, "d is NULL or misaligned");
  const int splits = frnnt_matmul_tn_splits(M, N, R);
  FRNNT_REQUIRE((splits == 1 && a_colsum == nullptr) || (scratch != nullptr && (uintptr_t)scratch % 16 == 0),
                FRNNT_EINVAL, "a scratch of frnnt_matmul_tn_scratch_floats() floats is required");
  float *partials = splits > 1 ? scratch : nullptr;
  float *cs_partials = a_colsum != nullptr ? scratch + (splits > 1 ? (size_t)splits * M * N : 0) : nullptr;
  CUtensorMap ma, mb;
  // operands contiguous along M / N: boxes of 32 values x 32 reduction rows, 32-byte swizzle atoms
  rc = make_operand_map(&ma, a, R, M, M, 0, 0, true);
  if (rc == FRNNT_OK) rc = make_operand_map(&mb, b, R, N, N, 0, 0, true);
  if (rc != FRNNT_OK) return rc;
  const int mt = (M + kLinTile - 1) / kLinTile, nt = (N + kLinTile - 1) / kLinTile;
  const int kblocks = (R + kLinBK - 1) / kLinBK;
  const int k_per_split = ((kblocks + splits - 1) / splits) * kLinBK;
  const LinShape shape{M, N, R, k_per_split, mt, nt, splits};
  cudaStream_t st = (cudaStream_t)stream;
  float *out = splits == 1 ? d : partials;
  if (a_colsum != nullptr)
    rc = launch_linear_umma<true, true>(ma, mb, shape, PlainLinearExt<true>{out, nullptr, nullptr, cs_partials, M, N}, st);
  else
    rc = launch_linear_umma<true, true>(ma, mb, shape, PlainLinearExt<false>{out, nullptr, nullptr, nullptr, M, N}, st);
  if (rc != FRNNT_OK) return rc;
  if (splits > 1) {
    const long long n = (long long)M * N;
    FRNNT_KERNEL(splitk_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partials, d, n, splits));
    FRNNT_CUDA(cudaGetLastError());
  }
  if (a_colsum != nullptr) {
    FRNNT_KERNEL(splitk_reduce_kernel<<<(unsigned)((M + 255) / 256), 256, 0, st>>>(cs_partials, a_colsum, M,
                                                                              2 * splits));
    FRNNT_CUDA(cudaGetLastError());
  }
  return FRNNT_OK;
}

extern "C" int frnnt_matmul_tn(const float *a, const float *b, float *d, float *partials, int M,
                               int N, int R, void *stream) {
  return frnnt_matmul_tn_colsum(a, b, d, nullptr, partials, M, N, R, stream);
}
