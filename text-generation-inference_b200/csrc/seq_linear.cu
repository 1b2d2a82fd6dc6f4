// C[z][m][n] = sum_k A[z][m][k] * W[z][n][k] (+ bias[n]) for bfloat16 / float operands in any combination, fp32 accumulation
// in ascending k, so a row's result does not depend on how many other rows the call has (batch invariance), and the fp32
// instance is a true 32-bit product.  `z` strides let one launch do a per-head product on slices of wider activations
// (the latent-attention up-projections).  Tiles of 64 x 64 outputs, 16-wide k steps through shared memory, 4 x 4 outputs
// per thread.
#include "seq_common.cuh"

namespace b200 {
namespace seq {

constexpr int kTile = 64, kStep = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) linear_kernel(const TA* __restrict__ A, int64_t lda, int64_t sA, const TW* __restrict__ W, int64_t ldw,
                                                     int64_t sW, const TW* __restrict__ bias, TC* __restrict__ C, int64_t ldc, int64_t sC,
                                                     int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[kStep][kTile + 4];
  __shared__ float Ws[kStep][kTile + 4];
  const int z = blockIdx.z;
  A += (int64_t)z * sA;
  W += (int64_t)z * sW;
  C += (int64_t)z * sC;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row of the tile, first of 4 consecutive k
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kStep) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + i][lr] = (m < M && k < K) ? ldf(A + (int64_t)m * lda + k) : 0.f;
      Ws[lk + i][lr] = (n < N && k < K) ? ldf(W + (int64_t)n * ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kStep; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[k][ty * 4 + i];
        w[i] = Ws[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stf(C + (int64_t)m * ldc + n, acc[i][j] + (bias ? ldf(bias + n) : 0.f));
    }
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

template <typename TA, typename TW, typename TC>
static int launch_linear(const void* A, int64_t lda, int64_t sA, const void* W, int64_t ldw, int64_t sW, const void* bias, void* C, int64_t ldc,
                         int64_t sC, int64_t M, int64_t N, int64_t K, int64_t Z, cudaStream_t st) {
  dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)((M + kTile - 1) / kTile), (unsigned)Z);
  B200_LAUNCH((linear_kernel<TA, TW, TC>), grid, dim3(256), 0, st, (const TA*)A, lda, sA, (const TW*)W, ldw, sW, (const TW*)bias, (TC*)C, ldc, sC,
              (int)M, (int)N, (int)K);
  b200_count_launches(1);
  return B200_OK;
}

// a_dt / w_dt / c_dt: B200_DT_*.  Strides in elements.  Z independent products (z strides may be 0 for a shared operand).
extern "C" int b200_seq_linear(const void* A, int a_dt, int64_t lda, int64_t strideA, const void* W, int w_dt, int64_t ldw, int64_t strideW,
                               const void* bias, void* C, int c_dt, int64_t ldc, int64_t strideC, int64_t M, int64_t N, int64_t K, int64_t Z,
                               void* stream) {
  if (M == 0 || N == 0 || Z == 0) return B200_OK;
  if (M < 0 || N < 0 || K <= 0 || Z < 0 || (M + kTile - 1) / kTile > 65535 || Z > 65535) {
    b200_set_last_error("seq_linear: bad sizes");
    return B200_ERR_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int key = a_dt * 4 + w_dt * 2 + c_dt;
#define CASE(a, w, c, TA, TW, TC) \
  case a * 4 + w * 2 + c: return launch_linear<TA, TW, TC>(A, lda, strideA, W, ldw, strideW, bias, C, ldc, strideC, M, N, K, Z, st)
  switch (key) {
    CASE(0, 0, 0, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    CASE(0, 0, 1, __nv_bfloat16, __nv_bfloat16, float);
    CASE(1, 0, 0, float, __nv_bfloat16, __nv_bfloat16);
    CASE(1, 0, 1, float, __nv_bfloat16, float);
    CASE(1, 1, 1, float, float, float);
    default: break;
  }
#undef CASE
  b200_set_last_error("seq_linear: unsupported combination of element types");
  return B200_ERR_UNSUPPORTED;
}
