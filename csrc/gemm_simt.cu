// D[M, N] = A[M, K] B[N, K]^T in true fp32 (FFMA, sequential-k accumulation per output): the exact-precision path for
// fp32 inference, where the tensor-core route would round the operands to TF32. 64 x 64 tiles, 16-deep k steps, 4 x 4
// outputs per thread; any M, N, K and any row strides.
#include "common.cuh"
#include "../include/b200_ops.h"

namespace b200 {
constexpr int kSB = 64, kSK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ D, int M, int N, int K,
                long long lda, long long ldb, long long ldd) {
  __shared__ float As[kSK][kSB + 4];
  __shared__ float Bs[kSK][kSB + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * kSB, n0 = blockIdx.x * kSB;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kSK) {
    for (int i = threadIdx.x; i < kSB * kSK; i += 256) {
      const int r = i / kSK, c = i % kSK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(long long)gm * lda + gk] : 0.f;
      Bs[c][r] = (gn < N && gk < K) ? B[(long long)gn * ldb + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kSK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) D[(long long)gm * ldd + gn] = acc[i][j];
    }
}
}  // namespace b200

B200_API int b200_gemm_f32_exact(const float* A, const float* B, float* D, int M, int N, int K, long long lda, long long ldb,
                                 long long ldd, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return B200_ERR_BAD_SHAPE;
  dim3 grid((N + b200::kSB - 1) / b200::kSB, (M + b200::kSB - 1) / b200::kSB);
  b200::gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, B, D, M, N, K, lda, ldb, ldd);
  B200_LAUNCH_CHECK();
  return 0;
}
