// True 32-bit matrix product for the float32 path:  C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
//
// Plain FMA on CUDA cores: no tensor cores, no TF32, no split accumulation. Each output
// element is one chain of FMAs over k = 0..K-1 in order, so a row's result does not depend on
// how many other rows are in the call. Linear layers are x * W^T with W stored
// [out_features, in_features] (python/instinct/backends/base.py:83-101).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kGemmThreads = (BM / TM) * (BN / TN);  // 256

__device__ __forceinline__ void load_tile(const float* __restrict__ src, int rows, int ld, int K,
                                          int row0, int k0, bool vec, float (*dst)[BM + 4]) {
  // 64 rows x 16 k: each thread brings 4 consecutive k of one row and stores them transposed.
  const int r = threadIdx.x >> 2;
  const int kk = (threadIdx.x & 3) * 4;
  const int row = row0 + r;
  const int k = k0 + kk;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (row < rows) {
    const float* p = src + static_cast<int64_t>(row) * ld + k;
    if (vec && k + 3 < K) {
      const float4 f = *reinterpret_cast<const float4*>(p);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (k + i < K) v[i] = p[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[kk + i][r] = v[i];
}

__global__ void __launch_bounds__(kGemmThreads)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, float* __restrict__ C, int M, int N, int K,
                int lda, int ldw, int ldc, bool vec) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int ty = threadIdx.x / (BN / TN), tx = threadIdx.x % (BN / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    load_tile(A, M, lda, K, m0, k0, vec, As);
    load_tile(W, N, ldw, K, n0, k0, vec, Ws);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[static_cast<int64_t>(m) * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace

B200_API int b200_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M,
                           int N, int K, int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  B200_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_f32: bad sizes %d x %d x %d", M, N, K);
  B200_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: leading dimensions too small");
  const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) &&
                   (reinterpret_cast<uintptr_t>(A) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(W) % 16 == 0);
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  B200_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows (%d)", M);
  gemm_f32_kernel<<<grid, kGemmThreads, 0, stream>>>(A, W, bias, C, M, N, K, lda, ldw, ldc, vec);
  return b200_check_launch("gemm_f32");
}
