// Matrix product for a handful of tokens (decode steps):  Y[M,N] = X[M,K] * W[N,K]^T, M <= 64.
//
// With so few rows the product is a stream of the weight matrix through the GPU once, so the
// kernel is built around that stream. The roles of the operands are swapped for the tensor
// cores: 16 rows of W are the "A" tile of mma.sync m16n8k16 and 8 tokens are its "B" tile.
// Each lane fetches its share of a 16 x 32 slab of W with two 16-byte loads straight from
// global memory into fragment registers (the order of k inside a slab is permuted the same
// way for W and X, which a dot product does not notice), several slabs ahead, so that every
// warp keeps a few KB in flight. The 8 warps of a block are `row_groups` groups of 16 weight
// rows times `k_splits` slices of K; the slices' partial sums meet in shared memory and are
// added in slice order, so the result does not depend on timing. Linear layers are x W^T with
// W stored [out, in] (python/instinct/backends/base.py:83-101); the reference sends them to
// cuBLASLt (cuda/execution_context.cu:95-110).
//
// Epilogues: bfloat16 or float32 rows of Y, or SwiGLU over interleaved rows of W (row 2j is
// gate_j, row 2j + 1 is up_j): out[m, j] = silu(y[m, 2j]) * y[m, 2j + 1]
// (python/instinct/backends/dense.py:124-128).
#include "common.cuh"

namespace {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyThreads = kSkinnyWarps * 32;
constexpr int kChunk = 32;  // k per slab
constexpr int kAhead = 4;   // slabs fetched ahead per warp

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int MT>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                   void* __restrict__ Y, int M, int N, int K, int row_groups, int epilogue) {
  extern __shared__ float partial[];  // [k_splits][row_groups * 16][MT * 8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k_splits = kSkinnyWarps / row_groups;
  const int rg = warp % row_groups, ks = warp / row_groups;
  const int block_rows = row_groups * 16;
  const int n0 = blockIdx.x * block_rows + rg * 16;

  const int chunks = (K + kChunk - 1) / kChunk;
  const int per_split = (chunks + k_splits - 1) / k_splits;
  const int c_begin = ks * per_split, c_end = min(chunks, c_begin + per_split);

  const int row_a = n0 + g, row_b = n0 + g + 8;
  const bool live_a = row_a < N, live_b = row_b < N;
  const __nv_bfloat16* wa = W + static_cast<int64_t>(live_a ? row_a : 0) * K + t * 8;
  const __nv_bfloat16* wb = W + static_cast<int64_t>(live_b ? row_b : 0) * K + t * 8;

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  uint4 fa[kAhead], fb[kAhead];
#pragma unroll
  for (int i = 0; i < kAhead; ++i) {
    const int c = c_begin + i;
    const bool in = c < c_end && c * kChunk + t * 8 < K;
    fa[i] = (in && live_a) ? load_stream(wa + c * kChunk) : zero;
    fb[i] = (in && live_b) ? load_stream(wb + c * kChunk) : zero;
  }

  for (int c0 = c_begin; c0 < c_end; c0 += kAhead) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const int c = c0 + i;
      if (c >= c_end) break;
      const uint4 a = fa[i], b = fb[i];
      // Refill this slot with the slab kAhead further on.
      {
        const int cn = c + kAhead;
        const bool in = cn < c_end && cn * kChunk + t * 8 < K;
        fa[i] = (in && live_a) ? load_stream(wa + cn * kChunk) : zero;
        fb[i] = (in && live_b) ? load_stream(wb + cn * kChunk) : zero;
      }
      const bool k_in = c * kChunk + t * 8 < K;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int token = mt * 8 + g;
        uint4 x = zero;
        if (token < M && k_in)
          x = __ldg(reinterpret_cast<const uint4*>(X + static_cast<int64_t>(token) * K + c * kChunk + t * 8));
        mma_bf16_16816(acc[mt], a.x, b.x, a.y, b.y, x.x, x.y);
        mma_bf16_16816(acc[mt], a.z, b.z, a.w, b.w, x.z, x.w);
      }
    }
  }

  // Partial sums of this warp: rows (rg * 16 + g, + 8), tokens mt * 8 + 2t, + 1.
  const int tokens_pad = MT * 8;
  float* mine = partial + (static_cast<int64_t>(ks) * block_rows + rg * 16) * tokens_pad;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    mine[g * tokens_pad + mt * 8 + 2 * t] = acc[mt][0];
    mine[g * tokens_pad + mt * 8 + 2 * t + 1] = acc[mt][1];
    mine[(g + 8) * tokens_pad + mt * 8 + 2 * t] = acc[mt][2];
    mine[(g + 8) * tokens_pad + mt * 8 + 2 * t + 1] = acc[mt][3];
  }
  __syncthreads();

  const int block_n0 = blockIdx.x * block_rows;
  if (epilogue == EPI_SWIGLU) {
    const int pairs = block_rows / 2;
    for (int item = threadIdx.x; item < M * pairs; item += kSkinnyThreads) {
      const int m = item / pairs, j = item - m * pairs;
      const int n = block_n0 + 2 * j;
      if (n >= N) continue;
      float gate = 0.f, up = 0.f;
      for (int s = 0; s < k_splits; ++s) {
        gate += partial[(static_cast<int64_t>(s) * block_rows + 2 * j) * tokens_pad + m];
        up += partial[(static_cast<int64_t>(s) * block_rows + 2 * j + 1) * tokens_pad + m];
      }
      static_cast<__nv_bfloat16*>(Y)[static_cast<int64_t>(m) * (N / 2) + n / 2] =
          __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
    }
  } else {
    for (int item = threadIdx.x; item < M * block_rows; item += kSkinnyThreads) {
      const int m = item / block_rows, r = item - m * block_rows;
      const int n = block_n0 + r;
      if (n >= N) continue;
      float sum = 0.f;
      for (int s = 0; s < k_splits; ++s) sum += partial[(static_cast<int64_t>(s) * block_rows + r) * tokens_pad + m];
      if (epilogue == EPI_F32) static_cast<float*>(Y)[static_cast<int64_t>(m) * N + n] = sum;
      else static_cast<__nv_bfloat16*>(Y)[static_cast<int64_t>(m) * N + n] = __float2bfloat16_rn(sum);
    }
  }
}

template <int MT>
int launch_skinny(const __nv_bfloat16* W, const __nv_bfloat16* X, void* Y, int M, int N, int K,
                  int row_groups, int epilogue, cudaStream_t stream) {
  const int block_rows = row_groups * 16;
  const int blocks = (N + block_rows - 1) / block_rows;
  const int k_splits = kSkinnyWarps / row_groups;
  const size_t smem = static_cast<size_t>(k_splits) * block_rows * MT * 8 * sizeof(float);
  skinny_gemm_kernel<MT><<<blocks, kSkinnyThreads, smem, stream>>>(W, X, Y, M, N, K, row_groups, epilogue);
  return b200_check_launch("skinny_gemm");
}

}  // namespace

// Shapes the kernel takes: at most 64 rows, K a multiple of 8 (16-byte rows), 16-byte aligned
// operands; for the SwiGLU epilogue N even.
B200_API int b200_skinny_gemm_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > 64 || N < 1 || K < 8 || K % 8) return 0;
  if (epilogue == EPI_SWIGLU && N % 2) return 0;
  return 1;
}

B200_API int b200_skinny_gemm(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue,
                              cudaStream_t stream) {
  B200_REQUIRE(b200_skinny_gemm_supported(M, N, K, epilogue), "skinny_gemm: unsupported shape %d x %d x %d", M, N, K);
  B200_REQUIRE(epilogue >= EPI_BF16 && epilogue <= EPI_SWIGLU, "skinny_gemm: unknown epilogue %d", epilogue);
  B200_REQUIRE(reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0,
               "skinny_gemm: operands must be 16-byte aligned");
  // Rows of W per block: as large as still leaves a few blocks per SM. The choice depends on
  // N alone, so a token's sums are added in the same order whatever else is in the batch.
  const int mt = (M + 7) / 8;
  int row_groups = 1;
  while (row_groups < kSkinnyWarps && (N + row_groups * 32 - 1) / (row_groups * 32) >= 3 * 148) row_groups *= 2;
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W);
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
  if (mt <= 1) return launch_skinny<1>(w, x, Y, M, N, K, row_groups, epilogue, stream);
  if (mt <= 2) return launch_skinny<2>(w, x, Y, M, N, K, row_groups, epilogue, stream);
  if (mt <= 4) return launch_skinny<4>(w, x, Y, M, N, K, row_groups, epilogue, stream);
  return launch_skinny<8>(w, x, Y, M, N, K, row_groups, epilogue, stream);
}
