// Matrix product for a handful of tokens (decode steps):  Y[M,N] = X[M,K] * W[N,K]^T, M <= 16.
//
// With so few rows the product is a stream of the weight matrix through the GPU once, so the
// kernel is built around that stream. The roles of the operands are swapped for the tensor
// cores: 16 rows of W are the "A" tile of mma.sync m16n8k16 and 8 tokens are its "B" tile.
// Each lane owns its share of a 16 x 32 slab of W as two 16-byte pieces in fragment order (the
// order of k inside a slab is permuted the same way for W and X, which a dot product does not
// notice). The pieces travel global -> shared memory with cp.async into a private ring of
// `kStages` slabs per warp, so every warp keeps kStages KB in flight without holding them in
// registers, and a lane reads back only what it fetched itself (no barriers in the loop).
// The weights of the first slabs are requested before the kernel waits for its predecessor
// on the stream, so their latency hides behind the previous kernel's tail.
// The 8 warps of a block are `row_groups` groups of 16 weight
// rows times `k_splits` slices of K; the slices' partial sums meet in shared memory and are
// added in slice order, so the result does not depend on timing. When W has too few rows to
// give every SM a block, several blocks share a column of rows and split K among them: each
// writes its sums to scratch memory and the one that finishes last adds them in block order.
// Linear layers are x W^T with
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
constexpr int kChunk = 32;   // k per slab
// Slabs in flight per warp: 12 for up to 8 tokens, 8 for up to 16 (whose slabs carry one more
// piece). Measured in the 1.5B decode step: 8 -> 12 saves 3 % at batch 8, costs 2 % at batch 16.
template <int MT>
struct SkinnyStages {
  static constexpr int value = MT == 1 ? 12 : 8;
};

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void copy_async_16(void* dst, const void* src, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int bytes = valid ? 16 : 0;  // zero-fills when not valid
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Sum of the k-slices' partial results for output (row r, token m) of this block, in slice order.
__device__ __forceinline__ float block_sum_at(const float* partial, int k_splits, int block_rows,
                                              int tokens_pad, int r, int m) {
  float sum = 0.f;
  for (int s = 0; s < k_splits; ++s) sum += partial[(static_cast<int64_t>(s) * block_rows + r) * tokens_pad + m];
  return sum;
}

// One instantiation per (token tiles, epilogue, folded norm or not): a block runs its epilogue
// once, from a cold instruction cache, and code it shares with forms it does not take costs it
// time (measured on the tcgen05 product, gemm_tcgen05.cu).
template <int MT, int EPI, bool FOLDED>
__global__ void __launch_bounds__(kSkinnyThreads)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* X,
                   void* Y, int M, int N, int K, int row_groups,
                   float* scratch, int* counters, const NormFold fold) {
  // Ring: [warp][stage][piece][lane] of 16-byte pieces; piece 0/1 = W rows g / g + 8, 2.. = X.
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* ring = reinterpret_cast<uint4*>(smem_raw);
  __shared__ int ticket_shared;
  __shared__ float rstd_s[kFoldTokens];
  constexpr int kPieces = 2 + MT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k_splits = kSkinnyWarps / row_groups;
  const int rg = warp % row_groups, ks = warp / row_groups;
  const int block_rows = row_groups * 16;
  const int n0 = blockIdx.x * block_rows + rg * 16;
  constexpr int kStages = SkinnyStages<MT>::value;
  uint4* my_ring = ring + static_cast<int64_t>(warp) * kStages * kPieces * 32;

  // K is cut first across the blocks of a column (gridDim.y), then across this block's warps.
  const int chunks = (K + kChunk - 1) / kChunk;
  const int per_block = (chunks + gridDim.y - 1) / gridDim.y;
  const int b_begin = blockIdx.y * per_block, b_end = min(chunks, b_begin + per_block);
  const int per_split = (max(0, b_end - b_begin) + k_splits - 1) / k_splits;
  const int c_begin = b_begin + ks * per_split, c_end = min(b_end, c_begin + per_split);

  const int row_a = n0 + g, row_b = n0 + g + 8;
  const bool live_a = row_a < N, live_b = row_b < N;
  const __nv_bfloat16* wa = W + static_cast<int64_t>(live_a ? row_a : 0) * K + t * 8;
  const __nv_bfloat16* wb = W + static_cast<int64_t>(live_b ? row_b : 0) * K + t * 8;

  auto fetch_w = [&](int c, int stage) {
    const bool in = c < c_end && c * kChunk + t * 8 < K;
    uint4* slot = my_ring + stage * kPieces * 32;
    copy_async_16(slot + lane, wa + (in ? c * kChunk : 0), in && live_a);
    copy_async_16(slot + 32 + lane, wb + (in ? c * kChunk : 0), in && live_b);
  };
  auto fetch_x = [&](int c, int stage) {
    const bool in = c < c_end && c * kChunk + t * 8 < K;
    uint4* slot = my_ring + stage * kPieces * 32;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const bool live = mt * 8 + g < M;
      const __nv_bfloat16* x = X + static_cast<int64_t>(live ? mt * 8 + g : 0) * K + t * 8;
      copy_async_16(slot + (2 + mt) * 32 + lane, x + (in ? c * kChunk : 0), in && live);
    }
  };

  let_successor_start();
  // Weights do not depend on the previous kernel: request them first, then wait for it.
  // Rolled on purpose, like the loop over X below: unrolled, the two took 5 KB of the kernel's 24.
#pragma unroll 1
  for (int i = 0; i < kStages; ++i) fetch_w(c_begin + i, i);
  copy_async_commit();
  wait_for_predecessor();
  let_successor_start();
#pragma unroll 1
  for (int i = 0; i < kStages; ++i) fetch_x(c_begin + i, i);
  copy_async_commit();
  if (FOLDED && fold.ss_in != nullptr) {
    // The operand is the stream times a norm's scale: each token's 1 / rms, applied to the sums
    // at the end. Two tokens per warp, while the first slabs are on their way.
    for (int m = warp; m < M; m += kSkinnyWarps) {
      const float r = fold_rstd(fold, m);
      if (lane == 0) rstd_s[m] = r;
    }
  }
  copy_async_wait<0>();

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  int stage = 0;
  for (int c = c_begin; c < c_end; ++c) {
    // Every iteration commits one group, so all but the newest kStages - 1 are complete here.
    copy_async_wait<kStages - 1>();
    const uint4* slot = my_ring + stage * kPieces * 32;
    const uint4 a = slot[lane], b = slot[32 + lane];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const uint4 x = slot[(2 + mt) * 32 + lane];
      mma_bf16_16816(acc[mt], a.x, b.x, a.y, b.y, x.x, x.y);
      mma_bf16_16816(acc[mt], a.z, b.z, a.w, b.w, x.z, x.w);
    }
    // The pieces are in registers and used; refill the slot with the slab kStages further on.
    fetch_w(c + kStages, stage);
    fetch_x(c + kStages, stage);
    copy_async_commit();
    stage = stage + 1 == kStages ? 0 : stage + 1;
  }
  copy_async_wait<0>();
  __syncthreads();  // the ring is reused for the partial sums below

  // Partial sums of this warp: rows (rg * 16 + g, + 8), tokens mt * 8 + 2t, + 1.
  float* partial = reinterpret_cast<float*>(smem_raw);  // [k_splits][block_rows][MT * 8]
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

  const int tile = block_rows * tokens_pad;
  const float* sums = nullptr;  // when set: [gridDim.y][tile] partials of every block of this column
  if (gridDim.y > 1) {
    // Hand this block's sums to the column's scratch; the block that arrives last adds all of
    // them in block order, so the result does not depend on which block that is.
    float* column = scratch + static_cast<int64_t>(blockIdx.x) * gridDim.y * tile;
    for (int item = threadIdx.x; item < tile; item += kSkinnyThreads)
      column[static_cast<int64_t>(blockIdx.y) * tile + item] =
          block_sum_at(partial, k_splits, block_rows, tokens_pad, item / tokens_pad, item % tokens_pad);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_shared = atomicAdd(&counters[blockIdx.x], 1);
    __syncthreads();
    if (ticket_shared != static_cast<int>(gridDim.y) - 1) return;
    __threadfence();
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;  // ready for the next launch
    sums = column;
  }

  const int block_n0 = blockIdx.x * block_rows;
  const bool scaled = FOLDED && fold.ss_in != nullptr;
  auto total = [&](int r, int m) -> float {
    float sum = 0.f;
    if (sums == nullptr) {
      sum = block_sum_at(partial, k_splits, block_rows, tokens_pad, r, m);
    } else {
      for (int s = 0; s < static_cast<int>(gridDim.y); ++s)
        sum += __ldcg(sums + static_cast<int64_t>(s) * tile + r * tokens_pad + m);
    }
    return scaled ? sum * rstd_s[m] : sum;
  };
  if (FOLDED && fold.x != nullptr) {
    // The product goes into the residual stream; the stream times the next norm's scale and this
    // block's partial sums of squares go out for the product that follows that norm.
    __shared__ float squares[FOLDED ? kFoldTokens * kSkinnyWarps * 16 : 1];  // [m][row of the block]
    for (int item = threadIdx.x; item < M * block_rows; item += kSkinnyThreads) {
      const int m = item / block_rows, r = item - m * block_rows;
      const int n = block_n0 + r;
      float sq = 0.f;
      if (n < N) {
        const int64_t at = static_cast<int64_t>(m) * N + n;
        const float now = fold.x[at] + total(r, m);
        fold.x[at] = now;
        fold.xn[at] = __float2bfloat16_rn(now * fold.next_weight[n]);
        sq = now * now;
      }
      squares[m * block_rows + r] = sq;
    }
    __syncthreads();
    if (threadIdx.x < M) {
      float sum = 0.f;
      for (int r = 0; r < block_rows; ++r) sum += squares[threadIdx.x * block_rows + r];
      fold.ss_out[static_cast<int64_t>(blockIdx.x) * kFoldTokens + threadIdx.x] = sum;
    }
    return;
  }
  if constexpr (EPI == EPI_SWIGLU) {
    const int pairs = block_rows / 2;
    for (int item = threadIdx.x; item < M * pairs; item += kSkinnyThreads) {
      const int m = item / pairs, j = item - m * pairs;
      const int n = block_n0 + 2 * j;
      if (n >= N) continue;
      const float gate = total(2 * j, m), up = total(2 * j + 1, m);
      static_cast<__nv_bfloat16*>(Y)[static_cast<int64_t>(m) * (N / 2) + n / 2] =
          __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
    }
  } else {
    for (int item = threadIdx.x; item < M * block_rows; item += kSkinnyThreads) {
      const int m = item / block_rows, r = item - m * block_rows;
      const int n = block_n0 + r;
      if (n >= N) continue;
      const float sum = total(r, m);
      if constexpr (EPI == EPI_F32) static_cast<float*>(Y)[static_cast<int64_t>(m) * N + n] = sum;
      else static_cast<__nv_bfloat16*>(Y)[static_cast<int64_t>(m) * N + n] = __float2bfloat16_rn(sum);
    }
  }
}

// How the launcher cuts the work; a function of N and K only, so that a token's sums are added
// in the same order whatever else is in the batch. The aim is one wave of long-lived warps:
// about two blocks per SM, each warp streaming a contiguous run of slabs.
struct SkinnyPlan {
  int row_groups;
  int column_blocks;  // blocks that share one column of W rows and split K
  int blocks;
};

constexpr int kSkinnyMaxDevices = 64;

SkinnyPlan plan_skinny(int N, int K) {
  const int tiles = (N + 15) / 16;
  const int chunks = (K + kChunk - 1) / kChunk;
  const int wave = 2 * b200_sm_count_host() * kSkinnyWarps;
  int slices = (wave + tiles / 2) / tiles;            // K slices per 16 rows, over all blocks
  slices = max(1, min(slices, max(1, chunks / 6)));  // every warp keeps a few slabs to stream
  int k_splits = 1;
  while (k_splits < kSkinnyWarps && k_splits < slices) k_splits *= 2;
  SkinnyPlan plan;
  plan.row_groups = kSkinnyWarps / k_splits;
  plan.column_blocks = max(1, min(8, (slices + k_splits - 1) / k_splits));
  const int block_rows = plan.row_groups * 16;
  plan.blocks = (N + block_rows - 1) / block_rows;
  return plan;
}

template <int MT, int EPI, bool FOLDED>
int launch_skinny_as(const __nv_bfloat16* W, const __nv_bfloat16* X, void* Y, int M, int N, int K,
                     const SkinnyPlan& plan, float* scratch, int* counters, cudaStream_t stream,
                     bool ordered, const NormFold& fold) {
  const int block_rows = plan.row_groups * 16;
  const int k_splits = kSkinnyWarps / plan.row_groups;
  const size_t ring = static_cast<size_t>(kSkinnyWarps) * SkinnyStages<MT>::value * (2 + MT) * 32 * 16;
  const size_t sums = static_cast<size_t>(k_splits) * block_rows * MT * 8 * sizeof(float);
  const size_t smem = ring > sums ? ring : sums;
  // The shared-memory opt-in is a property of the function on one device: set once per device.
  static size_t configured[kSkinnyMaxDevices] = {};  // one array per instantiation
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kSkinnyMaxDevices)
    return b200_fail("skinny_gemm: cannot tell the current device");
  if (configured[device] < smem) {
    if (cudaFuncSetAttribute(skinny_gemm_kernel<MT, EPI, FOLDED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return b200_fail("skinny_gemm: cannot size shared memory");
    configured[device] = smem;
  }
  const dim3 grid(plan.blocks, plan.column_blocks);
  cudaError_t status = launch_kernel_as(ordered, skinny_gemm_kernel<MT, EPI, FOLDED>, grid, dim3(kSkinnyThreads), smem,
                                        stream, W, X, Y, M, N, K, plan.row_groups, scratch, counters, fold);
  if (status != cudaSuccess) return b200_fail("skinny_gemm: %s", cudaGetErrorString(status));
  return 0;
}

template <int MT, int EPI>
int launch_skinny_epilogue(const __nv_bfloat16* W, const __nv_bfloat16* X, void* Y, int M, int N, int K,
                           const SkinnyPlan& plan, float* scratch, int* counters, cudaStream_t stream,
                           bool ordered, const NormFold& fold) {
  if (fold.ss_in != nullptr || fold.x != nullptr)
    return launch_skinny_as<MT, EPI, true>(W, X, Y, M, N, K, plan, scratch, counters, stream, ordered, fold);
  return launch_skinny_as<MT, EPI, false>(W, X, Y, M, N, K, plan, scratch, counters, stream, ordered, fold);
}

template <int MT>
int launch_skinny(const __nv_bfloat16* W, const __nv_bfloat16* X, void* Y, int M, int N, int K,
                  const SkinnyPlan& plan, int epilogue, float* scratch, int* counters, cudaStream_t stream,
                  bool ordered = false,
                  const NormFold& fold = NormFold{}) {
  switch (epilogue) {
    case EPI_F32:
      return launch_skinny_epilogue<MT, EPI_F32>(W, X, Y, M, N, K, plan, scratch, counters, stream, ordered, fold);
    case EPI_SWIGLU:
      return launch_skinny_epilogue<MT, EPI_SWIGLU>(W, X, Y, M, N, K, plan, scratch, counters, stream, ordered, fold);
    default:
      return launch_skinny_epilogue<MT, EPI_BF16>(W, X, Y, M, N, K, plan, scratch, counters, stream, ordered, fold);
  }
}

}  // namespace

constexpr int kSkinnyMaxRows = 16;

// Shapes the kernel takes: at most 16 rows, K a multiple of 8 (16-byte rows), 16-byte aligned
// operands; for the SwiGLU epilogue N even.
B200_API int b200_skinny_gemm_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > kSkinnyMaxRows || N < 1 || K < 8 || K % 8) return 0;
  if (epilogue == EPI_SWIGLU && N % 2) return 0;
  return 1;
}

// Scratch the product needs when blocks share a column: `floats` 32-bit words of partial sums
// and `counters` ints that must be zero before the first launch (each launch leaves them zero).
B200_API void b200_skinny_gemm_scratch(int M, int N, int K, int64_t* floats, int* counters) {
  const SkinnyPlan plan = plan_skinny(N, K);
  const int tokens_pad = (M + 7) / 8 * 8;
  *floats = plan.column_blocks > 1
                ? static_cast<int64_t>(plan.blocks) * plan.column_blocks * plan.row_groups * 16 * tokens_pad
                : 0;
  *counters = plan.column_blocks > 1 ? plan.blocks : 0;
}

// With a folded norm behind it (see NormFold): how many rows of partial sums of squares a launch
// with the residual epilogue writes, one per block of rows.
B200_API int b200_skinny_gemm_fold_parts(int N, int K) { return plan_skinny(N, K).blocks; }

static int skinny_gemm_run(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, float* scratch,
                           int64_t scratch_floats, int* counters, int num_counters, const NormFold& fold,
                           cudaStream_t stream);

B200_API int b200_skinny_gemm(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue,
                              float* scratch, int64_t scratch_floats, int* counters, int num_counters,
                              cudaStream_t stream) {
  return skinny_gemm_run(W, X, Y, M, N, K, epilogue, scratch, scratch_floats, counters, num_counters, NormFold{}, stream);
}

// The same product around a folded RMSNorm (NormFold in common.cuh). With `ss_in` the operand X is
// the residual stream times the norm's scale and every token's outputs are multiplied by its
// 1 / rms (any epilogue). With `x` the result is not written to Y (which may be null) but added
// into the residual stream x[M, N]; xn and ss_out receive the stream times `next_weight` and
// this launch's b200_skinny_gemm_fold_parts(N, K) rows of partial sums of squares (epilogue 0).
B200_API int b200_skinny_gemm_fold(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue,
                                   float* scratch, int64_t scratch_floats, int* counters, int num_counters,
                                   const float* ss_in, int ss_parts, int width, float eps, float* x,
                                   const float* next_weight, void* xn, float* ss_out, cudaStream_t stream) {
  NormFold fold{};
  fold.ss_in = ss_in;
  fold.ss_parts = ss_parts;
  fold.width = width;
  fold.eps = eps;
  fold.x = x;
  fold.next_weight = next_weight;
  fold.xn = static_cast<__nv_bfloat16*>(xn);
  fold.ss_out = ss_out;
  B200_REQUIRE(M <= kFoldTokens, "skinny_gemm_fold: at most %d tokens", kFoldTokens);
  B200_REQUIRE(ss_in == nullptr || (ss_parts > 0 && width > 0), "skinny_gemm_fold: partial sums without their count");
  B200_REQUIRE(x == nullptr || (next_weight != nullptr && xn != nullptr && ss_out != nullptr && epilogue == EPI_BF16),
               "skinny_gemm_fold: the residual epilogue needs the next norm's scale, xn and ss_out");
  B200_REQUIRE(x != nullptr || Y != nullptr, "skinny_gemm_fold: no output");
  return skinny_gemm_run(W, X, Y, M, N, K, epilogue, scratch, scratch_floats, counters, num_counters, fold, stream);
}

static int skinny_gemm_run(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, float* scratch,
                           int64_t scratch_floats, int* counters, int num_counters, const NormFold& fold,
                           cudaStream_t stream) {
  B200_REQUIRE(b200_skinny_gemm_supported(M, N, K, epilogue), "skinny_gemm: unsupported shape %d x %d x %d", M, N, K);
  B200_REQUIRE(epilogue >= EPI_BF16 && epilogue <= EPI_SWIGLU, "skinny_gemm: unknown epilogue %d", epilogue);
  B200_REQUIRE(reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0,
               "skinny_gemm: operands must be 16-byte aligned");
  const SkinnyPlan plan = plan_skinny(N, K);
  int64_t need_floats;
  int need_counters;
  b200_skinny_gemm_scratch(M, N, K, &need_floats, &need_counters);
  B200_REQUIRE(scratch_floats >= need_floats && num_counters >= need_counters,
               "skinny_gemm: scratch too small (%lld floats, %d counters needed)",
               static_cast<long long>(need_floats), need_counters);
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W);
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
  if (M <= 8)
    return launch_skinny<1>(w, x, Y, M, N, K, plan, epilogue, scratch, counters, stream, false, fold);
  return launch_skinny<2>(w, x, Y, M, N, K, plan, epilogue, scratch, counters, stream, false, fold);
}

// ---- the variant that allocates nothing (declared and documented in gemm_skinny_static.h) ----
#include <mutex>

#include "gemm_skinny_static.h"

namespace {

constexpr long long kStaticScratchFloats = 128 * 1024;  // 512 KiB of partial sums
constexpr int kStaticCounters = 1024;
constexpr int kMaxDevices = 64;

// In host code these names are stand-ins for the device arrays, not device addresses: the
// addresses come from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) int g_static_counters[kStaticCounters];

struct StaticScratch {
  float* scratch = nullptr;
  int* counters = nullptr;
};
StaticScratch g_static_by_device[kMaxDevices];
std::mutex g_static_mutex;

// The device addresses of the arrays on the current device, looked up once per device.
int static_scratch(StaticScratch* out) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return b200_fail("skinny_gemm_static: cannot tell the current device");
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticScratch& entry = g_static_by_device[device];
  if (entry.scratch == nullptr) {
    float* scratch = nullptr;
    int* counters = nullptr;
    cudaError_t status = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_static_scratch);
    if (status != cudaSuccess)
      return b200_fail("skinny_gemm_static: cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(status));
    status = cudaGetSymbolAddress(reinterpret_cast<void**>(&counters), g_static_counters);
    if (status != cudaSuccess)
      return b200_fail("skinny_gemm_static: cudaGetSymbolAddress(counters) failed: %s", cudaGetErrorString(status));
    entry.scratch = scratch;
    entry.counters = counters;
  }
  *out = entry;
  return 0;
}

}  // namespace

B200_API long long b200_skinny_gemm_static_capacity_floats(void) { return kStaticScratchFloats; }

B200_API int b200_skinny_gemm_static(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue,
                                     cudaStream_t stream) {
  B200_REQUIRE(b200_skinny_gemm_supported(M, N, K, epilogue),
               "skinny_gemm_static: unsupported shape %d x %d x %d (at most 16 rows, K a multiple of 8)", M, N, K);
  B200_REQUIRE(epilogue >= EPI_BF16 && epilogue <= EPI_SWIGLU, "skinny_gemm_static: unknown epilogue %d", epilogue);
  B200_REQUIRE(W != nullptr && X != nullptr && Y != nullptr, "skinny_gemm_static: null operand");
  B200_REQUIRE(reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0,
               "skinny_gemm_static: operands must be 16-byte aligned");
  int64_t need_floats = 0;
  int need_counters = 0;
  b200_skinny_gemm_scratch(M, N, K, &need_floats, &need_counters);
  B200_REQUIRE(need_floats <= kStaticScratchFloats && need_counters <= kStaticCounters,
               "skinny_gemm_static: %d x %d x %d needs %lld floats and %d counters of scratch; the static scratch "
               "holds %lld floats and %d counters",
               M, N, K, static_cast<long long>(need_floats), need_counters, kStaticScratchFloats, kStaticCounters);
  StaticScratch mine;
  if (static_scratch(&mine) != 0) return -1;
  if (need_counters > 0) {
    // The counters are the only part that must start at zero.
    const cudaError_t status = cudaMemsetAsync(mine.counters, 0, sizeof(int) * need_counters, stream);
    if (status != cudaSuccess)
      return b200_fail("skinny_gemm_static: clearing the counters failed: %s", cudaGetErrorString(status));
  }
  const SkinnyPlan plan = plan_skinny(N, K);
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(W);
  const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
  // Launched the ordinary way (no programmatic overlap with the kernel before it): a caller's W may
  // be the output of that kernel, and this kernel requests its first slabs of W before it would wait.
  if (M <= 8)
    return launch_skinny<1>(w, x, Y, M, N, K, plan, epilogue, mine.scratch, mine.counters, stream, true);
  return launch_skinny<2>(w, x, Y, M, N, K, plan, epilogue, mine.scratch, mine.counters, stream, true);
}
