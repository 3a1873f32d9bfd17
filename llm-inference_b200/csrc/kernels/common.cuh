// Shared device helpers and the error channel of the kernel library.
//
// Every launcher is `extern "C"`, takes raw device pointers and a stream, allocates
// nothing unless it says so, and returns 0 on success or a negative code after storing a
// message that `b200_last_error()` returns.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#define B200_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side.
enum : int { DTYPE_F32 = 0, DTYPE_BF16 = 1 };

// Bits a kernel may set in the device-side error word it is handed.
enum : int {
  ERRBIT_BAD_PAGE = 1,      // a block-table entry was negative or past the arena
  ERRBIT_BAD_TOKEN = 2,     // a token id was outside the embedding table
  ERRBIT_BAD_POSITION = 4,  // a position did not fit the block table
};

int b200_fail(const char* fmt, ...);
int b200_check_launch(const char* what);

#define B200_REQUIRE(cond, ...)                 \
  do {                                          \
    if (!(cond)) return b200_fail(__VA_ARGS__); \
  } while (0)

// Programmatic dependent launch. A kernel launched through `launch_kernel` with overlap
// enabled may start while its predecessor on the stream is still running; it must call
// `wait_for_predecessor()` before it reads anything the predecessor wrote or writes anything
// at all, and may read constants (weights) and the step's metadata before that.
// `let_successor_start()` tells the scheduler that the next kernel on the stream may be made
// resident as soon as every block of this one has said so and there is room; the kernels of
// the decode chain say so first thing, before their own wait, so that a kernel's successor
// can fetch its weights while the kernel itself still waits for its predecessor (a successor
// waits for the whole of its predecessor, which waited for its own, so the order of the
// chain is kept). In a kernel launched the ordinary way both calls do nothing.
// A pointer to anything an earlier kernel of the chain writes must not be `__restrict__` in such a
// kernel: the qualifier promises the compiler that nothing else touches the data while the kernel
// runs, and it then may fetch it (through the read-only path) ahead of the wait. That happened
// to the kernel that merges the attention splits; only weights, constants and the step's
// metadata keep the qualifier.
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_successor_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Thread-block clusters: a barrier over every thread of every block of the cluster, and a
// 32-bit load from the same shared-memory address in another block of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float load_peer_f32(const float* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ float4 load_peer_f32x4(const float* local, uint32_t rank) {  // 16-byte aligned
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}
// The address, in the cluster's shared-memory window, of `local` in block `rank`; and a 32-bit
// store to such an address plus a byte offset.
__device__ __forceinline__ uint32_t peer_address(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
  return remote;
}
__device__ __forceinline__ void store_peer_f32(uint32_t remote, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// RMSNorm folded into the matrix products around it (decode steps of up to 16 tokens).
//
// A product whose input is a normalised residual stream may take, instead of the normalised
// rows, the stream times the norm's scale (`xn`, bfloat16) and apply each token's 1 / rms to
// its outputs afterwards: the factor commutes with the product. The sum of squares it needs
// arrives as partial sums `ss_in[part][16]`, one row per block of the product that produced
// the stream, added here in a fixed order. That producer is a product launched with the
// second half of this struct: it adds its result into the 32-bit stream `x`, writes the
// stream times the scale of the norm that FOLLOWS (`xn`) and its block's partial sums of
// squares (`ss_out`). Either half, or both, may be unused (null pointers).
struct NormFold {
  const float* ss_in;   // [ss_parts][16]
  int ss_parts;
  int width;            // the stream's width: mean of squares = sum / width
  float eps;
  float* x;             // [M, N] residual stream, updated in place
  const float* next_weight;  // [N] scale of the norm that follows
  __nv_bfloat16* xn;    // [M, N]
  float* ss_out;        // [parts of this launch][16]
};
constexpr int kFoldTokens = 16;  // row length of the partial sums

// 1 / rms of token m from the partial sums, by one warp: each lane adds every 32nd part in
// order, the lanes' sums meet in a fixed tree.
__device__ __forceinline__ float fold_rstd(const NormFold& fold, int m) {
  const int lane = threadIdx.x & 31;
  float sum = 0.f;
  for (int p0 = lane; p0 < fold.ss_parts; p0 += 32 * 4) {
    float part[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + 32 * j;
      part[j] = p < fold.ss_parts ? __ldcg(fold.ss_in + p * kFoldTokens + m) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) sum += part[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  return rsqrtf(sum / static_cast<float>(fold.width) + fold.eps);
}

bool b200_overlap_enabled();
int b200_sm_count_host();  // SMs of the current device (cached)

// `ordered` launches the ordinary way whatever the library's overlap setting: the kernel starts
// only after everything before it on the stream has finished.
template <typename... KernelArgs, typename... Args>
cudaError_t launch_kernel_as(bool ordered, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = !ordered && b200_overlap_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

template <typename... KernelArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
  return launch_kernel_as(false, kernel, grid, block, smem, stream, args...);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. Every thread gets the
// result, and the order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < warps) ? scratch[lane] : 0.f;
  total = warp_sum(total);
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < warps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

// Offset (in elements) of row `row` of kv head `head` in page `page` of one layer's K or V
// arena laid out [pages][kv_heads][page_size][head_dim].
__device__ __forceinline__ int64_t kv_row_offset(int page, int head, int row, int kv_heads,
                                                 int page_size, int head_dim) {
  return ((static_cast<int64_t>(page) * kv_heads + head) * page_size + row) * head_dim;
}
