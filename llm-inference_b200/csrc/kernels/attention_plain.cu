// Attention of a step's new tokens over the paged cache: the plain kernel.
//
// One block per (new token, query head). The token at absolute position `pos` of its
// request attends to keys lo..pos of that request, lo = 0 or pos - window + 1 for a windowed
// layer (python/instinct/batches.py:110-113), read through the request's block table. Query
// head h uses kv head h / (q_heads / kv_heads) (python/instinct/backends/portable.py:175-178).
// Scores, the running softmax and the weighted sum of values are 32-bit
// (portable.py:173-188); keys are taken 128 at a time with the usual max/sum rescaling, so
// any context length works. This kernel serves the 32-bit path and every shape the tuned
// kernels refuse.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kMaxDimsPerThread = 8;  // head_dim <= 1024

__device__ __forceinline__ float dot_row(const float* __restrict__ q, const float* __restrict__ k,
                                         int d) {
  float acc = 0.f;
  for (int i = 0; i < d; i += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(k + i);
    acc = fmaf(q[i], kv.x, acc);
    acc = fmaf(q[i + 1], kv.y, acc);
    acc = fmaf(q[i + 2], kv.z, acc);
    acc = fmaf(q[i + 3], kv.w, acc);
  }
  return acc;
}

__device__ __forceinline__ float dot_row(const float* __restrict__ q,
                                         const __nv_bfloat16* __restrict__ k, int d) {
  float acc = 0.f;
  for (int i = 0; i < d; i += 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(pairs[j]);
      acc = fmaf(q[i + 2 * j], f.x, acc);
      acc = fmaf(q[i + 2 * j + 1], f.y, acc);
    }
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
paged_attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_arena,
                             const T* __restrict__ v_arena, const int* __restrict__ positions,
                             const int* __restrict__ token_seq,
                             const int* __restrict__ block_table, int max_pages, int num_pages,
                             T* __restrict__ out, int q_heads, int kv_heads, int head_dim,
                             int page_size, int window, float scale, int* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                  // [head_dim]
  float* probs = qs + head_dim;                                    // [kThreads]
  int64_t* offsets = reinterpret_cast<int64_t*>(probs + kThreads);  // [kThreads]
  __shared__ float scratch[32];

  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t];
  const int seq = token_seq[t];
  const int kvh = h / (q_heads / kv_heads);
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = block_table + static_cast<int64_t>(seq) * max_pages;

  const T* qrow = q + (static_cast<int64_t>(t) * q_heads + h) * head_dim;
  for (int i = tid; i < head_dim; i += kThreads) qs[i] = to_f32<T>(qrow[i]);
  __syncthreads();

  float acc[kMaxDimsPerThread];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerThread; ++i) acc[i] = 0.f;
  float running_max = -INFINITY, running_sum = 0.f;

  for (int k0 = lo; k0 <= pos; k0 += kThreads) {
    const int j = k0 + tid;
    float s = -INFINITY;
    int64_t off = -1;
    if (j <= pos) {
      const int logical = j / page_size;
      const int page = logical < max_pages ? table[logical] : -1;
      if (page < 0 || page >= num_pages) {
        atomicOr(err, ERRBIT_BAD_PAGE);
      } else {
        off = kv_row_offset(page, kvh, j % page_size, kv_heads, page_size, head_dim);
        s = dot_row(qs, k_arena + off, head_dim) * scale;
      }
    }
    offsets[tid] = off;
    const float chunk_max = block_max(s, scratch);
    const float new_max = fmaxf(running_max, chunk_max);
    const float p = (off >= 0 && new_max > -INFINITY) ? expf(s - new_max) : 0.f;
    probs[tid] = p;
    const float chunk_sum = block_sum(p, scratch);
    const float alpha = (running_max > -INFINITY) ? expf(running_max - new_max) : 0.f;
    running_sum = running_sum * alpha + chunk_sum;
    running_max = new_max;
    __syncthreads();
    const int count = min(kThreads, pos - k0 + 1);
#pragma unroll
    for (int i = 0; i < kMaxDimsPerThread; ++i) {
      const int d = tid + i * kThreads;
      if (d < head_dim) {
        float a = acc[i] * alpha;
        for (int jj = 0; jj < count; ++jj) {
          const int64_t o = offsets[jj];
          if (o >= 0) a = fmaf(probs[jj], to_f32<T>(v_arena[o + d]), a);
        }
        acc[i] = a;
      }
    }
    __syncthreads();
  }
  T* orow = out + (static_cast<int64_t>(t) * q_heads + h) * head_dim;
  const float inv = running_sum > 0.f ? 1.f / running_sum : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxDimsPerThread; ++i) {
    const int d = tid + i * kThreads;
    if (d < head_dim) orow[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace

B200_API int b200_paged_attention_plain(const void* q, const void* k_arena, const void* v_arena,
                                        const int* positions, const int* token_seq,
                                        const int* block_table, int max_pages, int num_pages,
                                        void* out, int tokens, int q_heads, int kv_heads,
                                        int head_dim, int page_size, int window, float scale,
                                        int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
               "paged_attention_plain: %d query heads over %d kv heads", q_heads, kv_heads);
  B200_REQUIRE(head_dim > 0 && head_dim % 8 == 0 && head_dim <= kThreads * kMaxDimsPerThread,
               "paged_attention_plain: head_dim %d must be a multiple of 8, at most %d", head_dim,
               kThreads * kMaxDimsPerThread);
  B200_REQUIRE(q_heads <= 65535, "paged_attention_plain: too many heads");
  B200_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "paged_attention_plain: bad geometry");
  const dim3 grid(tokens, q_heads);
  const size_t smem = sizeof(float) * (head_dim + kThreads) + sizeof(int64_t) * kThreads;
  if (dtype == DTYPE_F32) {
    paged_attention_plain_kernel<float><<<grid, kThreads, smem, stream>>>(
        static_cast<const float*>(q), static_cast<const float*>(k_arena),
        static_cast<const float*>(v_arena), positions, token_seq, block_table, max_pages,
        num_pages, static_cast<float*>(out), q_heads, kv_heads, head_dim, page_size, window, scale,
        err);
  } else if (dtype == DTYPE_BF16) {
    paged_attention_plain_kernel<__nv_bfloat16><<<grid, kThreads, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_arena),
        static_cast<const __nv_bfloat16*>(v_arena), positions, token_seq, block_table, max_pages,
        num_pages, static_cast<__nv_bfloat16*>(out), q_heads, kv_heads, head_dim, page_size,
        window, scale, err);
  } else {
    return b200_fail("paged_attention_plain: unknown dtype %d", dtype);
  }
  return b200_check_launch("paged_attention_plain");
}
