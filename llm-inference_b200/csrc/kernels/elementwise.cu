// Embedding gather, RMSNorm (with the residual add fused in) and SwiGLU's gate.
//
// The residual stream is kept in 32-bit in both precisions; norms, the residual sum and
// the activation are computed in 32-bit and rounded once on the way out.
#include "common.cuh"

// out[t, :] = table[ids[t], :]  (reference: cuda/kernels.cu:59-68, one row per block here)
template <typename T>
__global__ void embedding_gather_kernel(const T* __restrict__ table, const int* ids,
                                        float* out, int hidden, int vocab,
                                        int* err) {
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + static_cast<int64_t>(t) * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  const T* src = table + static_cast<int64_t>(id) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

B200_API int b200_embedding_gather(const void* table, int table_dtype, const int* ids, float* out,
                                   int tokens, int hidden, int vocab, int* err,
                                   cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding_gather: bad sizes");
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == DTYPE_F32) {
    launch_kernel(embedding_gather_kernel<float>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const float*>(table), ids, out, hidden, vocab, err);
  } else if (table_dtype == DTYPE_BF16) {
    launch_kernel(embedding_gather_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  static_cast<const __nv_bfloat16*>(table), ids, out, hidden, vocab, err);
  } else {
    return b200_fail("embedding_gather: unknown dtype %d", table_dtype);
  }
  return b200_check_launch("embedding_gather");
}

// RMSNorm of row r of the residual stream x (32-bit), optionally after adding the pending
// branch output `delta` to it:  v = x[r] + delta[r];  y = v * rsqrt(mean(v^2) + eps) * w.
// With `rows` == nullptr every row is normed and v is written back to x; with `rows` the
// kernel norms only x[rows[i]] into out[i] and leaves x alone (the model's last norm, which
// only the wanted positions need). Formula: python/instinct/backends/portable.py:144-149;
// the fused add follows cuda/kernels.cu:85-98 but keeps the sum in 32-bit.
// Each thread keeps its share of the row (up to kNormCache values) in registers between the sum
// of squares and the scaling, so the row is read from memory once; wider rows re-read.
constexpr int kNormCache = 8;

template <typename T>
__global__ void rmsnorm_kernel(float* x, const T* delta,
                               const float* __restrict__ weight, T* out,
                               const int* rows, int hidden, float eps) {
  __shared__ float scratch[32];
  wait_for_predecessor();
  let_successor_start();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + static_cast<int64_t>(r) * hidden;
  const T* dr = delta ? delta + static_cast<int64_t>(r) * hidden : nullptr;
  T* outr = out + static_cast<int64_t>(blockIdx.x) * hidden;
  const bool cached = hidden <= kNormCache * static_cast<int>(blockDim.x);
  float v[kNormCache];
  float ss = 0.f;
  if (cached) {
#pragma unroll
    for (int j = 0; j < kNormCache; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = 0.f;
      if (i < hidden) {
        v[j] = xr[i] + (dr ? to_f32<T>(dr[i]) : 0.f);
        if (dr && !rows) xr[i] = v[j];
        ss += v[j] * v[j];
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float value = xr[i];
      if (dr) {
        value += to_f32<T>(dr[i]);
        if (!rows) xr[i] = value;
      }
      ss += value * value;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
  if (cached) {
#pragma unroll
    for (int j = 0; j < kNormCache; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < hidden) outr[i] = from_f32<T>(v[j] * inv * weight[i]);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float value = xr[i];
      if (dr && rows) value += to_f32<T>(dr[i]);
      outr[i] = from_f32<T>(value * inv * weight[i]);
    }
  }
}

// The same with 16-byte accesses of the residual (four values per thread and turn), for rows
// whose length is a multiple of four and buffers aligned to 16 bytes: the usual case. Up to
// kNormVecCache turns stay in registers; wider rows go to the kernel above.
constexpr int kNormVecCache = 2;

template <typename T>
struct Quad;
template <>
struct Quad<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Quad<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a(__float2bfloat16_rn(v.x), __float2bfloat16_rn(v.y));
    const __nv_bfloat162 b(__float2bfloat16_rn(v.z), __float2bfloat16_rn(v.w));
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

template <typename T>
__global__ void rmsnorm_vec4_kernel(float* x, const T* delta,
                                    const float* __restrict__ weight, T* out,
                                    const int* rows, int hidden, float eps) {
  __shared__ float scratch[32];
  // The weights are constants and the row list is part of the step's metadata: both are read
  // before the wait for the kernel in front. After it, everything else this thread reads (its
  // piece of the row and of the pending branch output) is requested before anything is used.
  let_successor_start();
  float4 v[kNormVecCache], d[kNormVecCache], w[kNormVecCache];
#pragma unroll
  for (int j = 0; j < kNormVecCache; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    w[j] = i < hidden ? *reinterpret_cast<const float4*>(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  wait_for_predecessor();
  let_successor_start();
  float* xr = x + static_cast<int64_t>(r) * hidden;
  const T* dr = delta ? delta + static_cast<int64_t>(r) * hidden : nullptr;
  T* outr = out + static_cast<int64_t>(blockIdx.x) * hidden;
#pragma unroll
  for (int j = 0; j < kNormVecCache; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    v[j] = d[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < hidden) {
      v[j] = *reinterpret_cast<const float4*>(xr + i);
      if (dr) d[j] = Quad<T>::load(dr + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormVecCache; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    if (i < hidden) {
      if (dr) {
        v[j].x += d[j].x;
        v[j].y += d[j].y;
        v[j].z += d[j].z;
        v[j].w += d[j].w;
        if (!rows) *reinterpret_cast<float4*>(xr + i) = v[j];
      }
      ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int j = 0; j < kNormVecCache; ++j) {
    const int i = 4 * (threadIdx.x + j * blockDim.x);
    if (i < hidden)
      Quad<T>::store(outr + i, make_float4(v[j].x * inv * w[j].x, v[j].y * inv * w[j].y, v[j].z * inv * w[j].z,
                                           v[j].w * inv * w[j].w));
  }
}

template <typename T>
bool rmsnorm_vec4(float* x, const T* delta, const float* weight, T* out, const int* rows, int num_rows, int hidden,
                  float eps, cudaStream_t stream) {
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (hidden % 4 != 0 || hidden > 4 * 1024 * kNormVecCache || !aligned(x) || !aligned(delta) || !aligned(weight) ||
      !aligned(out))
    return false;
  const int quads = hidden / 4;
  int threads = quads <= 1024 ? quads : (quads + kNormVecCache - 1) / kNormVecCache;
  threads = (threads + 31) / 32 * 32;
  launch_kernel(rmsnorm_vec4_kernel<T>, dim3(num_rows), dim3(threads), 0, stream, x, delta, weight, out, rows, hidden, eps);
  return true;
}

B200_API int b200_rmsnorm(float* x, const void* delta, const float* weight, void* out,
                          const int* rows, int num_rows, int hidden, float eps, int dtype,
                          cudaStream_t stream) {
  if (num_rows == 0) return 0;
  B200_REQUIRE(num_rows > 0 && hidden > 0, "rmsnorm: bad sizes");
  if (dtype == DTYPE_F32 && rmsnorm_vec4<float>(x, static_cast<const float*>(delta), weight, static_cast<float*>(out), rows,
                                                num_rows, hidden, eps, stream))
    return b200_check_launch("rmsnorm");
  if (dtype == DTYPE_BF16 &&
      rmsnorm_vec4<__nv_bfloat16>(x, static_cast<const __nv_bfloat16*>(delta), weight, static_cast<__nv_bfloat16*>(out),
                                  rows, num_rows, hidden, eps, stream))
    return b200_check_launch("rmsnorm");
  const int threads = hidden >= 4096 ? 1024 : (hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128));
  if (dtype == DTYPE_F32) {
    launch_kernel(rmsnorm_kernel<float>, dim3(num_rows), dim3(threads), 0, stream, x,
                  static_cast<const float*>(delta), weight, static_cast<float*>(out), rows, hidden, eps);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(rmsnorm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), 0, stream, x,
                  static_cast<const __nv_bfloat16*>(delta), weight, static_cast<__nv_bfloat16*>(out), rows,
                  hidden, eps);
  } else {
    return b200_fail("rmsnorm: unknown dtype %d", dtype);
  }
  return b200_check_launch("rmsnorm");
}

// out[t, i] = silu(gate[t, i]) * up[t, i],  silu(g) = g / (1 + exp(-g))
// (python/instinct/backends/dense.py:124-128; cuda/kernels.cu:100-106). The input row holds
// gate and up interleaved: gu[t, 2i] is gate_i and gu[t, 2i + 1] is up_i, which is how the
// feed-forward stores its fused gate/up matrix.
template <typename T>
__global__ void silu_mul_kernel(const T* gu, T* out, int64_t total) {
  wait_for_predecessor();
  let_successor_start();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const float g = to_f32<T>(gu[2 * idx]);
  const float u = to_f32<T>(gu[2 * idx + 1]);
  out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

// bfloat16, eight outputs per thread: two 16-byte loads, one 16-byte store.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out,
                                       int64_t groups) {
  wait_for_predecessor();
  let_successor_start();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const uint4* src = reinterpret_cast<const uint4*>(gu) + 2 * idx;
  const uint4 lo = src[0], hi = src[1];
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi);
  __nv_bfloat16 r[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __bfloat1622float2(a[i]);
    const float2 q = __bfloat1622float2(b[i]);
    r[i] = __float2bfloat16_rn(p.x / (1.f + expf(-p.x)) * p.y);
    r[4 + i] = __float2bfloat16_rn(q.x / (1.f + expf(-q.x)) * q.y);
  }
  reinterpret_cast<uint4*>(out)[idx] = *reinterpret_cast<const uint4*>(r);
}

B200_API int b200_silu_mul(const void* gate_up, void* out, int tokens, int inter, int dtype,
                           cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && inter > 0, "silu_mul: bad sizes");
  const int64_t total = static_cast<int64_t>(tokens) * inter;
  const int threads = 256;
  if (dtype == DTYPE_F32) {
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
    launch_kernel(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                  static_cast<const float*>(gate_up), static_cast<float*>(out), total);
  } else if (dtype == DTYPE_BF16) {
    const bool vec = total % 8 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0;
    if (vec) {
      const int64_t groups = total / 8;
      const unsigned blocks = static_cast<unsigned>((groups + threads - 1) / threads);
      launch_kernel(silu_mul_bf16x8_kernel, dim3(blocks), dim3(threads), 0, stream,
                    static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), groups);
    } else {
      const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
      launch_kernel(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                    static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), total);
    }
  } else {
    return b200_fail("silu_mul: unknown dtype %d", dtype);
  }
  return b200_check_launch("silu_mul");
}
