// Position encoding and cache write in one pass over a step's Q/K/V rows.
//
// For each new token: add the projection bias, rotate every query and key head at the
// token's absolute position (half-split pairing i <-> i + rot/2, angle = pos * inv_freq[i],
// all in 32-bit; python/instinct/backends/portable.py:115-132, cuda/kernels.cu:123-170),
// store the rotated query densely and the rotated key and the value into the token's page
// of the layer's arena: row = table[pos / page] * page + pos % page
// (python/instinct/paged_kv.py:259-265).
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ block_table, int max_pages,
                                     int num_pages, T* __restrict__ k_arena,
                                     T* __restrict__ v_arena, T* __restrict__ q_out, int q_heads,
                                     int kv_heads, int head_dim, int rot, int page_size,
                                     int write_kv, int* __restrict__ err) {
  extern __shared__ float trig[];  // cos[rot/2], sin[rot/2]
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half_rot = rot / 2;
  for (int i = threadIdx.x; i < half_rot; i += blockDim.x) {
    float s, c;
    sincosf(static_cast<float>(pos) * inv_freq[i], &s, &c);
    trig[i] = c;
    trig[half_rot + i] = s;
  }
  __syncthreads();

  int page = -1;
  if (write_kv) {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      page = block_table[static_cast<int64_t>(token_seq[t]) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_PAGE);
        page = -1;
      }
    }
  }
  const int row = pos % page_size;
  const int width = (q_heads + 2 * kv_heads) * head_dim;
  const T* src = qkv + static_cast<int64_t>(t) * width;
  const int half = head_dim / 2;
  const int rotated_heads = q_heads + kv_heads;

  // One work item per (head, pair slot): slots below rot/2 are rotated pairs, the rest copy
  // the two trailing dims that a partial rotation leaves alone.
  for (int item = threadIdx.x; item < rotated_heads * half; item += blockDim.x) {
    const int head = item / half;
    const int slot = item - head * half;
    int d0, d1;
    float y0, y1;
    if (slot < half_rot) {
      d0 = slot;
      d1 = slot + half_rot;
    } else {
      d0 = rot + 2 * (slot - half_rot);
      d1 = d0 + 1;
    }
    float x0 = to_f32<T>(src[head * head_dim + d0]);
    float x1 = to_f32<T>(src[head * head_dim + d1]);
    if (bias) {
      x0 += bias[head * head_dim + d0];
      x1 += bias[head * head_dim + d1];
    }
    if (slot < half_rot) {
      const float c = trig[slot], s = trig[half_rot + slot];
      y0 = x0 * c - x1 * s;
      y1 = x1 * c + x0 * s;
    } else {
      y0 = x0;
      y1 = x1;
    }
    if (head < q_heads) {
      T* dst = q_out + (static_cast<int64_t>(t) * q_heads + head) * head_dim;
      dst[d0] = from_f32<T>(y0);
      dst[d1] = from_f32<T>(y1);
    } else if (page >= 0) {
      T* dst = k_arena + kv_row_offset(page, head - q_heads, row, kv_heads, page_size, head_dim);
      dst[d0] = from_f32<T>(y0);
      dst[d1] = from_f32<T>(y1);
    }
  }
  if (page >= 0) {
    const int v_base = rotated_heads * head_dim;
    for (int item = threadIdx.x; item < kv_heads * head_dim; item += blockDim.x) {
      const int head = item / head_dim;
      const int d = item - head * head_dim;
      float x = to_f32<T>(src[v_base + item]);
      if (bias) x += bias[v_base + item];
      v_arena[kv_row_offset(page, head, row, kv_heads, page_size, head_dim) + d] = from_f32<T>(x);
    }
  }
}

B200_API int b200_rope_kv_write(const void* qkv, const float* bias, const float* inv_freq,
                                const int* positions, const int* token_seq,
                                const int* block_table, int max_pages, int num_pages,
                                void* k_arena, void* v_arena, void* q_out, int tokens,
                                int q_heads, int kv_heads, int head_dim, int rot, int page_size,
                                int write_kv, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200_REQUIRE(tokens > 0 && q_heads > 0 && kv_heads > 0, "rope_kv_write: bad sizes");
  B200_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope_kv_write: head_dim %d must be even",
               head_dim);
  B200_REQUIRE(rot >= 0 && rot <= head_dim && rot % 2 == 0,
               "rope_kv_write: rotary dims %d must be even and at most head_dim %d", rot, head_dim);
  B200_REQUIRE(page_size > 0 && max_pages > 0, "rope_kv_write: bad page geometry");
  const int threads = 128;
  const size_t smem = sizeof(float) * (rot > 0 ? rot : 2);
  if (dtype == DTYPE_F32) {
    launch_kernel(rope_kv_write_kernel<float>, dim3(tokens), dim3(threads), smem, stream,
        static_cast<const float*>(qkv), bias, inv_freq, positions, token_seq, block_table,
        max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena),
        static_cast<float*>(q_out), q_heads, kv_heads, head_dim, rot, page_size, write_kv, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(rope_kv_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), smem, stream,
        static_cast<const __nv_bfloat16*>(qkv), bias, inv_freq, positions, token_seq, block_table,
        max_pages, num_pages, static_cast<__nv_bfloat16*>(k_arena),
        static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), q_heads,
        kv_heads, head_dim, rot, page_size, write_kv, err);
  } else {
    return b200_fail("rope_kv_write: unknown dtype %d", dtype);
  }
  return b200_check_launch("rope_kv_write");
}
