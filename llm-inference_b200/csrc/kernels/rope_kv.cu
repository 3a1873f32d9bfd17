// Position encoding and cache write in one pass over a step's Q/K/V rows.
//
// For each new token: add the projection bias, rotate every query and key head at the
// token's absolute position (half-split pairing i <-> i + rot/2, angle = pos * inv_freq[i],
// all in 32-bit; python/instinct/backends/portable.py:115-132, cuda/kernels.cu:123-170),
// store the rotated query densely and the rotated key and the value into the token's page
// of the layer's arena: row = table[pos / page] * page + pos % page
// (python/instinct/paged_kv.py:259-265).
//
// Pages are handed from request to request without being cleared, and the tensor-core attention
// kernels load whole tiles of a page and mask the rows past a request's last key only in the
// scores: what such a row holds still meets a probability of zero in the PV product, and zero
// times a non-finite leftover would be NaN. So the token that starts a page (position a multiple
// of the page size: the first write of its request to that page) also clears the rows of the
// page that this step does not fill. From then on every row of a page a request holds is either
// the request's own or zero.
#include "common.cuh"

// Clears rows `first_row .. page_size` of one (page, kv head) tile, which are contiguous.
template <typename T>
__device__ __forceinline__ void clear_page_tail(T* tile, int first_row, int page_size, int head_dim) {
  if (first_row >= page_size) return;
  const int64_t begin = static_cast<int64_t>(first_row) * head_dim * sizeof(T);
  const int64_t end = static_cast<int64_t>(page_size) * head_dim * sizeof(T);
  unsigned char* base = reinterpret_cast<unsigned char*>(tile);
  if ((static_cast<int64_t>(head_dim) * sizeof(T)) % 16 == 0 && reinterpret_cast<uintptr_t>(base) % 16 == 0) {
    for (int64_t at = begin + threadIdx.x * 16; at < end; at += static_cast<int64_t>(blockDim.x) * 16)
      *reinterpret_cast<uint4*>(base + at) = make_uint4(0u, 0u, 0u, 0u);
  } else {
    T* elems = tile + static_cast<int64_t>(first_row) * head_dim;
    const int count = (page_size - first_row) * head_dim;
    for (int i = threadIdx.x; i < count; i += blockDim.x) elems[i] = from_f32<T>(0.f);
  }
}

constexpr int kWideTokens = 64;  // from this many tokens on, one block per token (below)

// One block per (token, head): query heads first, then key heads, then value heads. Thread i
// handles pair slot i of its head (see below), so a decode step spreads over
// tokens * (q_heads + 2 * kv_heads) small blocks instead of one block per token.
template <typename T>
__global__ void rope_kv_write_kernel(const T* qkv, const float* __restrict__ bias,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ seq_kv_len,
                                     const int* __restrict__ block_table, int max_pages,
                                     int num_pages, T* k_arena,
                                     T* v_arena, T* q_out, int q_heads,
                                     int kv_heads, int head_dim, int rot, int page_size,
                                     int write_kv, int* err) {
  let_successor_start();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0 .. q_heads + 2 * kv_heads
  const int rotated_heads = q_heads + kv_heads;
  const bool is_q = head < q_heads, is_k = !is_q && head < rotated_heads;
  if (!is_q && !write_kv) {
    wait_for_predecessor();
    let_successor_start();
    return;
  }
  // Where the row goes and by what angle it turns comes from the step's metadata and from
  // constants, both on the device before the kernel in front ran: fetched before the wait for
  // it, the chain position -> table entry costs nothing afterwards.
  const int pos = positions[t];
  const int half_rot = rot / 2, half = head_dim / 2;
  T* dst = nullptr;
  int clear_from = 0;  // for the token that starts a page: the first row this step leaves unwritten
  if (is_q) {
    dst = q_out + (static_cast<int64_t>(t) * q_heads + head) * head_dim;
  } else {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      const int page = block_table[static_cast<int64_t>(token_seq[t]) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_PAGE);
      } else {
        const int kv_head = is_k ? head - q_heads : head - rotated_heads;
        dst = (is_k ? k_arena : v_arena) + kv_row_offset(page, kv_head, pos % page_size, kv_heads, page_size, head_dim);
        if (pos % page_size == 0 && seq_kv_len != nullptr) clear_from = max(1, seq_kv_len[token_seq[t]] - pos);
      }
    }
  }
  const int width = (q_heads + 2 * kv_heads) * head_dim;
  const T* src = qkv + static_cast<int64_t>(t) * width + head * head_dim;
  const float* b = bias ? bias + head * head_dim : nullptr;
  // This thread's first pair slot (the only one when the block has a thread per slot): its
  // bias and its sine and cosine, also ahead of the wait.
  const int first_slot = threadIdx.x;
  float first_b0 = 0.f, first_b1 = 0.f, first_sn = 0.f, first_cs = 1.f;
  if (first_slot < half) {
    const int d0 = first_slot < half_rot ? first_slot : rot + 2 * (first_slot - half_rot);
    const int d1 = first_slot < half_rot ? first_slot + half_rot : d0 + 1;
    if (b) {
      first_b0 = b[d0];
      first_b1 = b[d1];
    }
    if ((is_q || is_k) && first_slot < half_rot) sincosf(static_cast<float>(pos) * inv_freq[first_slot], &first_sn, &first_cs);
  }
  wait_for_predecessor();
  let_successor_start();
  if (dst == nullptr) return;
  if (clear_from > 0) clear_page_tail(dst, clear_from, page_size, head_dim);  // dst is row 0 of the tile

  // Pair slot i: below rot/2 it is the rotated pair (i, i + rot/2); the rest are the two
  // trailing dims a partial rotation leaves alone. Value heads are copied (bias added).
  for (int slot = threadIdx.x; slot < half; slot += blockDim.x) {
    int d0, d1;
    const bool rotate = (is_q || is_k) && slot < half_rot;
    if (slot < half_rot) {
      d0 = slot;
      d1 = slot + half_rot;
    } else {
      d0 = rot + 2 * (slot - half_rot);
      d1 = d0 + 1;
    }
    float x0 = to_f32<T>(src[d0]), x1 = to_f32<T>(src[d1]);
    float sn = first_sn, cs = first_cs;
    if (slot == first_slot) {
      x0 += first_b0;
      x1 += first_b1;
    } else {
      if (b) {
        x0 += b[d0];
        x1 += b[d1];
      }
      if (rotate) sincosf(static_cast<float>(pos) * inv_freq[slot], &sn, &cs);
    }
    if (rotate) {
      const float y0 = x0 * cs - x1 * sn, y1 = x1 * cs + x0 * sn;
      x0 = y0;
      x1 = y1;
    }
    dst[d0] = from_f32<T>(x0);
    dst[d1] = from_f32<T>(x1);
  }
}

// The same work for many tokens (prompt portions): one block per token. The token's sines and
// cosines are computed once into shared memory and shared by all its heads, and every thread
// moves two adjacent dims at a time (one 32-bit access for bfloat16). Full rotation only
// (rot == head_dim, head_dim a multiple of 4); the arithmetic per element is that of the
// kernel above.
template <typename T>
struct Pair;
template <>
struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __nv_bfloat162(__float2bfloat16_rn(a), __float2bfloat16_rn(b));
  }
};

template <typename T>
__global__ void rope_kv_write_wide_kernel(const T* qkv, const float* __restrict__ bias,
                                          const float* __restrict__ inv_freq,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ token_seq,
                                          const int* __restrict__ seq_kv_len,
                                          const int* __restrict__ block_table, int max_pages,
                                          int num_pages, T* k_arena,
                                          T* v_arena, T* q_out, int q_heads,
                                          int kv_heads, int head_dim, int page_size, int write_kv,
                                          int* err) {
  extern __shared__ float angles[];  // cos[half], sin[half]
  wait_for_predecessor();
  let_successor_start();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = head_dim / 2;
  for (int slot = threadIdx.x; slot < half; slot += blockDim.x) {
    float sn, cs;
    sincosf(static_cast<float>(pos) * inv_freq[slot], &sn, &cs);
    angles[slot] = cs;
    angles[half + slot] = sn;
  }
  int64_t kv_row = -1;
  if (write_kv) {
    const int logical = pos / page_size;
    if (pos < 0 || logical >= max_pages) {
      if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_POSITION);
    } else {
      const int page = block_table[static_cast<int64_t>(token_seq[t]) * max_pages + logical];
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, ERRBIT_BAD_PAGE);
      } else {
        kv_row = kv_row_offset(page, 0, pos % page_size, kv_heads, page_size, head_dim);
        if (pos % page_size == 0 && seq_kv_len != nullptr) {
          // This token starts the page: clear the rows of every kv head's tile that the step's
          // later tokens will not fill (kv_row is row 0 of head 0's tile here).
          const int clear_from = max(1, seq_kv_len[token_seq[t]] - pos);
          for (int h = 0; h < kv_heads; ++h) {
            const int64_t tile = kv_row + static_cast<int64_t>(h) * page_size * head_dim;
            clear_page_tail(k_arena + tile, clear_from, page_size, head_dim);
            clear_page_tail(v_arena + tile, clear_from, page_size, head_dim);
          }
        }
      }
    }
  }
  __syncthreads();
  const int rotated_heads = q_heads + kv_heads;
  const int heads = write_kv ? q_heads + 2 * kv_heads : q_heads;
  const int pairs = half / 2;  // pairs of adjacent slots per head
  const int width = (q_heads + 2 * kv_heads) * head_dim;
  const T* row = qkv + static_cast<int64_t>(t) * width;
  const int64_t head_stride = static_cast<int64_t>(page_size) * head_dim;  // between kv heads of a page
  for (int item = threadIdx.x; item < heads * pairs; item += blockDim.x) {
    const int head = item / pairs, slot = 2 * (item - head * pairs);
    T* dst;
    if (head < q_heads) {
      dst = q_out + (static_cast<int64_t>(t) * q_heads + head) * head_dim;
    } else {
      if (kv_row < 0) continue;
      const bool is_k = head < rotated_heads;
      dst = (is_k ? k_arena : v_arena) + kv_row + (is_k ? head - q_heads : head - rotated_heads) * head_stride;
    }
    const T* src = row + head * head_dim;
    float2 lo = Pair<T>::load(src + slot), hi = Pair<T>::load(src + half + slot);
    if (bias) {
      const float* b = bias + head * head_dim;
      lo.x += b[slot];
      lo.y += b[slot + 1];
      hi.x += b[half + slot];
      hi.y += b[half + slot + 1];
    }
    if (head < rotated_heads) {
      const float c0 = angles[slot], c1 = angles[slot + 1], s0 = angles[half + slot], s1 = angles[half + slot + 1];
      const float a0 = lo.x * c0 - hi.x * s0, b0 = hi.x * c0 + lo.x * s0;
      const float a1 = lo.y * c1 - hi.y * s1, b1 = hi.y * c1 + lo.y * s1;
      lo = make_float2(a0, a1);
      hi = make_float2(b0, b1);
    }
    Pair<T>::store(dst + slot, lo.x, lo.y);
    Pair<T>::store(dst + half + slot, hi.x, hi.y);
  }
}

// `seq_kv_len` (may be null: nothing is cleared then) holds, per request of the step, the number
// of keys the request has after the step.
B200_API int b200_rope_kv_write(const void* qkv, const float* bias, const float* inv_freq,
                                const int* positions, const int* token_seq, const int* seq_kv_len,
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
  if (tokens >= kWideTokens && rot == head_dim && head_dim % 4 == 0) {
    const size_t angles = static_cast<size_t>(head_dim) * sizeof(float);
    const dim3 wide_grid(tokens), wide_block(256);
    if (dtype == DTYPE_F32) {
      launch_kernel(rope_kv_write_wide_kernel<float>, wide_grid, wide_block, angles, stream,
          static_cast<const float*>(qkv), bias, inv_freq, positions, token_seq, seq_kv_len, block_table,
          max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena),
          static_cast<float*>(q_out), q_heads, kv_heads, head_dim, page_size, write_kv, err);
    } else if (dtype == DTYPE_BF16) {
      launch_kernel(rope_kv_write_wide_kernel<__nv_bfloat16>, wide_grid, wide_block, angles, stream,
          static_cast<const __nv_bfloat16*>(qkv), bias, inv_freq, positions, token_seq, seq_kv_len, block_table,
          max_pages, num_pages, static_cast<__nv_bfloat16*>(k_arena),
          static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), q_heads,
          kv_heads, head_dim, page_size, write_kv, err);
    } else {
      return b200_fail("rope_kv_write: unknown dtype %d", dtype);
    }
    return b200_check_launch("rope_kv_write");
  }
  const int threads = head_dim >= 128 ? 64 : 32;
  const size_t smem = 0;
  const dim3 grid(tokens, q_heads + 2 * kv_heads);
  B200_REQUIRE(grid.y <= 65535, "rope_kv_write: too many heads");
  if (dtype == DTYPE_F32) {
    launch_kernel(rope_kv_write_kernel<float>, grid, dim3(threads), smem, stream,
        static_cast<const float*>(qkv), bias, inv_freq, positions, token_seq, seq_kv_len, block_table,
        max_pages, num_pages, static_cast<float*>(k_arena), static_cast<float*>(v_arena),
        static_cast<float*>(q_out), q_heads, kv_heads, head_dim, rot, page_size, write_kv, err);
  } else if (dtype == DTYPE_BF16) {
    launch_kernel(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream,
        static_cast<const __nv_bfloat16*>(qkv), bias, inv_freq, positions, token_seq, seq_kv_len, block_table,
        max_pages, num_pages, static_cast<__nv_bfloat16*>(k_arena),
        static_cast<__nv_bfloat16*>(v_arena), static_cast<__nv_bfloat16*>(q_out), q_heads,
        kv_heads, head_dim, rot, page_size, write_kv, err);
  } else {
    return b200_fail("rope_kv_write: unknown dtype %d", dtype);
  }
  return b200_check_launch("rope_kv_write");
}
