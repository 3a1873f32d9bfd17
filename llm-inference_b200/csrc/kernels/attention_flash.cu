// Paged flash attention on tensor cores for bfloat16: prefill portions and decoded tokens.
//
// Work is laid out per (request, kv head). The query rows of that pair are every
// (new token, query head of the kv head's group) combination, so one pass over the
// request's keys and values serves all `q_heads / kv_heads` heads that share them
// (the reference's Metal kernel shares each K/V row the same way,
// python/instinct/backends/metal_kernels.py:9-17,18-101). Keys and values are read straight
// from the arena's pages through the block table, 64 keys at a time, into a ring of swizzled
// shared-memory tiles with cp.async (two tiles deep; three blocks share an SM and cover each
// other's waits); scores and the weighted sum use mma.sync
// m16n8k16 with 32-bit accumulators and a 32-bit running softmax (max and sum per row).
//
// Two shapes of block, one body:
//   * prefill: 4 warps own 16 query rows each (64 rows per block) and walk all keys;
//   * decode : the request has one new token, its <= 16 rows are shared by the 4 warps, each
//     warp takes a quarter of every 64-key tile, and the key range is cut into `splits`
//     blocks whose partial results (max, sum, unnormalised output) a second small kernel
//     merges, as python/instinct/backends/metal_kernels.py:103-124 does. A decode block
//     starts fetching keys that earlier steps wrote before it waits for the kernel in front
//     of it on the stream, which only produces the newest key.
// Masking follows python/instinct/batches.py:110-113: key <= query position, and with a
// window key > position - window.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int kTileKeys = 64;
constexpr int kWarps = 4;
constexpr int kFlashThreads = kWarps * 32;
constexpr int kMaxClusterSplits = 16;  // splits that may merge on chip: the widest cluster

// An engine built for long requests cuts the key range more than 16 ways (the split count is
// fixed when a decode step is captured, for the longest request allowed). A short request then
// gives each split at least two 64-key tiles and leaves the other splits empty, which is how
// it would have been cut with 16.
__device__ __forceinline__ int min_tiles_per_split(int splits) { return splits > kMaxClusterSplits ? 2 : 1; }
constexpr float kLog2e = 1.4426950408889634f;

struct FlashParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_arena;
  const __nv_bfloat16* v_arena;
  __nv_bfloat16* out;
  const int* block_table;
  const int* seq_q_start;
  const int* seq_q_len;
  const int* seq_kv_len;
  float* partial_out;  // [tokens, q_heads, splits, head_dim]
  float* partial_ml;   // [tokens, q_heads, splits, 2]
  int* err;
  int first_seq;
  int max_pages, num_pages;
  int q_heads, kv_heads, group;
  int page_shift, page_mask;
  int window;
  int splits;
  int cluster_merge;  // the splits of a (request, kv head) are one thread-block cluster and merge on chip
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a swizzled [rows][HEAD_DIM] bf16 tile.
template <int HEAD_DIM>
__device__ __forceinline__ int tile_offset(int row, int chunk) {
  return row * (HEAD_DIM * 2) + ((chunk ^ (row & 7)) << 4);
}

// Copies keys and values [tile_start, tile_start + 64) of one kv head into their shared-memory
// tiles; rows outside [lo, hi] are zero-filled (they may lie in pages the request no longer
// holds). The block-table entries of all of a thread's rows are fetched first, in one batch
// of independent loads, and serve both the key and the value copy: looked up row by row, each
// copy would wait a full memory round trip for its page id.
template <int HEAD_DIM>
__device__ __forceinline__ void load_tile(unsigned char* k_dst, unsigned char* v_dst, const int* table,
                                          const FlashParams& p, int kv_head, int tile_start, int lo, int hi) {
  constexpr int kChunks = HEAD_DIM / 8;
  constexpr int kRowsPerPass = kFlashThreads / kChunks;
  constexpr int kPasses = kTileKeys / kRowsPerPass;
  const int chunk = threadIdx.x % kChunks;
  const int row0 = threadIdx.x / kChunks;
  const int page_size = p.page_mask + 1;
  if (page_size >= kTileKeys) {
    // The whole tile lies in one page (tiles start at multiples of 64 and the page size is a
    // power of two): one table entry, then a fixed stride from row to row.
    const bool any = tile_start + kTileKeys - 1 >= lo && tile_start <= hi;
    const int page = any ? __ldg(table + (tile_start >> p.page_shift)) : 0;
    const bool page_ok = page >= 0 && page < p.num_pages;
    if (any && !page_ok) atomicOr(p.err, ERRBIT_BAD_PAGE);
    const int64_t base = page_ok ? ((static_cast<int64_t>(page) * p.kv_heads + kv_head) * page_size +
                                    (tile_start & p.page_mask) + row0) * HEAD_DIM + chunk * 8
                                 : 0;
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
      const int row = row0 + pass * kRowsPerPass;
      const int key = tile_start + row;
      const bool valid = page_ok && key >= lo && key <= hi;
      const int64_t offset = valid ? base + static_cast<int64_t>(pass) * kRowsPerPass * HEAD_DIM : 0;
      cp_async_16(smem_u32(k_dst + tile_offset<HEAD_DIM>(row, chunk)), p.k_arena + offset, valid);
      cp_async_16(smem_u32(v_dst + tile_offset<HEAD_DIM>(row, chunk)), p.v_arena + offset, valid);
    }
    return;
  }
  int pages[kPasses];
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int key = tile_start + row0 + pass * kRowsPerPass;
    pages[pass] = (key >= lo && key <= hi) ? __ldg(table + (key >> p.page_shift)) : -1;
  }
#pragma unroll
  for (int pass = 0; pass < kPasses; ++pass) {
    const int row = row0 + pass * kRowsPerPass;
    const int key = tile_start + row;
    const bool in_range = key >= lo && key <= hi;
    const int page = pages[pass];
    bool valid = in_range && page >= 0 && page < p.num_pages;
    if (in_range && !valid) atomicOr(p.err, ERRBIT_BAD_PAGE);
    const int64_t offset = valid ? ((static_cast<int64_t>(page) * p.kv_heads + kv_head) * page_size +
                                    (key & p.page_mask)) * HEAD_DIM + chunk * 8
                                 : 0;
    cp_async_16(smem_u32(k_dst + tile_offset<HEAD_DIM>(row, chunk)), p.k_arena + offset, valid);
    cp_async_16(smem_u32(v_dst + tile_offset<HEAD_DIM>(row, chunk)), p.v_arena + offset, valid);
  }
}

// The end of a decode block: the four warps hold partial results (running maximum, sum and
// unnormalised output) for disjoint keys of the same <= 16 rows. They are merged through shared
// memory (`smem`, at least (kWarps + 1) * 16 * (HEAD_DIM + 2) floats that nothing else uses any
// more); the block's result is then final (one split), handed to the merge kernel through
// scratch, or merged with the other splits on chip when they form a thread-block cluster.
// How a decode block's result leaves it: as the answer (one split), as a partial result for the
// merge kernel, or through the cluster's shared memory. FINISH_ANY decides at run time; the
// kernels that are compiled for one way carry no code for the others (a block runs this once,
// from a cold instruction cache).
enum : int { FINISH_ANY = -1, FINISH_WHOLE = 0, FINISH_PARTIAL = 1, FINISH_CLUSTER = 2 };

template <int HEAD_DIM, int FINISH = FINISH_ANY>
__device__ __forceinline__ void finish_decode_block(const FlashParams& p, unsigned char* smem,
                                                    const float (&o)[HEAD_DIM / 8][4], float m0, float l0,
                                                    float m1, float l1, int rows_total, int kv_head,
                                                    int q_start, int split) {
  constexpr int kDimTiles = HEAD_DIM / 8;
  const bool whole = FINISH == FINISH_ANY ? p.splits == 1 : FINISH == FINISH_WHOLE;
  const bool cluster = FINISH == FINISH_ANY ? (p.splits > 1 && p.cluster_merge) : FINISH == FINISH_CLUSTER;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (lane & 3) * 2;
  // Merge the four warps' partial results through shared memory (the K/V tiles are
  // no longer needed), then either finish or hand the block's partial to the merge kernel.
  __syncthreads();
  float* merge_o = reinterpret_cast<float*>(smem);                  // [warps][16][HEAD_DIM]
  float* merge_ml = merge_o + kWarps * 16 * HEAD_DIM;                // [warps][16][2]
  float* block_o = merge_ml + kWarps * 16 * 2;                       // [16][HEAD_DIM], this block's result
  float* block_ml = block_o + 16 * HEAD_DIM;                         // [16][2]
  {
    const int lr0 = lane >> 2, lr1 = lr0 + 8;
#pragma unroll
    for (int i = 0; i < kDimTiles; ++i) {
      float* a = merge_o + (warp * 16 + lr0) * HEAD_DIM + i * 8 + col;
      float* b = merge_o + (warp * 16 + lr1) * HEAD_DIM + i * 8 + col;
      a[0] = o[i][0];
      a[1] = o[i][1];
      b[0] = o[i][2];
      b[1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      merge_ml[(warp * 16 + lr0) * 2 + 0] = m0;
      merge_ml[(warp * 16 + lr0) * 2 + 1] = l0;
      merge_ml[(warp * 16 + lr1) * 2 + 0] = m1;
      merge_ml[(warp * 16 + lr1) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  for (int item = threadIdx.x; item < rows_total * HEAD_DIM; item += kFlashThreads) {
    const int row = item / HEAD_DIM, d = item - row * HEAD_DIM;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, merge_ml[(w * 16 + row) * 2]);
    const float use = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = exp2f(merge_ml[(w * 16 + row) * 2] - use);
      l += merge_ml[(w * 16 + row) * 2 + 1] * f;
      acc += merge_o[(w * 16 + row) * HEAD_DIM + d] * f;
    }
    const int tok = row / p.group;
    const int head = kv_head * p.group + (row - tok * p.group);
    const int64_t out_row = static_cast<int64_t>(q_start + tok) * p.q_heads + head;
    if (whole) {
      p.out[out_row * HEAD_DIM + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else if (cluster) {
      block_o[row * HEAD_DIM + d] = acc;
      if (d == 0) {
        block_ml[row * 2 + 0] = m;
        block_ml[row * 2 + 1] = l;
      }
    } else {
      p.partial_out[(out_row * p.splits + split) * HEAD_DIM + d] = acc;
      if (d == 0) {
        p.partial_ml[(out_row * p.splits + split) * 2 + 0] = m;
        p.partial_ml[(out_row * p.splits + split) * 2 + 1] = l;
      }
    }
  }
  if (!cluster) return;

  // The splits of this (request, kv head) are the blocks of one cluster. Each left its partial
  // result in its own shared memory; after a cluster barrier every block finishes a slice of
  // the head dims, adding the splits in rank order through distributed shared memory:
  // out = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M).
  cluster_sync_all();
  {
    // Weights of the splits per row, gathered once: weight[r][row] = 2^(m_r - M) / L.
    float* weight = merge_o;  // [splits][16]; the warps' partials are no longer needed
    // Loads from the other blocks' shared memory are requested together and used afterwards:
    // one round trip through the cluster, not one per value.
    constexpr int kItems = (kMaxClusterSplits * 16 + kFlashThreads - 1) / kFlashThreads;
    float2 gathered[kItems];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const int item = threadIdx.x + i * kFlashThreads;
      const int r = item >> 4, row = item & 15;
      gathered[i] = make_float2(-INFINITY, 0.f);
      if (item < p.splits * 16 && row < rows_total) {
        gathered[i].x = load_peer_f32(block_ml + row * 2, r);
        gathered[i].y = load_peer_f32(block_ml + row * 2 + 1, r);
      }
    }
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const int item = threadIdx.x + i * kFlashThreads;
      if (item < p.splits * 16) {
        weight[item] = gathered[i].x;
        weight[p.splits * 16 + item] = gathered[i].y;
      }
    }
    __syncthreads();
    if (threadIdx.x < 16) {
      const int row = threadIdx.x;
      float m = -INFINITY;
      for (int r = 0; r < p.splits; ++r) m = fmaxf(m, weight[r * 16 + row]);
      const float use = m == -INFINITY ? 0.f : m;
      float l = 0.f;
      for (int r = 0; r < p.splits; ++r) l += weight[p.splits * 16 + r * 16 + row] * exp2f(weight[r * 16 + row] - use);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      for (int r = 0; r < p.splits; ++r) weight[r * 16 + row] = exp2f(weight[r * 16 + row] - use) * inv;
    }
    __syncthreads();
    const int slice = (HEAD_DIM + p.splits - 1) / p.splits;
    const int d_begin = split * slice, d_end = min(HEAD_DIM, d_begin + slice);
    const int width = max(0, d_end - d_begin);
    for (int item = threadIdx.x; item < rows_total * width; item += kFlashThreads) {
      const int row = item / width, d = d_begin + (item - row * width);
      float values[kMaxClusterSplits];
#pragma unroll
      for (int r = 0; r < kMaxClusterSplits; ++r)
        if (r < p.splits) values[r] = load_peer_f32(block_o + row * HEAD_DIM + d, r);
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxClusterSplits; ++r)
        if (r < p.splits) acc += values[r] * weight[r * 16 + row];
      const int tok = row / p.group;
      const int head = kv_head * p.group + (row - tok * p.group);
      const int64_t out_row = static_cast<int64_t>(q_start + tok) * p.q_heads + head;
      p.out[out_row * HEAD_DIM + d] = __float2bfloat16_rn(acc);
    }
  }
  cluster_sync_all();  // nobody leaves while its shared memory is still being read
}

template <int HEAD_DIM, bool DECODE>
__global__ void __launch_bounds__(kFlashThreads)
paged_flash_attention_kernel(const FlashParams p) {
  constexpr int kKSteps = HEAD_DIM / 16;   // k-steps of the score product
  constexpr int kDimTiles = HEAD_DIM / 8;  // n-tiles of the output
  constexpr int kTileBytes = kTileKeys * HEAD_DIM * 2;
  constexpr int kRing = 2;  // tiles in flight; small, so that three blocks share an SM and hide each other's waits

  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* k_tiles = smem;
  unsigned char* v_tiles = smem + kRing * kTileBytes;

  // The step's metadata (lengths, block tables) was copied to the device before any kernel of
  // the step ran, so it may be read before the wait; queries and the newest keys may not.
  if (!DECODE) wait_for_predecessor();
  let_successor_start();
  const int seq = p.first_seq + blockIdx.z;
  const int kv_head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_len = p.seq_q_len[seq];
  const int kv_len = p.seq_kv_len[seq];
  const int q_start = p.seq_q_start[seq];
  const int first_pos = kv_len - q_len;  // position of the request's first new token
  const int rows_total = q_len * p.group;
  const int* table = p.block_table + static_cast<int64_t>(seq) * p.max_pages;

  int row_base;  // first row of this warp's 16-row block
  int split = 0;
  if (DECODE) {
    row_base = 0;
    split = blockIdx.x;
  } else {
    row_base = blockIdx.x * (kWarps * 16) + warp * 16;
    if (blockIdx.x * (kWarps * 16) >= rows_total) return;
  }

  // Key range this block walks.
  int block_first_token, block_last_token;
  if (DECODE) {
    block_first_token = 0;
    block_last_token = q_len - 1;
  } else {
    block_first_token = (blockIdx.x * (kWarps * 16)) / p.group;
    block_last_token = min(q_len - 1, (blockIdx.x * (kWarps * 16) + kWarps * 16 - 1) / p.group);
  }
  int lo = p.window > 0 ? max(0, first_pos + block_first_token - p.window + 1) : 0;
  int hi = first_pos + block_last_token;  // inclusive
  int tile_begin = lo / kTileKeys, tile_end = hi / kTileKeys + 1;
  if (DECODE && p.splits > 1) {
    const int tiles = tile_end - tile_begin;
    const int per_split = max(min_tiles_per_split(p.splits), (tiles + p.splits - 1) / p.splits);
    tile_begin = tile_begin + split * per_split;
    tile_end = min(tile_end, tile_begin + per_split);
  }
  const int num_tiles = max(0, tile_end - tile_begin);

  // This thread's two rows (r0 = lane / 4 and r0 + 8 of the warp's block).
  const int r0 = row_base + (lane >> 2), r1 = r0 + 8;
  const int tok0 = r0 / p.group, tok1 = r1 / p.group;
  const int head0 = kv_head * p.group + (r0 - tok0 * p.group);
  const int head1 = kv_head * p.group + (r1 - tok1 * p.group);
  const bool live0 = r0 < rows_total, live1 = r1 < rows_total;
  const int pos0 = first_pos + tok0, pos1 = first_pos + tok1;

  float o[kDimTiles][4];
#pragma unroll
  for (int i = 0; i < kDimTiles; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // Fill the ring. Tiles that hold only keys of earlier steps are requested before the wait
  // for the kernel in front (decode only); they always come first in the block's range. Every
  // slot of the ring gets its own commit group, empty if the range is shorter.
  auto fetch = [&](int it) {
    const int slot = it % kRing;
    load_tile<HEAD_DIM>(k_tiles + slot * kTileBytes, v_tiles + slot * kTileBytes, table, p, kv_head,
                        (tile_begin + it) * kTileKeys, lo, hi);
  };
  int issued = 0;
  if (DECODE) {
    while (issued < kRing && issued < num_tiles && (tile_begin + issued + 1) * kTileKeys <= first_pos) {
      fetch(issued);
      cp_async_commit();
      ++issued;
    }
    wait_for_predecessor();
  }
  for (; issued < kRing; ++issued) {
    if (issued < num_tiles) fetch(issued);
    cp_async_commit();
  }

  // Query fragments, straight from global memory.
  uint32_t qf[kKSteps][4];
  {
    const __nv_bfloat16* q0 = p.q + (static_cast<int64_t>(q_start + tok0) * p.q_heads + head0) * HEAD_DIM;
    const __nv_bfloat16* q1 = p.q + (static_cast<int64_t>(q_start + tok1) * p.q_heads + head1) * HEAD_DIM;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      qf[ks][0] = live0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + col) : 0u;
      qf[ks][1] = live1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + col) : 0u;
      qf[ks][2] = live0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + col) : 0u;
      qf[ks][3] = live1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + col) : 0u;
    }
  }


  for (int it = 0; it < num_tiles; ++it) {
    const int stage = it % kRing;
    const int tile_start = (tile_begin + it) * kTileKeys;
    // One group is committed per iteration, so all but the newest kRing - 1 have landed.
    cp_async_wait<kRing - 1>();
    __syncthreads();

    const uint32_t k_base = smem_u32(k_tiles + stage * kTileBytes);
    const uint32_t v_base = smem_u32(v_tiles + stage * kTileBytes);
    // Does any element of this tile need masking for this warp's rows?
    const bool tile_needs_mask =
        (tile_start + kTileKeys - 1 > first_pos + min(tok0, q_len - 1)) ||
        (p.window > 0 && tile_start <= pos1 - p.window) || (tile_start < lo) || !live1;

    {
      // A prefill warp takes all 64 keys of the tile for its 16 rows (eight independent score
      // tiles, one softmax update per tile); a decode warp takes its quarter of the tile.
      constexpr int kGroups = DECODE ? 1 : kTileKeys / 16;  // groups of 16 keys per warp per tile
      const int group0 = DECODE ? warp : 0;
      const int key_base = tile_start + group0 * 16;
      float s[2 * kGroups][4];
#pragma unroll
      for (int n = 0; n < 2 * kGroups; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      {
        const int mi = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
          for (int gidx = 0; gidx < kGroups; ++gidx) {
            const int krow = (group0 + gidx) * 16 + (mi >> 1) * 8 + (lane & 7);
            uint32_t b[4];
            ldmatrix_x4(b, k_base + tile_offset<HEAD_DIM>(krow, ks * 2 + (mi & 1)));
            mma_bf16(s[2 * gidx], qf[ks], b[0], b[1]);
            mma_bf16(s[2 * gidx + 1], qf[ks], b[2], b[3]);
          }
        }
      }
      // Scale, mask, running softmax. Element (n, e): row = e < 2 ? r0 : r1,
      // key = key_base + n * 8 + (lane % 4) * 2 + (e & 1).
      float tile_max0 = -INFINITY, tile_max1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2 * kGroups; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[n][e] * p.scale_log2;
          if (tile_needs_mask) {
            const int key = key_base + n * 8 + (lane & 3) * 2 + (e & 1);
            const int pos = e < 2 ? pos0 : pos1;
            const bool live = e < 2 ? live0 : live1;
            const bool visible = live && key <= pos && key >= lo && (p.window == 0 || key > pos - p.window);
            if (!visible) v = -INFINITY;
          }
          s[n][e] = v;
          if (e < 2) tile_max0 = fmaxf(tile_max0, v);
          else tile_max1 = fmaxf(tile_max1, v);
        }
      }
      tile_max0 = fmaxf(tile_max0, __shfl_xor_sync(0xffffffffu, tile_max0, 1));
      tile_max0 = fmaxf(tile_max0, __shfl_xor_sync(0xffffffffu, tile_max0, 2));
      tile_max1 = fmaxf(tile_max1, __shfl_xor_sync(0xffffffffu, tile_max1, 1));
      tile_max1 = fmaxf(tile_max1, __shfl_xor_sync(0xffffffffu, tile_max1, 2));
      const float new0 = fmaxf(m0, tile_max0), new1 = fmaxf(m1, tile_max1);
      const float use0 = new0 == -INFINITY ? 0.f : new0, use1 = new1 == -INFINITY ? 0.f : new1;
      const float alpha0 = exp2f(m0 - use0), alpha1 = exp2f(m1 - use1);
      m0 = new0;
      m1 = new1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pf[kGroups][4];
#pragma unroll
      for (int n = 0; n < 2 * kGroups; ++n) {
        const float p00 = exp2f(s[n][0] - use0), p01 = exp2f(s[n][1] - use0);
        const float p10 = exp2f(s[n][2] - use1), p11 = exp2f(s[n][3] - use1);
        sum0 += p00 + p01;
        sum1 += p10 + p11;
        pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p00, p01);  // rows r0: a0/a1 (even n), a4/a5 (odd n)
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p10, p11);  // rows r1: a2/a3 (even n), a6/a7 (odd n)
      }
      l0 = l0 * alpha0 + sum0;
      l1 = l1 * alpha1 + sum1;
      // Rescale the running output only when some row's maximum moved (the whole warp decides).
      if (__any_sync(0xffffffffu, alpha0 != 1.f || alpha1 != 1.f)) {
#pragma unroll
        for (int i = 0; i < kDimTiles; ++i) {
          o[i][0] *= alpha0;
          o[i][1] *= alpha0;
          o[i][2] *= alpha1;
          o[i][3] *= alpha1;
        }
      }
      // O += P V over the warp's keys, 16 at a time.
      {
        const int mi = lane >> 3;
#pragma unroll
        for (int gidx = 0; gidx < kGroups; ++gidx) {
          const int vrow = (group0 + gidx) * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
          for (int c = 0; c < kDimTiles; c += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_base + tile_offset<HEAD_DIM>(vrow, c + (mi >> 1)));
            mma_bf16(o[c], pf[gidx], b[0], b[1]);
            mma_bf16(o[c + 1], pf[gidx], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
    // The slot is free again: refill it with the tile kRing further on.
    if (it + kRing < num_tiles) fetch(it + kRing);
    cp_async_commit();
  }
  cp_async_wait<0>();

  // Row sums live in the four lanes that share a row.
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  const int col = (lane & 3) * 2;
  if (!DECODE) {
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    __nv_bfloat16* out0 = p.out + (static_cast<int64_t>(q_start + tok0) * p.q_heads + head0) * HEAD_DIM;
    __nv_bfloat16* out1 = p.out + (static_cast<int64_t>(q_start + tok1) * p.q_heads + head1) * HEAD_DIM;
#pragma unroll
    for (int i = 0; i < kDimTiles; ++i) {
      if (live0) *reinterpret_cast<uint32_t*>(out0 + i * 8 + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
      if (live1) *reinterpret_cast<uint32_t*>(out1 + i * 8 + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
    return;
  }

  finish_decode_block<HEAD_DIM>(p, smem, o, m0, l0, m1, l1, rows_total, kv_head, q_start, split);
}

// out[row, :] = sum_i partial_out[row, i, :] * 2^(m_i - M) / sum_i l_i * 2^(m_i - M), one block
// per (token, query head) row (python/instinct/backends/metal_kernels.py:103-124). The block
// is [head dims, groups]: group g takes splits 16 g .. 16 g + 15, so up to 64 splits cost one
// round trip to L2 and one pass through shared memory; a block of one group loops over more.
constexpr int kMergeGroups = 4;

__host__ __device__ constexpr int merge_groups(int splits) {
  return splits <= kMaxClusterSplits * kMergeGroups ? (splits + kMaxClusterSplits - 1) / kMaxClusterSplits : 1;
}

// FAST: at most kMaxClusterSplits splits per group of the block and a thread per head dim (the
// launcher knows); the general form loops. Two instantiations, so that the usual one is short.
// The partial results are written by the kernel in front while this one may already be resident
// (programmatic dependent launch): they are not `__restrict__`, which would allow the compiler
// to fetch them through the read-only path ahead of the wait for that kernel.
template <int HEAD_DIM, bool FAST>
__global__ void flash_merge_kernel(const float* partial_out, const float* partial_ml, __nv_bfloat16* out, int splits) {
  __shared__ float group_acc[kMergeGroups][HEAD_DIM];
  __shared__ float2 group_ml[kMergeGroups];
  let_successor_start();
  wait_for_predecessor();
  const int64_t row = blockIdx.x;
  const float2* ml = reinterpret_cast<const float2*>(partial_ml + row * splits * 2);
  const int groups = static_cast<int>(blockDim.y);
  if constexpr (FAST) {
    // Every load of this thread (its splits' maxima and sums, and its dim of each of their
    // outputs) is requested before the first is used: one round trip to L2 instead of three.
    const int d = threadIdx.x, g = threadIdx.y, base = g * kMaxClusterSplits;
    float2 stats[kMaxClusterSplits];
    float values[kMaxClusterSplits];
#pragma unroll
    for (int i = 0; i < kMaxClusterSplits; ++i) {
      const bool live = base + i < splits;
      stats[i] = live ? ml[base + i] : make_float2(-INFINITY, 0.f);
      values[i] = live && d < HEAD_DIM ? partial_out[(row * splits + base + i) * HEAD_DIM + d] : 0.f;
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxClusterSplits; ++i) m = fmaxf(m, stats[i].x);
    float use = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxClusterSplits; ++i) {
      const float f = exp2f(stats[i].x - use);
      l += stats[i].y * f;
      acc += values[i] * f;
    }
    if (groups > 1) {
      // The groups' results meet in shared memory and are added in group order.
      if (d < HEAD_DIM) group_acc[g][d] = acc;
      if (d == 0) group_ml[g] = make_float2(m, l);
      __syncthreads();
      if (g != 0) return;
      m = -INFINITY;
      for (int j = 0; j < groups; ++j) m = fmaxf(m, group_ml[j].x);
      use = m == -INFINITY ? 0.f : m;
      l = 0.f, acc = 0.f;
      for (int j = 0; j < groups; ++j) {
        const float f = exp2f(group_ml[j].x - use);
        l += group_ml[j].y * f;
        if (d < HEAD_DIM) acc += group_acc[j][d] * f;
      }
    }
    if (d < HEAD_DIM) out[row * HEAD_DIM + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  } else {
    if (threadIdx.y != 0) return;
    float m = -INFINITY;
#pragma unroll 8
    for (int i = 0; i < splits; ++i) m = fmaxf(m, ml[i].x);
    const float use = m == -INFINITY ? 0.f : m;
    float l = 0.f;
#pragma unroll 8
    for (int i = 0; i < splits; ++i) l += ml[i].y * exp2f(ml[i].x - use);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int d = threadIdx.x; d < HEAD_DIM; d += blockDim.x) {
      float acc = 0.f;
#pragma unroll 8
      for (int i = 0; i < splits; ++i)
        acc += partial_out[(row * splits + i) * HEAD_DIM + d] * exp2f(ml[i].x - use);
      out[row * HEAD_DIM + d] = __float2bfloat16_rn(acc * inv);
    }
  }
}

// The merge kernel for `splits` splits: the fast form when the block it is launched with
// (a thread per head dim x merge_groups(splits)) covers them.
template <int HEAD_DIM>
cudaError_t launch_merge(const float* partial_out, const float* partial_ml, __nv_bfloat16* out, int rows, int splits,
                         cudaStream_t stream) {
  const int groups = merge_groups(splits);
  const dim3 block(HEAD_DIM <= 64 ? 64 : 128, groups);
  if (splits <= kMaxClusterSplits * groups && HEAD_DIM <= 128)
    return launch_kernel(flash_merge_kernel<HEAD_DIM, true>, dim3(rows), block, 0, stream, partial_out, partial_ml, out, splits);
  return launch_kernel(flash_merge_kernel<HEAD_DIM, false>, dim3(rows), block, 0, stream, partial_out, partial_ml, out, splits);
}

// ---- decode with keys and values brought in by TMA ------------------------------------------
//
// The same split-key decode step as above for head_dim 128 and pages of at least 64 rows, with
// another way of feeding the warps. Above, all four warps copy a 64-key tile together with
// cp.async (16 copies and their addresses per thread and tile) and meet at two block barriers
// per tile. Here every warp owns its quarter of each tile outright: lane 0 asks the TMA unit
// for the warp's 16 keys and 16 values (four boxes of 16 rows x 64 dims, 128-byte swizzle, a
// (page, kv head) tile being contiguous in the arena), completion is counted on the warp's own
// mbarriers, and the warps never wait for each other before the end. A request costs one
// thread a handful of instructions, so the ring can be as deep as shared memory allows.
constexpr int kTmaDim = 128;
constexpr int kTmaMaxStages = 6;
constexpr int kWarpStageBytes = 2 * 16 * kTmaDim * 2;  // a warp's 16 keys and 16 values of one tile
constexpr int kTmaStagedTiles = 512;                    // page ids a block keeps in shared memory
constexpr long long kDecodeWaitCycles = 4000000000LL;   // about two seconds
constexpr int ERRBIT_TIMEOUT_D = 8;

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity; gives up after about two seconds.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - start > kDecodeWaitCycles) return false;
  }
}
// One box of the arena map: columns [x, x + 64) of rows [y, y + 16). x is 0 or 64 (a multiple
// of 8 elements, as the copy's 16-byte rule wants).
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` (0..15) in a warp's K or V piece:
// two boxes of 16 rows x 128 bytes, each swizzled as the TMA unit writes it (chunk ^ row % 8).
__device__ __forceinline__ int box_offset(int row, int chunk) {
  return (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

template <int FINISH>
__global__ void __launch_bounds__(kFlashThreads)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        const FlashParams p, const int stages) {
  constexpr int kKSteps = kTmaDim / 16;
  constexpr int kDimTiles = kTmaDim / 8;
  extern __shared__ unsigned char tma_smem_raw[];
  // The swizzle pattern is a function of the address: pieces start on 1,024-byte boundaries.
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tma_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + kWarps * stages * kWarpStageBytes);  // [warps][kTmaMaxStages]
  int* staged_pages = reinterpret_cast<int*>(bars + kWarps * kTmaMaxStages);                // [kTmaStagedTiles]

  let_successor_start();
  const int seq = p.first_seq + blockIdx.z;
  const int kv_head = blockIdx.y;
  const int split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_len = p.seq_kv_len[seq];
  const int q_start = p.seq_q_start[seq];
  const int first_pos = kv_len - 1;  // the one new token's position
  const int rows_total = p.group;
  const int* table = p.block_table + static_cast<int64_t>(seq) * p.max_pages;
  const int page_size = p.page_mask + 1;

  const int lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int hi = first_pos;
  int tile_begin = lo / kTileKeys, tile_end = hi / kTileKeys + 1;
  if (p.splits > 1) {
    const int tiles = tile_end - tile_begin;
    const int per_split = max(min_tiles_per_split(p.splits), (tiles + p.splits - 1) / p.splits);
    tile_begin = tile_begin + split * per_split;
    tile_end = min(tile_end, tile_begin + per_split);
  }
  const int num_tiles = max(0, tile_end - tile_begin);

  // Page ids of the block's tiles, checked once (a tile lies inside one page).
  auto lookup = [&](int it) -> int {
    const int page = __ldg(table + (((tile_begin + it) * kTileKeys) >> p.page_shift));
    if (page < 0 || page >= p.num_pages) {
      atomicOr(p.err, ERRBIT_BAD_PAGE);
      return 0;
    }
    return page;
  };
  for (int it = threadIdx.x; it < min(num_tiles, kTmaStagedTiles); it += kFlashThreads) staged_pages[it] = lookup(it);
  uint64_t* full = bars + warp * kTmaMaxStages;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // The warp's quarter of tile `it` holds keys key0(it) .. key0(it) + 15; the tiles in which
  // some of them lie in [lo, hi] are consecutive: [mine_begin, mine_end).
  const int key_off = tile_begin * kTileKeys + warp * 16;
  int mine_begin = 0, mine_end = num_tiles;
  while (mine_begin < mine_end && key_off + mine_begin * kTileKeys + 15 < lo) ++mine_begin;
  while (mine_end > mine_begin && key_off + (mine_end - 1) * kTileKeys > hi) --mine_end;
  const int mine = mine_end - mine_begin;

  unsigned char* my_ring = ring + warp * stages * kWarpStageBytes;
  auto request = [&](int j) {  // lane 0 only: the warp's j-th piece into slot j % stages
    const int it = mine_begin + j;
    const int page = it < kTmaStagedTiles ? staged_pages[it] : lookup(it);
    const int tile_start = (tile_begin + it) * kTileKeys;
    const int arena_row = (page * p.kv_heads + kv_head) * page_size + (tile_start & p.page_mask) + warp * 16;
    const int s = j % stages;
    unsigned char* dst = my_ring + s * kWarpStageBytes;
    mbar_expect_tx(&full[s], kWarpStageBytes);
    tma_box(dst, &k_map, &full[s], 0, arena_row);
    tma_box(dst + 2048, &k_map, &full[s], 64, arena_row);
    tma_box(dst + 4096, &v_map, &full[s], 0, arena_row);
    tma_box(dst + 6144, &v_map, &full[s], 64, arena_row);
  };
  // Pieces that hold only keys of earlier steps are requested before the wait for the kernel
  // in front on the stream, which writes the newest key.
  int requested = 0;
  while (requested < stages && requested < mine &&
         key_off + (mine_begin + requested) * kTileKeys + 16 <= first_pos) {
    if (lane == 0) request(requested);
    ++requested;
  }
  wait_for_predecessor();
  while (requested < stages && requested < mine) {
    if (lane == 0) request(requested);
    ++requested;
  }

  // This thread's two rows (lane / 4 and + 8) of the <= 16 query heads that share the kv head.
  const int r0 = lane >> 2, r1 = r0 + 8;
  const bool live0 = r0 < rows_total, live1 = r1 < rows_total;
  uint32_t qf[kKSteps][4];
  {
    const __nv_bfloat16* q0 = p.q + (static_cast<int64_t>(q_start) * p.q_heads + kv_head * p.group + r0) * kTmaDim;
    const __nv_bfloat16* q1 = p.q + (static_cast<int64_t>(q_start) * p.q_heads + kv_head * p.group + r1) * kTmaDim;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      qf[ks][0] = live0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + col) : 0u;
      qf[ks][1] = live1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + col) : 0u;
      qf[ks][2] = live0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + col) : 0u;
      qf[ks][3] = live1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + col) : 0u;
    }
  }

  float o[kDimTiles][4];
#pragma unroll
  for (int i = 0; i < kDimTiles; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int mi = lane >> 3;

  for (int j = 0; j < mine; ++j) {
    const int slot = j % stages;
    if (!mbar_wait(&full[slot], (j / stages) & 1)) {
      if (lane == 0) atomicOr(p.err, ERRBIT_TIMEOUT_D);
      // Give the copies still on their way the same bounded time, then leave the loop.
      for (int rest = j + 1; rest < requested; ++rest) mbar_wait(&full[rest % stages], (rest / stages) & 1);
      break;
    }
    const uint32_t k_base = smem_u32(my_ring + slot * kWarpStageBytes);
    const uint32_t v_base = k_base + kWarpStageBytes / 2;
    const int key_base = key_off + (mine_begin + j) * kTileKeys;

    // Scores of 16 rows x 16 keys; even and odd k-steps add into accumulators of their own, so
    // that no product waits for more than three others.
    float s[2][4], s_odd[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = s_odd[n][e] = 0.f;
    {
      const int krow = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < kKSteps; ks += 2) {
        uint32_t b[4], c[4];
        ldmatrix_x4(b, k_base + box_offset(krow, ks * 2 + (mi & 1)));
        ldmatrix_x4(c, k_base + box_offset(krow, ks * 2 + 2 + (mi & 1)));
        mma_bf16(s[0], qf[ks], b[0], b[1]);
        mma_bf16(s[1], qf[ks], b[2], b[3]);
        mma_bf16(s_odd[0], qf[ks + 1], c[0], c[1]);
        mma_bf16(s_odd[1], qf[ks + 1], c[2], c[3]);
      }
    }
    // Scale, mask, running softmax. Element (n, e): row = e < 2 ? r0 : r1,
    // key = key_base + n * 8 + (lane % 4) * 2 + (e & 1). Rows past the group compute on
    // zero queries and are never written.
    const bool needs_mask = key_base + 15 > hi || key_base < lo;
    float tile_max0 = -INFINITY, tile_max1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = (s[n][e] + s_odd[n][e]) * p.scale_log2;
        if (needs_mask) {
          const int key = key_base + n * 8 + (lane & 3) * 2 + (e & 1);
          if (key > hi || key < lo) v = -INFINITY;
        }
        s[n][e] = v;
        if (e < 2) tile_max0 = fmaxf(tile_max0, v);
        else tile_max1 = fmaxf(tile_max1, v);
      }
    }
    tile_max0 = fmaxf(tile_max0, __shfl_xor_sync(0xffffffffu, tile_max0, 1));
    tile_max0 = fmaxf(tile_max0, __shfl_xor_sync(0xffffffffu, tile_max0, 2));
    tile_max1 = fmaxf(tile_max1, __shfl_xor_sync(0xffffffffu, tile_max1, 1));
    tile_max1 = fmaxf(tile_max1, __shfl_xor_sync(0xffffffffu, tile_max1, 2));
    const float new0 = fmaxf(m0, tile_max0), new1 = fmaxf(m1, tile_max1);
    const float use0 = new0 == -INFINITY ? 0.f : new0, use1 = new1 == -INFINITY ? 0.f : new1;
    const float alpha0 = exp2f(m0 - use0), alpha1 = exp2f(m1 - use1);
    m0 = new0;
    m1 = new1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p00 = exp2f(s[n][0] - use0), p01 = exp2f(s[n][1] - use0);
      const float p10 = exp2f(s[n][2] - use1), p11 = exp2f(s[n][3] - use1);
      sum0 += p00 + p01;
      sum1 += p10 + p11;
      pf[n * 2 + 0] = pack_bf16(p00, p01);
      pf[n * 2 + 1] = pack_bf16(p10, p11);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
    if (__any_sync(0xffffffffu, alpha0 != 1.f || alpha1 != 1.f)) {
#pragma unroll
      for (int i = 0; i < kDimTiles; ++i) {
        o[i][0] *= alpha0;
        o[i][1] *= alpha0;
        o[i][2] *= alpha1;
        o[i][3] *= alpha1;
      }
    }
    {
      const int vrow = (mi & 1) * 8 + (lane & 7);
#pragma unroll
      for (int c = 0; c < kDimTiles; c += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_base + box_offset(vrow, c + (mi >> 1)));
        mma_bf16(o[c], pf, b[0], b[1]);
        mma_bf16(o[c + 1], pf, b[2], b[3]);
      }
    }
    // Every lane has read the slot; lane 0 hands it back to the TMA unit for piece j + stages.
    __syncwarp();
    if (requested < mine) {
      if (lane == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        request(requested);
      }
      ++requested;
    }
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  finish_decode_block<kTmaDim, FINISH>(p, ring, o, m0, l0, m1, l1, rows_total, kv_head, q_start, split);
}

template <int HEAD_DIM>
constexpr size_t flash_smem_bytes(bool decode) {
  (void)decode;
  const size_t tiles = 4 * static_cast<size_t>(kTileKeys) * HEAD_DIM * 2;
  const size_t merge = static_cast<size_t>(kWarps + 1) * 16 * (HEAD_DIM + 2) * sizeof(float);
  return tiles > merge ? tiles : merge;
}

template <int HEAD_DIM>
int launch_flash(const FlashParams& p, int num_seqs, int decode, int max_q_len, int tokens,
                 cudaStream_t stream) {
  const size_t smem = flash_smem_bytes<HEAD_DIM>(decode != 0);
  static bool configured = false;
  if (!configured) {
    cudaError_t a = cudaFuncSetAttribute(paged_flash_attention_kernel<HEAD_DIM, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(flash_smem_bytes<HEAD_DIM>(true)));
    cudaError_t b = cudaFuncSetAttribute(paged_flash_attention_kernel<HEAD_DIM, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(flash_smem_bytes<HEAD_DIM>(false)));
    if (a != cudaSuccess || b != cudaSuccess) return b200_fail("flash attention: cannot size shared memory");
    configured = true;
  }
  if (decode) {
    const dim3 grid(p.splits, p.kv_heads, num_seqs);
    if (p.splits > 1 && p.cluster_merge) {
      static bool wide_clusters = false;
      if (p.splits > 8 && !wide_clusters) {
        if (cudaFuncSetAttribute(paged_flash_attention_kernel<HEAD_DIM, true>,
                                 cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
          return b200_fail("flash attention: clusters of %d blocks are not allowed here", p.splits);
        wide_clusters = true;
      }
      cudaLaunchConfig_t config = {};
      config.gridDim = grid;
      config.blockDim = dim3(kFlashThreads);
      config.dynamicSmemBytes = smem;
      config.stream = stream;
      cudaLaunchAttribute attributes[2];
      attributes[0].id = cudaLaunchAttributeClusterDimension;
      attributes[0].val.clusterDim.x = p.splits;
      attributes[0].val.clusterDim.y = 1;
      attributes[0].val.clusterDim.z = 1;
      attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attributes[1].val.programmaticStreamSerializationAllowed = 1;
      config.attrs = attributes;
      config.numAttrs = b200_overlap_enabled() ? 2 : 1;
      const cudaError_t status = cudaLaunchKernelEx(&config, paged_flash_attention_kernel<HEAD_DIM, true>, p);
      if (status != cudaSuccess) return b200_fail("flash attention: %s", cudaGetErrorString(status));
      return 0;
    }
    launch_kernel(paged_flash_attention_kernel<HEAD_DIM, true>, grid, dim3(kFlashThreads), smem, stream, p);
    if (p.splits > 1) {
      launch_merge<HEAD_DIM>(p.partial_out, p.partial_ml, p.out, tokens * p.q_heads, p.splits, stream);
    }
  } else {
    const int row_blocks = (max_q_len * p.group + kWarps * 16 - 1) / (kWarps * 16);
    const dim3 grid(row_blocks, p.kv_heads, num_seqs);
    launch_kernel(paged_flash_attention_kernel<HEAD_DIM, false>, grid, dim3(kFlashThreads), smem, stream, p);
  }
  return b200_check_launch("paged_flash_attention");
}

using EncodeTiledD = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// One layer's K or V arena [pages, kv_heads, page_size, 128] seen as rows of 128 bfloat16, cut
// into boxes of 64 columns x 16 rows with the 128-byte swizzle.
int decode_arena_map(CUtensorMap* map, const void* arena, int64_t rows) {
  static EncodeTiledD encode = nullptr;
  if (encode == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeTiledD>(ptr);
  }
  if (encode == nullptr) return b200_fail("decode attention: the driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {kTmaDim, static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {kTmaDim * 2};
  const cuuint32_t box[2] = {64, 16};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(arena), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return b200_fail("decode attention: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(status));
  return 0;
}

size_t decode_tma_smem_bytes(int stages) {
  return 1024 + static_cast<size_t>(kWarps) * stages * kWarpStageBytes + kWarps * kTmaMaxStages * sizeof(uint64_t) +
         kTmaStagedTiles * sizeof(int);
}

}  // namespace

// Whether the tuned kernel takes this shape; the caller uses the plain kernel otherwise.
B200_API int b200_flash_attention_supported(int q_heads, int kv_heads, int head_dim, int page_size,
                                            int decode) {
  if (head_dim != 64 && head_dim != 128) return 0;
  if (q_heads % kv_heads) return 0;
  if (page_size <= 0 || (page_size & (page_size - 1))) return 0;
  if (decode && q_heads / kv_heads > 16) return 0;
  if (kv_heads > 65535) return 0;
  return 1;
}

// Scratch floats the decode form needs for `tokens` rows cut into `splits`.
B200_API int64_t b200_flash_attention_scratch_floats(int tokens, int q_heads, int head_dim, int splits) {
  return splits > 1 ? static_cast<int64_t>(tokens) * q_heads * splits * (head_dim + 2) : 0;
}

// Attention for requests [first_seq, first_seq + num_seqs) of the step. With `decode` each of
// them has exactly one new token and `tokens` = num_seqs. With splits > 1 the partial results
// are merged either on chip (scratch == nullptr, at most 16 splits: they form a thread-block
// cluster) or through `scratch` by a second kernel. Query and output rows are indexed by the
// step's token rows.
B200_API int b200_paged_flash_attention(const void* q, const void* k_arena, const void* v_arena,
                                        void* out, const int* block_table, const int* seq_q_start,
                                        const int* seq_q_len, const int* seq_kv_len, int first_seq,
                                        int num_seqs, int tokens, int max_q_len, int max_pages,
                                        int num_pages, int q_heads, int kv_heads, int head_dim,
                                        int page_size, int window, float scale, int decode, int splits,
                                        float* scratch, int* err, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  B200_REQUIRE(b200_flash_attention_supported(q_heads, kv_heads, head_dim, page_size, decode),
               "paged_flash_attention: unsupported shape (heads %d/%d, head_dim %d, page %d)", q_heads,
               kv_heads, head_dim, page_size);
  B200_REQUIRE(num_seqs > 0 && num_seqs <= 65535 && splits >= 1 && max_q_len >= 1,
               "paged_flash_attention: bad batch");
  B200_REQUIRE(splits == 1 || (decode && (scratch != nullptr || splits <= 16)),
               "paged_flash_attention: more than 16 splits need scratch");
  FlashParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_arena = static_cast<const __nv_bfloat16*>(k_arena);
  p.v_arena = static_cast<const __nv_bfloat16*>(v_arena);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_q_start = seq_q_start;
  p.seq_q_len = seq_q_len;
  p.seq_kv_len = seq_kv_len;
  p.first_seq = first_seq;
  p.max_pages = max_pages;
  p.num_pages = num_pages;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = q_heads / kv_heads;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  p.page_shift = shift;
  p.page_mask = page_size - 1;
  p.window = window;
  p.splits = decode ? splits : 1;
  p.cluster_merge = (scratch == nullptr && p.splits > 1) ? 1 : 0;
  p.scale_log2 = scale * kLog2e;
  p.err = err;
  p.partial_out = scratch;
  p.partial_ml = scratch ? scratch + static_cast<int64_t>(tokens) * q_heads * p.splits * head_dim : nullptr;
  if (head_dim == 64) return launch_flash<64>(p, num_seqs, decode, max_q_len, tokens, stream);
  return launch_flash<128>(p, num_seqs, decode, max_q_len, tokens, stream);
}

// Shapes the TMA-fed decode kernel takes: head_dim 128, pages of at least 64 rows (a 64-key
// tile then lies inside one page), at most 16 query heads per kv head.
B200_API int b200_decode_attention_tma_supported(int q_heads, int kv_heads, int head_dim, int page_size) {
  if (head_dim != kTmaDim || q_heads % kv_heads || q_heads / kv_heads > 16) return 0;
  if (page_size < kTileKeys || (page_size & (page_size - 1))) return 0;
  if (kv_heads > 65535) return 0;
  return 1;
}

// Decode attention for requests [0, num_seqs) of the step, one new token each, with keys and
// values loaded by TMA into per-warp rings of `stages` pieces (2 to 6). With splits > 1 the
// partial results go through `scratch` (b200_flash_attention_scratch_floats) and the merge
// kernel, or, without scratch and with at most 16 splits, the splits form a thread-block
// cluster and merge on chip. The arenas must be 16-byte aligned and hold finite numbers in every row of a page
// that a block table names, written or not: whole 16-row pieces are loaded and the rows past
// a request's length are masked by weight zero, not skipped.
B200_API int b200_paged_decode_attention_tma(const void* q, const void* k_arena, const void* v_arena, void* out,
                                             const int* block_table, const int* seq_q_start, const int* seq_q_len,
                                             const int* seq_kv_len, int num_seqs, int max_pages, int num_pages,
                                             int q_heads, int kv_heads, int head_dim, int page_size, int window,
                                             float scale, int splits, int stages, float* scratch, int* err,
                                             cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  B200_REQUIRE(b200_decode_attention_tma_supported(q_heads, kv_heads, head_dim, page_size),
               "decode attention (TMA): unsupported shape (heads %d/%d, head_dim %d, page %d)", q_heads, kv_heads,
               head_dim, page_size);
  B200_REQUIRE(num_seqs > 0 && num_seqs <= 65535 && splits >= 1 && splits <= 65535, "decode attention (TMA): bad batch");
  B200_REQUIRE(stages >= 2 && stages <= kTmaMaxStages, "decode attention (TMA): 2 to %d stages, not %d", kTmaMaxStages, stages);
  B200_REQUIRE(splits == 1 || scratch != nullptr || splits <= kMaxClusterSplits,
               "decode attention (TMA): more than %d splits need scratch", kMaxClusterSplits);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(k_arena) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_arena) & 15) == 0,
               "decode attention (TMA): arenas must be 16-byte aligned");
  FlashParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_arena = static_cast<const __nv_bfloat16*>(k_arena);
  p.v_arena = static_cast<const __nv_bfloat16*>(v_arena);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_q_start = seq_q_start;
  p.seq_q_len = seq_q_len;
  p.seq_kv_len = seq_kv_len;
  p.first_seq = 0;
  p.max_pages = max_pages;
  p.num_pages = num_pages;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = q_heads / kv_heads;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  p.page_shift = shift;
  p.page_mask = page_size - 1;
  p.window = window;
  p.splits = splits;
  p.cluster_merge = (scratch == nullptr && splits > 1) ? 1 : 0;
  p.scale_log2 = scale * kLog2e;
  p.err = err;
  p.partial_out = scratch;
  p.partial_ml = scratch ? scratch + static_cast<int64_t>(num_seqs) * q_heads * splits * head_dim : nullptr;
  CUtensorMap k_map, v_map;
  const int64_t rows = static_cast<int64_t>(num_pages) * kv_heads * page_size;
  if (decode_arena_map(&k_map, k_arena, rows) != 0) return -1;
  if (decode_arena_map(&v_map, v_arena, rows) != 0) return -1;
  static bool configured = false;
  if (!configured) {
    const int most = static_cast<int>(decode_tma_smem_bytes(kTmaMaxStages));
    if (cudaFuncSetAttribute(paged_decode_tma_kernel<FINISH_WHOLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(paged_decode_tma_kernel<FINISH_PARTIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(paged_decode_tma_kernel<FINISH_CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess)
      return b200_fail("decode attention (TMA): cannot size shared memory");
    configured = true;
  }
  const dim3 grid(splits, kv_heads, num_seqs);
  cudaError_t status;
  if (p.cluster_merge) {
    // The splits of a (request, kv head) form one thread-block cluster and merge on chip.
    static bool wide_clusters = false;
    if (splits > 8 && !wide_clusters) {
      if (cudaFuncSetAttribute(paged_decode_tma_kernel<FINISH_CLUSTER>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return b200_fail("decode attention (TMA): clusters of %d blocks are not allowed here", splits);
      wide_clusters = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(kFlashThreads);
    config.dynamicSmemBytes = decode_tma_smem_bytes(stages);
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = b200_overlap_enabled() ? 2 : 1;
    status = cudaLaunchKernelEx(&config, paged_decode_tma_kernel<FINISH_CLUSTER>, k_map, v_map, p, stages);
  } else if (splits > 1) {
    status = launch_kernel(paged_decode_tma_kernel<FINISH_PARTIAL>, grid, dim3(kFlashThreads),
                           decode_tma_smem_bytes(stages), stream, k_map, v_map, p, stages);
  } else {
    status = launch_kernel(paged_decode_tma_kernel<FINISH_WHOLE>, grid, dim3(kFlashThreads),
                           decode_tma_smem_bytes(stages), stream, k_map, v_map, p, stages);
  }
  if (status != cudaSuccess) return b200_fail("decode attention (TMA): %s", cudaGetErrorString(status));
  if (splits > 1 && !p.cluster_merge) {
    status = launch_merge<kTmaDim>(p.partial_out, p.partial_ml, p.out, num_seqs * q_heads, splits, stream);
    if (status != cudaSuccess) return b200_fail("decode attention (TMA) merge: %s", cudaGetErrorString(status));
  }
  return b200_check_launch("paged_decode_attention_tma");
}
