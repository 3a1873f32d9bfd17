// Choosing the next token from 32-bit logits: a row is scanned by many blocks where it is long
// (the passes that read the whole vocabulary), and finished by one.
//
// Greedy rows take the arg-max, lowest index on ties (cuda/kernels.cu:327-348). Sampled rows
// follow python/instinct/sampling.py:47-101: candidates are the `kCandidates` largest logits;
// probabilities are softmax(logit / temperature) over the candidates; a candidate survives
// when its rank is below top_k, its probability is at least min_p times the largest, and
// the probability mass of strictly larger logits is below top_p; one survivor is drawn in
// proportion to its probability. Instead of sorting, thresholds are found by a radix search
// over the logits' bit patterns (counts for ranks, fixed-point mass for top_p), so equal
// logits are kept or dropped together. The draw uses a counter-based generator keyed per
// row, so a seeded request gets the same tokens whatever else is in the batch.
#include "common.cuh"

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kCandidates = 1024;

// Monotone map from float to unsigned: larger float <=> larger key.
__device__ __forceinline__ uint32_t float_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void __launch_bounds__(kSampleThreads)
argmax_rows_kernel(const float* logits, int vocab, int64_t row_stride,
                   const int* row_index, int* out) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  wait_for_predecessor();
  let_successor_start();
  const int src_row = row_index ? row_index[blockIdx.x] : blockIdx.x;
  const float* row = logits + src_row * row_stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  if (bi == 0x7fffffff) { bi = threadIdx.x < vocab ? threadIdx.x : 0; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    bv = lane < warps ? best_v[lane] : -INFINITY;
    bi = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[src_row] = bi;
  }
}

// The same over many blocks per row, for the few rows of a decode step (one block per row
// reads a 150k-entry row in 57 us; 37 blocks per row read eight rows in a few). Each block
// scans a slice and offers its best as one 64-bit key, value in the high half and the
// complement of the index in the low half, so that an atomic maximum keeps the largest value
// and among equals the smallest index, whatever the order of arrival. The block that arrives
// last at a row writes the token and leaves the row's key and counter cleared for the next launch.
constexpr int kArgmaxSliceThreads = 256;

__global__ void __launch_bounds__(kArgmaxSliceThreads)
argmax_slices_kernel(const float* logits, int vocab, int64_t row_stride, const int* row_index,
                     int* out, unsigned long long* best, int* arrived) {
  __shared__ unsigned long long block_best[kArgmaxSliceThreads / 32];
  wait_for_predecessor();
  let_successor_start();
  const int src_row = row_index ? row_index[blockIdx.y] : blockIdx.y;
  const float* row = logits + src_row * row_stride;
  const int slice = (vocab + gridDim.x - 1) / gridDim.x;
  const int begin = blockIdx.x * slice, end = min(vocab, begin + slice);
  unsigned long long key = 0;  // below every real key: float_key never yields 0 in the high half
  for (int i = begin + threadIdx.x; i < end; i += kArgmaxSliceThreads) {
    const unsigned long long k = (static_cast<unsigned long long>(float_key(row[i])) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
    key = k > key ? k : key;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) block_best[warp] = key;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxSliceThreads / 32; ++w) key = block_best[w] > key ? block_best[w] : key;
    atomicMax(&best[blockIdx.y], key);
    __threadfence();
    if (atomicAdd(&arrived[blockIdx.y], 1) == static_cast<int>(gridDim.x) - 1) {
      __threadfence();
      const unsigned long long winner = atomicExch(&best[blockIdx.y], 0ull);
      out[src_row] = static_cast<int>(0xffffffffu - static_cast<uint32_t>(winner & 0xffffffffull));
      arrived[blockIdx.y] = 0;
    }
  }
}

// The key of the k-th largest element (1-based), found byte by byte from the top.
__device__ uint32_t kth_largest_key(const float* row, int vocab, int k,
                                    unsigned int* hist /* [256] shared */) {
  uint32_t prefix = 0, mask = 0;
  int remaining = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t key = float_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    // Every thread walks the 256 bins the same way; cheap next to the scan above.
    int bin = 255;
    int above = 0;
    for (; bin > 0; --bin) {
      const int c = static_cast<int>(hist[bin]);
      if (above + c >= remaining) break;
      above += c;
    }
    remaining -= above;
    prefix |= static_cast<uint32_t>(bin) << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  return prefix;
}

// Key K such that keeping keys >= K keeps exactly the candidates whose strictly-larger mass
// is below `limit` (fixed-point). Only keys >= `floor_key` are candidates.
__device__ uint32_t top_p_key(const float* row, int vocab, float inv_temp,
                              float scaled_max, uint32_t floor_key, unsigned long long limit,
                              unsigned long long* mass /* [256] shared */) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long above_total = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) mass[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      const uint32_t key = float_key(v);
      if (key >= floor_key && (key & mask) == prefix) {
        const float p = expf(v * inv_temp - scaled_max);
        atomicAdd(&mass[(key >> shift) & 0xffu],
                  static_cast<unsigned long long>(p * 1099511627776.0f /* 2^40 */));
      }
    }
    __syncthreads();
    int bin = 255;
    unsigned long long above = above_total;
    for (; bin > 0; --bin) {
      const unsigned long long c = mass[bin];
      if (above + c >= limit) break;
      above += c;
    }
    above_total = above;
    prefix |= static_cast<uint32_t>(bin) << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  return prefix;
}

// One row, the whole vocabulary scanned by one block in every pass: what a row falls back to
// when the faster path below cannot hold its candidates, and the only path without scratch.
__device__ void sample_row_by_one_block(const float* logits, int vocab, int64_t row_stride,
                                        const float* temperature, const float* top_p,
                                        const float* min_p, const int* top_k,
                                        const unsigned long long* keys, const int* row_index,
                                        int* out, float* scratch /* [32] */, unsigned int* hist /* [256] */,
                                        unsigned long long* mass /* [256] */, float* partial /* [kSampleThreads] */,
                                        int* chosen_slot) {
  int& chosen = *chosen_slot;
  const int r = blockIdx.x;
  const int src_row = row_index ? row_index[r] : r;
  const float* row = logits + src_row * row_stride;
  const float temp = temperature[r];
  const float inv_temp = 1.f / temp;
  const int tid = threadIdx.x;

  float local_max = -INFINITY;
  for (int i = tid; i < vocab; i += blockDim.x) local_max = fmaxf(local_max, row[i]);
  const float max_logit = block_max(local_max, scratch);
  const float scaled_max = max_logit * inv_temp;

  // Candidates: the kCandidates largest logits.
  uint32_t keep_key = 0;
  if (vocab > kCandidates) keep_key = kth_largest_key(row, vocab, kCandidates, hist);
  const uint32_t candidate_key = keep_key;
  const int k = top_k[r];
  if (k > 0 && k < min(vocab, kCandidates)) {
    keep_key = max(keep_key, kth_largest_key(row, vocab, k, hist));
  }

  // Softmax denominator over the candidates.
  float local_sum = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (float_key(v) >= candidate_key) local_sum += expf(v * inv_temp - scaled_max);
  }
  const float denom = block_sum(local_sum, scratch);

  const float mp = min_p[r];
  if (mp > 0.f) {
    // p >= min_p * p_max  <=>  exp(logit / T - max / T) >= min_p; the survivors are the keys
    // at or above the smallest surviving logit's key.
    uint32_t local_key = 0xffffffffu;
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (expf(v * inv_temp - scaled_max) >= mp) local_key = min(local_key, float_key(v));
    }
    if (tid == 0) hist[0] = 0xffffffffu;
    __syncthreads();
    atomicMin(&hist[0], local_key);
    __syncthreads();
    keep_key = max(keep_key, hist[0]);
    __syncthreads();
  }
  const float tp = top_p[r];
  if (tp < 1.f) {
    const unsigned long long limit =
        static_cast<unsigned long long>(static_cast<double>(tp) * static_cast<double>(denom) *
                                        1099511627776.0);
    keep_key = max(keep_key, top_p_key(row, vocab, inv_temp, scaled_max, candidate_key, limit, mass));
  }

  // Draw among the survivors in index order: thread `tid` owns a contiguous slice.
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, tid * per), end = min(vocab, begin + per);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    const float v = row[i];
    if (float_key(v) >= keep_key) mine += expf(v * inv_temp - scaled_max);
  }
  partial[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    float total = 0.f;
    for (int i = 0; i < blockDim.x; ++i) total += partial[i];
    const uint64_t bits = splitmix64(keys[r]);
    const float u = static_cast<float>(bits >> 40) * (1.0f / 16777216.0f);
    const float target = u * total;
    // The owner is the first slice whose cumulative mass passes the target; rounding can
    // leave the target at the very top, in which case the last slice with survivors owns it.
    float running = 0.f, base = 0.f;
    int owner = -1;
    for (int i = 0; i < blockDim.x; ++i) {
      if (partial[i] > 0.f) {
        owner = i;
        base = running;
        if (running + partial[i] > target) break;
        running += partial[i];
      }
    }
    int pick = -1;
    if (owner >= 0) {
      const int b = min(vocab, owner * per), e = min(vocab, b + per);
      float acc = base;
      for (int i = b; i < e; ++i) {
        const float v = row[i];
        if (float_key(v) >= keep_key) {
          pick = i;
          acc += expf(v * inv_temp - scaled_max);
          if (acc > target) break;
        }
      }
    }
    chosen = pick;
  }
  __syncthreads();
  if (tid == 0) out[src_row] = chosen >= 0 ? chosen : 0;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* logits, int vocab, int64_t row_stride,
                   const float* temperature, const float* top_p,
                   const float* min_p, const int* top_k,
                   const unsigned long long* keys, const int* row_index,
                   int* out) {
  __shared__ float scratch[32];
  __shared__ unsigned int hist[256];
  __shared__ unsigned long long mass[256];
  __shared__ float partial[kSampleThreads];
  __shared__ int chosen;
  wait_for_predecessor();
  let_successor_start();
  sample_row_by_one_block(logits, vocab, row_stride, temperature, top_p, min_p, top_k, keys, row_index, out, scratch, hist,
                          mass, partial, &chosen);
}

// ---- the same with many blocks per row --------------------------------------------------------------
//
// One block needs 50 us to read a 150k-entry row once, and the filters above read it up to
// sixteen times. Here the row is read five times by many blocks each: four radix passes find
// the key of the kCandidates-th largest logit (counts in a per-row histogram in scratch; the
// block that arrives last at a row walks the bins), one pass collects the candidates, at most
// kListCap of them. Everything else works on that list in one block's shared memory, sorted
// by token index so that every sum has one order: ranks and the mass of strictly larger
// logits by comparing all pairs, the draw by a prefix sum. A row whose candidates do not fit
// the list (thousands of equal logits at the threshold) goes the long way above.
constexpr int kListCap = 2048;
constexpr int kSliceThreads = 256;

struct RowScratch {
  unsigned int hist[256];  // zero between launches
  unsigned int prefix, mask;
  int remaining;
  int arrived;   // zero between launches
  int cursor;    // zero between launches
  int overflow;  // zero between launches
  int pad[2];
  int list_index[kListCap];
  float list_value[kListCap];
};

__global__ void __launch_bounds__(kSliceThreads)
select_pass_kernel(const float* logits, int vocab, int64_t row_stride, const int* row_index,
                   RowScratch* rows, int shift) {
  __shared__ unsigned int local[256];
  wait_for_predecessor();
  let_successor_start();
  RowScratch& mine = rows[blockIdx.y];
  const int src_row = row_index ? row_index[blockIdx.y] : blockIdx.y;
  const float* row = logits + src_row * row_stride;
  const uint32_t prefix = shift == 24 ? 0u : mine.prefix, mask = shift == 24 ? 0u : mine.mask;
  for (int i = threadIdx.x; i < 256; i += kSliceThreads) local[i] = 0;
  __syncthreads();
  const int slice = (vocab + gridDim.x - 1) / gridDim.x;
  const int begin = blockIdx.x * slice, end = min(vocab, begin + slice);
  for (int i = begin + threadIdx.x; i < end; i += kSliceThreads) {
    const uint32_t key = float_key(row[i]);
    if ((key & mask) == prefix) atomicAdd(&local[(key >> shift) & 0xffu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 256; i += kSliceThreads)
    if (local[i]) atomicAdd(&mine.hist[i], local[i]);
  __threadfence();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = atomicAdd(&mine.arrived, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!last) return;
  // The block that arrived last: every thread fetches one bin (and clears it for the next
  // launch), one thread walks them.
  __threadfence();
  for (int i = threadIdx.x; i < 256; i += kSliceThreads) local[i] = atomicExch(&mine.hist[i], 0u);
  __syncthreads();
  if (threadIdx.x == 0) {
    const int remaining = shift == 24 ? kCandidates : mine.remaining;
    int bin = 255, above = 0;
    for (; bin > 0; --bin) {
      const int c = static_cast<int>(local[bin]);
      if (above + c >= remaining) break;
      above += c;
    }
    mine.remaining = remaining - above;
    mine.prefix = prefix | (static_cast<uint32_t>(bin) << shift);
    mine.mask = mask | (0xffu << shift);
    mine.arrived = 0;
  }
}

__global__ void __launch_bounds__(kSliceThreads)
collect_candidates_kernel(const float* logits, int vocab, int64_t row_stride,
                          const int* row_index, RowScratch* rows) {
  wait_for_predecessor();
  let_successor_start();
  RowScratch& mine = rows[blockIdx.y];
  const int src_row = row_index ? row_index[blockIdx.y] : blockIdx.y;
  const float* row = logits + src_row * row_stride;
  const uint32_t threshold = mine.prefix;
  const int slice = (vocab + gridDim.x - 1) / gridDim.x;
  const int begin = blockIdx.x * slice, end = min(vocab, begin + slice);
  // The block gathers its candidates in shared memory and reserves room in the row's list with
  // one atomic, not one per candidate.
  constexpr int kBlockCap = 1024;
  __shared__ int found_index[kBlockCap];
  __shared__ float found_value[kBlockCap];
  __shared__ int found, base;
  if (threadIdx.x == 0) found = 0;
  __syncthreads();
  for (int i = begin + threadIdx.x; i < end; i += kSliceThreads) {
    const float v = row[i];
    if (float_key(v) >= threshold) {
      const int slot = atomicAdd(&found, 1);
      if (slot < kBlockCap) {
        found_index[slot] = i;
        found_value[slot] = v;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    base = found > 0 ? atomicAdd(&mine.cursor, found) : 0;
    if (found > kBlockCap || base + found > kListCap) mine.overflow = 1;
  }
  __syncthreads();
  const int count = min(found, kBlockCap);
  for (int i = threadIdx.x; i < count; i += kSliceThreads) {
    if (base + i < kListCap) {
      mine.list_index[base + i] = found_index[i];
      mine.list_value[base + i] = found_value[i];
    }
  }
}

// Inclusive prefix sums of value[0..n) (n <= 2 * blockDim.x) in place, in a fixed order.
__device__ void block_prefix_sums(float* value, int n, float* warp_totals /* [32] */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int a = 2 * tid, b = a + 1;
  const float x = a < n ? value[a] : 0.f, y = b < n ? value[b] : 0.f;
  float sum = x + y;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, sum, o);
    if (lane >= o) sum += up;
  }
  if (lane == 31) warp_totals[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? warp_totals[lane] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, t, o);
      if (lane >= o) t += up;
    }
    warp_totals[lane] = t;
  }
  __syncthreads();
  const float before = (warp > 0 ? warp_totals[warp - 1] : 0.f) + (sum - x - y);
  if (a < n) value[a] = before + x;
  if (b < n) value[b] = before + x + y;
  __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads)
sample_from_candidates_kernel(const float* logits, int vocab, int64_t row_stride,
                              const float* temperature, const float* top_p,
                              const float* min_p, const int* top_k,
                              const unsigned long long* keys, const int* row_index,
                              int* out, RowScratch* rows, int direct) {
  // The fallback's shared memory and the list's are never live together.
  __shared__ float scratch[32];
  __shared__ unsigned int hist[256];
  __shared__ unsigned long long mass[256];
  __shared__ int chosen;
  __shared__ int index[kListCap];
  __shared__ __align__(16) float value[kListCap];   // logit, then exp, then the survivors' prefix sums
  __shared__ __align__(16) uint32_t sort_key[kListCap];
  __shared__ unsigned long long by_key[kListCap];  // (~key, position): the list by logit, largest first
  wait_for_predecessor();
  let_successor_start();
  const int r = blockIdx.x, tid = threadIdx.x;
  RowScratch& mine = rows[r];
  const int src_row = row_index ? row_index[r] : r;
  const float* row = logits + src_row * row_stride;
  int n;
  if (direct) {
    n = vocab;  // the whole row is the list, already in token order
  } else {
    const int found = mine.cursor, overflow = mine.overflow;
    __syncthreads();
    if (tid == 0) {
      mine.cursor = 0;
      mine.overflow = 0;
    }
    if (overflow || found > kListCap) {
      float* partial = value;  // kSampleThreads <= kListCap floats
      sample_row_by_one_block(logits, vocab, row_stride, temperature, top_p, min_p, top_k, keys, row_index, out, scratch,
                              hist, mass, partial, &chosen);
      return;
    }
    n = found;
  }
  // The list in shared memory, in token order (collected in arrival order: a bitonic sort by index).
  int padded = 1;
  while (padded < n) padded <<= 1;
  for (int i = tid; i < padded; i += kSampleThreads) {
    if (i < n) {
      index[i] = direct ? i : mine.list_index[i];
      value[i] = direct ? row[i] : mine.list_value[i];
    } else {
      index[i] = 0x7fffffff;
      value[i] = -INFINITY;
    }
  }
  __syncthreads();
  if (!direct) {
    for (int k = 2; k <= padded; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < padded; i += kSampleThreads) {
          const int partner = i ^ j;
          if (partner > i) {
            const bool ascending = (i & k) == 0;
            const int a = index[i], b = index[partner];
            if ((a > b) == ascending) {
              index[i] = b;
              index[partner] = a;
              const float t = value[i];
              value[i] = value[partner];
              value[partner] = t;
            }
          }
        }
        __syncthreads();
      }
    }
  }
  const float temp = temperature[r];
  const float inv_temp = 1.f / temp;
  float local_max = -INFINITY;
  for (int i = tid; i < n; i += kSampleThreads) {
    sort_key[i] = float_key(value[i]);
    local_max = fmaxf(local_max, value[i]);
  }
  const float scaled_max = block_max(local_max, scratch) * inv_temp;
  __syncthreads();
  // Candidates (direct lists only: a collected list holds nothing else): fewer than
  // kCandidates strictly larger logits. Everything below is over candidates.
  const bool rank_candidates = direct && n > kCandidates;
  const int k = top_k[r];
  const bool rank_top_k = k > 0 && k < min(vocab, kCandidates);
  const float mp = min_p[r], tp = top_p[r];
  if (!rank_candidates && !rank_top_k && tp >= 1.f) {
    // No filter that needs ranks: every entry is a candidate, min_p is a test per entry.
    for (int i = tid; i < n; i += kSampleThreads) {
      const float w = expf(value[i] * inv_temp - scaled_max);
      value[i] = (mp > 0.f && w < mp) ? 0.f : w;
    }
    __syncthreads();
  } else {
    // Ranks and the mass of strictly larger logits come from a second order of the list: by
    // logit, largest first, equal logits by position. An entry's number of strictly larger
    // logits is where its run of equal logits begins, and their mass the prefix sum up to there.
    for (int i = tid; i < padded; i += kSampleThreads)
      by_key[i] = i < n ? (static_cast<unsigned long long>(~sort_key[i]) << 32) | static_cast<unsigned long long>(i)
                        : 0xffffffffffffffffull;
    __syncthreads();
    for (int kk = 2; kk <= padded; kk <<= 1) {
      for (int j = kk >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < padded; i += kSampleThreads) {
          const int partner = i ^ j;
          if (partner > i) {
            const bool ascending = (i & kk) == 0;
            const unsigned long long x = by_key[i], y = by_key[partner];
            if ((x > y) == ascending) {
              by_key[i] = y;
              by_key[partner] = x;
            }
          }
        }
        __syncthreads();
      }
    }
    float* weight_by_rank = reinterpret_cast<float*>(sort_key);  // the keys live on in by_key
    int start[2], position[2];
    bool candidate[2];
    float weight[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int at = tid + e * kSampleThreads;
      start[e] = position[e] = 0;
      candidate[e] = false;
      weight[e] = 0.f;
      if (at < n) {
        const unsigned long long mine_key = by_key[at];
        position[e] = static_cast<int>(mine_key & 0xffffffffull);
        // Where the run of this logit begins: the first entry whose high half is not smaller.
        const unsigned long long floor_key = mine_key & 0xffffffff00000000ull;
        int lo = 0, hi = at;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (by_key[mid] < floor_key) lo = mid + 1;
          else hi = mid;
        }
        start[e] = lo;
        candidate[e] = !rank_candidates || lo < kCandidates;
        weight[e] = candidate[e] ? expf(value[position[e]] * inv_temp - scaled_max) : 0.f;
      }
    }
    __syncthreads();  // the logits in `value` and the keys in `sort_key` have been read
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int at = tid + e * kSampleThreads;
      if (at < n) {
        weight_by_rank[at] = weight[e];
        value[at] = weight[e];  // becomes the prefix sums in rank order
      }
    }
    __syncthreads();
    float denom = 0.f;
    if (tp < 1.f) {
      float local = 0.f;
      for (int i = tid; i < n; i += kSampleThreads) local += weight_by_rank[i];
      denom = block_sum(local, scratch);
      block_prefix_sums(value, n, scratch);
    }
    bool keep[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      keep[e] = candidate[e];
      if (rank_top_k && start[e] >= k) keep[e] = false;
      if (mp > 0.f && weight[e] < mp) keep[e] = false;
      if (tp < 1.f && keep[e]) {
        const float heavier = start[e] > 0 ? value[start[e] - 1] : 0.f;
        if (!(heavier < tp * denom)) keep[e] = false;
      }
    }
    __syncthreads();  // the prefix sums have been read: `value` goes back to token order
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int at = tid + e * kSampleThreads;
      if (at < n) value[position[e]] = keep[e] ? weight[e] : 0.f;
    }
    __syncthreads();
  }
  // The draw: inverse CDF over the survivors in token order.
  block_prefix_sums(value, n, scratch);
  if (tid == 0) chosen = 0x7fffffff;
  __syncthreads();
  const float total = value[n - 1];
  const uint64_t bits = splitmix64(keys[r]);
  const float u = static_cast<float>(bits >> 40) * (1.0f / 16777216.0f);
  const float target = u * total;
  int first = 0x7fffffff, last = -1;
  for (int i = tid; i < n; i += kSampleThreads) {
    const float before = i > 0 ? value[i - 1] : 0.f;
    if (value[i] > before) {  // a survivor
      last = max(last, i);
      if (value[i] > target) first = min(first, i);
    }
  }
  atomicMin(&chosen, first);
  __syncthreads();
  if (chosen == 0x7fffffff) {
    // Rounding left the target at the very top: the last survivor owns it.
    __syncthreads();
    if (tid == 0) chosen = -1;
    __syncthreads();
    atomicMax(&chosen, last);
    __syncthreads();
  }
  if (tid == 0) out[src_row] = chosen >= 0 && chosen < n ? index[chosen] : 0;
}

}  // namespace

// `best` (rows 64-bit words) and `arrived` (rows ints), both zero before the first launch and
// left zero by every launch, let few rows be scanned by many blocks each; without them (null)
// one block scans a row.
B200_API int b200_argmax_rows(const float* logits, int rows, int vocab, int64_t row_stride,
                              const int* row_index, int* out, unsigned long long* best, int* arrived,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && vocab > 0 && row_stride >= vocab, "argmax_rows: bad sizes");
  if (best != nullptr && arrived != nullptr && rows < b200_sm_count_host() && vocab >= 4096) {
    int slices = (2 * b200_sm_count_host() + rows - 1) / rows;
    slices = slices > 64 ? 64 : slices;
    launch_kernel(argmax_slices_kernel, dim3(slices, rows), dim3(kArgmaxSliceThreads), 0, stream, logits, vocab,
                  row_stride, row_index, out, best, arrived);
    return b200_check_launch("argmax_rows");
  }
  launch_kernel(argmax_rows_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, logits, vocab, row_stride,
                row_index, out);
  return b200_check_launch("argmax_rows");
}

// Row r of the call reads logits row `row_index[r]` (or r when row_index is null) and writes
// the token to out[that row], so greedy and sampled rows of one batch can share `out`.
// `keys[r]` seeds the row's single uniform draw.
// Bytes of scratch b200_sample_rows wants for `rows` rows: zero before the first launch, left
// in that state by every launch.
B200_API long long b200_sample_scratch_bytes(int rows) { return static_cast<long long>(rows) * sizeof(RowScratch); }

// `scratch` (may be null: then one block scans a row in every pass) lets large vocabularies be
// scanned by many blocks per row.
B200_API int b200_sample_rows(const float* logits, int rows, int vocab, int64_t row_stride,
                              const float* temperature, const float* top_p, const float* min_p,
                              const int* top_k, const unsigned long long* keys,
                              const int* row_index, int* out, void* scratch, long long scratch_bytes,
                              cudaStream_t stream) {
  if (rows == 0) return 0;
  B200_REQUIRE(rows > 0 && vocab > 0 && row_stride >= vocab, "sample_rows: bad sizes");
  if (scratch != nullptr) {
    B200_REQUIRE(scratch_bytes >= b200_sample_scratch_bytes(rows), "sample_rows: scratch too small");
    RowScratch* state = static_cast<RowScratch*>(scratch);
    if (vocab > kListCap) {
      int slices = (2 * b200_sm_count_host() + rows - 1) / rows;
      slices = slices > 64 ? 64 : slices;
      const dim3 grid(slices, rows);
      for (int shift = 24; shift >= 0; shift -= 8)
        launch_kernel(select_pass_kernel, grid, dim3(kSliceThreads), 0, stream, logits, vocab, row_stride, row_index, state,
                      shift);
      launch_kernel(collect_candidates_kernel, grid, dim3(kSliceThreads), 0, stream, logits, vocab, row_stride, row_index,
                    state);
    }
    launch_kernel(sample_from_candidates_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, logits, vocab, row_stride,
                  temperature, top_p, min_p, top_k, keys, row_index, out, state, vocab > kListCap ? 0 : 1);
    return b200_check_launch("sample_rows");
  }
  launch_kernel(sample_rows_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, logits, vocab, row_stride,
                temperature, top_p, min_p, top_k, keys, row_index, out);
  return b200_check_launch("sample_rows");
}
