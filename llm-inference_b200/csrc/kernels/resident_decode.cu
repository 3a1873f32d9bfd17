// A whole decode step of up to 16 requests as ONE resident kernel.
//
// A decode step of a small model is a chain of some 250 dependent kernels, each of which
// streams a few megabytes of weights and then waits: for its successor to be launched, for the
// first weights of that successor to arrive from HBM, for its own last block to drain. The
// bytes of such a step need half the time the chain takes. Here one block per SM stays
// resident for the whole step and walks a list of phases (embedding; per layer: q/k/v product,
// attention, output product, gate/up product, down product; last norm and output head), with
// a grid-wide barrier between phases. What makes this faster than the chain is that the
// weights never stop streaming: in every block one thread feeds a deep ring of shared-memory
// stages with TMA, in the fixed order of the whole step, and runs ahead of the phase the
// block computes by as much as the ring holds, so that while the blocks exchange activations
// at a barrier the next phase's weights are already arriving.
//
// A matrix product Y[T,N] = X[T,K] W[N,K]^T is cut into units of (128 rows of W, 64 of K) in
// row-major order, and every block takes an equal, contiguous run of units ("stream-K"): the
// load is balanced whatever N and K are. Per unit: TMA brings the 128 x 64 tile of W
// (128-byte swizzle), one thread issues tcgen05.mma (W as the 128-row operand, the padded 16
// tokens as the 16-column operand, fp32 accumulator in TMEM). The activations of the phase are
// built once per block in shared memory, in the tensor core's operand layout, by the
// block's worker warps right after the barrier: normalised residual rows (RMSNorm is folded in
// here: the sum of squares arrives as partial sums written by the product that produced the
// residual), SwiGLU outputs, or the merge of the attention splits. A run of units inside one
// row tile ends with the accumulator read back (tcgen05.ld); if the block holds all of the
// tile's K the result is final, otherwise it goes to scratch, and the block that arrives last
// at the tile's counter adds the parts in index order (so the sum does not depend on timing)
// and applies the epilogue: bias + rotary encoding + cache write (q/k/v), residual add plus
// partial sums of squares (o, down), SwiGLU (gate/up), or 32-bit logits (output head).
//
// Attention is the split-key decode scheme of attention_flash.cu: an item is (request, kv
// head, split), four warps each own a quarter of every 64-key tile and fetch it by TMA
// straight from the arena's pages; the splits' partial results are merged by the blocks of
// the output product when they build their operand.
//
// Formulas as everywhere in this library: python/instinct/backends/dense.py:80-134 (block
// order, residuals, SwiGLU), portable.py:115-149 (rotary encoding, RMSNorm), batches.py:110-113
// (causal and window mask), metal_kernels.py:103-124 (merging splits).
//
// Every wait (mbarrier, counter, grid barrier) is bounded. On a timeout the block records
// ERRBIT_TIMEOUT in the error word, which every other block polls in its own waits; from then
// on no wait blocks, all blocks run through the remaining control flow, free their TMEM and
// return. The kernel is launched cooperatively, so all blocks are resident at once and the
// barrier cannot wait for a block that has not started.
#include <cuda.h>

#include <cstring>
#include <vector>

#include "common.cuh"

namespace {

constexpr int kRows = 128;        // rows of W per unit = MMA M
constexpr int kBK = 64;           // K per unit: 128 bytes of bf16, one swizzle row
constexpr int kTok = 16;          // tokens padded to the MMA's N
constexpr int kStageBytes = kRows * kBK * 2;  // 16 KB
constexpr int kXTileBytes = kTok * kBK * 2;   // 2 KB
constexpr int kRegionBytes = 64 * 1024;       // X tiles | attention rings | attention merge area
constexpr int kMaxXTiles = kRegionBytes / kXTileBytes;  // 32
constexpr int kMaxStages = 9;
constexpr int kThreads = 256;     // warp 0: TMA, warp 1: MMA, warps 2-7: workers (2-5 also epilogue, 4-7 attention)
constexpr int kWorkers = 192;
constexpr int kEpiThreads = 128;
constexpr int kHeadDim = 128;
constexpr int kTileKeys = 64;
constexpr int kAttnStages = 2;
constexpr int kWarpStageBytes = 2 * 16 * kHeadDim * 2;  // a warp's 16 keys and 16 values of one tile: 8 KB
constexpr int kMaxSplits = 16;
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds
constexpr int ERRBIT_TIMEOUT = 8;
constexpr float kLog2e = 1.4426950408889634f;

enum : int { PH_EMBED = 0, PH_GEMM = 1, PH_ATTN = 2 };
enum : int { X_NORM = 0, X_ACT = 1, X_MERGE = 2 };
enum : int { E_QKV_ROPE = 0, E_RESIDUAL = 1, E_SWIGLU = 2, E_LOGITS = 3 };

struct alignas(128) Phase {
  CUtensorMap w_map;  // GEMM: W [N, K], boxes of 64 x 128
  CUtensorMap x_map;  // GEMM with X_NORM / X_ACT: the operand rows [16, K] in global memory, boxes of 64 x 16
  CUtensorMap k_map;  // ATTN: the layer's arenas as rows of 128, boxes of 64 x 16
  CUtensorMap v_map;
  int kind, xkind, ekind;
  int N, K;
  int window;
  int num_pages;
  float eps;
  const float* norm_weight;       // PH_EMBED, E_RESIDUAL: scale of the norm that follows (folded into xn)
  const float* bias;              // E_QKV_ROPE (may be null)
  __nv_bfloat16* k_arena;         // E_QKV_ROPE
  __nv_bfloat16* v_arena;
  const int* block_table;         // E_QKV_ROPE, ATTN: [T, max_pages] of the layer's cache group
  void* out;                      // E_SWIGLU: act; E_LOGITS: logits; PH_EMBED: the table (read)
};

struct StepParams {
  const Phase* phases;
  int num_phases;
  int T;            // requests = tokens of the step (padded ones included), at most 16
  int hidden;
  int q_heads, kv_heads;
  int page_size, page_shift, max_pages;
  int vocab;
  int splits;
  int stages;
  int table_dtype;  // embedding table: DTYPE_BF16
  float scale_log2;
  const float* inv_freq;  // [64]
  const int* token_ids;
  const int* positions;
  const int* seq_kv_len;
  float* x;         // residual stream [16, hidden] fp32
  __nv_bfloat16* xn;  // [16, hidden]: x times the scale of the norm that follows, the next product's operand
  float* ss;        // partial sums of squares [hidden / 32, 16]
  __nv_bfloat16* q_buf;  // [16, q_heads, 128]
  float* part_o;    // [16 * q_heads, splits, 128]
  float* part_ml;   // [16 * q_heads, splits, 2]
  float* scratch;   // [slots][16][128] partial accumulators
  int* counters;    // one per row tile, zero between phases
  unsigned int* bar;  // grid barrier counter, zero at launch
  int* err;
  // Optional, for profiling (null otherwise): [phases][4] timestamps in ns: block 0 enters the phase,
  // the last block has asked for its operand, the last block has finished, block 0 leaves the barrier.
  long long* trace;
};

__device__ __forceinline__ uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}

// The block's view of "something went wrong somewhere": its own flag and the timeout bit of
// the device's error word.
struct Abort {
  volatile int* local;
  int* err;
  __device__ __forceinline__ bool set() const { return *local != 0; }
  __device__ __forceinline__ bool poll() const {
    if (*local != 0) return true;
    if ((*reinterpret_cast<volatile int*>(err) & ERRBIT_TIMEOUT) != 0) {
      *local = 1;
      return true;
    }
    return false;
  }
  __device__ __forceinline__ void raise() const {
    *local = 1;
    atomicOr(err, ERRBIT_TIMEOUT);
  }
};

// Bounded wait for the phase with the given parity; false (at once, after the first failure
// anywhere) when the wait was given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Abort& abort) {
  if (abort.set()) return false;
  const uint32_t addr = saddr(bar);
  const long long start = clock64();
  uint32_t spins = 0;
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((++spins & 1023u) == 0) {
      if (abort.poll()) return false;
      if (clock64() - start > kWaitCycles) {
        abort.raise();
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(saddr(dst)), "l"(map), "r"(saddr(bar)), "r"(x), "r"(y)
      : "memory");
}

// K-major tile with 128-byte rows and 128-byte swizzle: groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}
// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = 16.
__device__ __forceinline__ uint32_t umma_instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTok >> 3) << 17) |
         (static_cast<uint32_t>(kRows >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
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
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` (0..15) in a warp's K or V piece:
// two boxes of 16 rows x 128 bytes, each swizzled as the TMA unit writes it.
__device__ __forceinline__ int box_offset(int row, int chunk) {
  return (chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// ---- how a product's units are dealt out --------------------------------------------------------

struct Deal {
  long long units;   // tiles * kbs
  long long groups;  // units / grain: what is dealt out
  int tiles, kbs;
  int grain;         // 1: any run of units (a row tile may be shared by blocks); kbs: whole row tiles only
  int blocks;
  __device__ __forceinline__ long long begin(int block) const { return groups * block / blocks * grain; }
  // The block whose run holds unit u: the largest b with begin(b) <= u.
  __device__ __forceinline__ int owner(long long u) const {
    return static_cast<int>(((u / grain + 1) * blocks + groups - 1) / groups) - 1;
  }
};

// Whole row tiles when that keeps at least 93 % of the blocks busy in every round (no partial sums
// through scratch then); otherwise equal runs of units.
__host__ __device__ __forceinline__ bool deal_whole_tiles(long long tiles, int blocks) {
  const long long rounds = (tiles + blocks - 1) / blocks;
  return tiles * 100 >= rounds * blocks * 93;
}

__device__ __forceinline__ Deal deal_of(const Phase& ph, int blocks) {
  Deal d;
  d.tiles = (ph.N + kRows - 1) / kRows;
  d.kbs = (ph.K + kBK - 1) / kBK;
  d.units = static_cast<long long>(d.tiles) * d.kbs;
  d.grain = deal_whole_tiles(d.tiles, blocks) ? d.kbs : 1;
  d.groups = d.units / d.grain;
  d.blocks = blocks;
  return d;
}

// ---- the grid-wide barrier -----------------------------------------------------------------------

// All worker threads of all blocks. `index` counts the barriers of this launch from 0.
__device__ __forceinline__ void grid_barrier(const StepParams& p, int index, const Abort& abort) {
  named_sync(1, kWorkers);
  if (threadIdx.x == 64) {
    __threadfence();
    atomicAdd(p.bar, 1u);
    const unsigned int target = static_cast<unsigned int>(index + 1) * gridDim.x;
    const long long start = clock64();
    uint32_t spins = 0;
    while (!abort.set()) {
      unsigned int seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.bar) : "memory");
      if (seen >= target) break;
      if ((++spins & 255u) == 0) {
        if (abort.poll()) break;
        if (clock64() - start > kWaitCycles) {
          abort.raise();
          break;
        }
      }
    }
    __threadfence();
  }
  named_sync(1, kWorkers);
}

// ---- phase bodies (worker warps) -----------------------------------------------------------------

// x[t, :] = table[token[t], :] widened to 32-bit, with partial sums of squares per 32 columns.
__device__ __forceinline__ void embed_phase(const StepParams& p, const Phase& ph) {
  const int warp = (threadIdx.x >> 5) - 2, lane = threadIdx.x & 31;
  const int col_tiles = p.hidden / kRows;
  const int items = p.T * col_tiles;
  const __nv_bfloat16* table = static_cast<const __nv_bfloat16*>(ph.out);
  for (int item = blockIdx.x * 6 + warp; item < items; item += gridDim.x * 6) {
    const int t = item / col_tiles, tile = item - t * col_tiles;
    const int token = p.token_ids[t];
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (token < 0 || token >= p.vocab) {
      if (lane == 0) atomicOr(p.err, ERRBIT_BAD_TOKEN);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(table + static_cast<int64_t>(token) * p.hidden + tile * kRows + lane * 4);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v[0] = __low2float(a);
      v[1] = __high2float(a);
      v[2] = __low2float(b);
      v[3] = __high2float(b);
    }
    *reinterpret_cast<float4*>(p.x + static_cast<int64_t>(t) * p.hidden + tile * kRows + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
    {
      const float4 w = *reinterpret_cast<const float4*>(ph.norm_weight + tile * kRows + lane * 4);
      uint2 scaled;
      scaled.x = pack_bf16(v[0] * w.x, v[1] * w.y);
      scaled.y = pack_bf16(v[2] * w.z, v[3] * w.w);
      *reinterpret_cast<uint2*>(p.xn + static_cast<int64_t>(t) * p.hidden + tile * kRows + lane * 4) = scaled;
    }
    float s = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if ((lane & 7) == 0) p.ss[(tile * 4 + (lane >> 3)) * kTok + t] = s;
  }
}

// Where 16-byte chunk c (8 elements of k) of token t goes inside an X tile.
__device__ __forceinline__ uint32_t x_chunk_offset(int t, int c) { return t * 128 + ((c ^ (t & 7)) << 4); }

// Builds X tiles for K blocks [kb_base, kb_base + count) of the output product: the merge of the
// attention splits, out = sum_i o_i 2^(m_i - M) / sum_i l_i 2^(m_i - M). All of a thread's loads
// of a round are requested before the first is used: the partial results come from L2.
__device__ __forceinline__ void build_x_merge(const StepParams& p, unsigned char* region, int kb_base, int count) {
  const int wt = threadIdx.x - 64;
  const int chunks = count * (kTok * 8);
  for (int i = wt; i < chunks; i += kWorkers) {
    const int slot = i >> 7, rem = i & 127;
    const int t = rem >> 3, c = rem & 7;
    const int k0 = (kb_base + slot) * kBK + c * 8;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (t < p.T && k0 < p.q_heads * kHeadDim) {
      const int head = k0 / kHeadDim, d0 = k0 - head * kHeadDim;
      const int64_t row = static_cast<int64_t>(t) * p.q_heads + head;
      const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + row * p.splits;
      float2 mls[kMaxSplits];
#pragma unroll
      for (int s = 0; s < kMaxSplits; ++s) mls[s] = s < p.splits ? __ldcg(ml + s) : make_float2(-INFINITY, 0.f);
      float m = -INFINITY;
#pragma unroll
      for (int s = 0; s < kMaxSplits; ++s) m = fmaxf(m, mls[s].x);
      const float use = m == -INFINITY ? 0.f : m;
      float l = 0.f;
      float f[kMaxSplits];
#pragma unroll
      for (int s = 0; s < kMaxSplits; ++s) {
        f[s] = exp2f(mls[s].x - use);  // 0 for splits that do not exist or saw no key
        l += mls[s].y * f[s];
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const float* o = p.part_o + row * p.splits * kHeadDim + d0;
#pragma unroll
      for (int s0 = 0; s0 < kMaxSplits; s0 += 8) {
        float4 a[8], b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool live = s0 + j < p.splits && f[s0 + j] != 0.f;
          a[j] = live ? __ldcg(reinterpret_cast<const float4*>(o + (s0 + j) * kHeadDim)) : make_float4(0.f, 0.f, 0.f, 0.f);
          b[j] = live ? __ldcg(reinterpret_cast<const float4*>(o + (s0 + j) * kHeadDim + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = f[s0 + j];
          acc[0] += a[j].x * w; acc[1] += a[j].y * w; acc[2] += a[j].z * w; acc[3] += a[j].w * w;
          acc[4] += b[j].x * w; acc[5] += b[j].y * w; acc[6] += b[j].z * w; acc[7] += b[j].w * w;
        }
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
      packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
      packed.z = pack_bf16(acc[4] * inv, acc[5] * inv);
      packed.w = pack_bf16(acc[6] * inv, acc[7] * inv);
    }
    *reinterpret_cast<uint4*>(region + slot * kXTileBytes + x_chunk_offset(t, c)) = packed;
  }
}

// The epilogue of one finished row tile: `v[t]` is output row n = tile * 128 + r for token t.
// Called by the 128 epilogue threads (r = their row); `stage` is [16][128] floats of shared memory.
__device__ __forceinline__ void apply_epilogue(const StepParams& p, const Phase& ph, int tile, int r, float (&v)[16],
                                               float* stage, const float* rstd) {
  const int lane = threadIdx.x & 31;
  const int n = tile * kRows + r;
  if (ph.xkind == X_NORM) {
    // The operand was x times the norm's scale; the token's 1 / rms commutes with the product.
#pragma unroll
    for (int t = 0; t < kTok; ++t) v[t] *= rstd[t];
  }
  if (ph.ekind == E_SWIGLU) {
    __nv_bfloat16* act = static_cast<__nv_bfloat16*>(ph.out);
    const int inter = ph.N / 2;
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      const float up = __shfl_down_sync(0xffffffffu, v[t], 1);
      if ((lane & 1) == 0 && t < p.T && n < ph.N)
        act[static_cast<int64_t>(t) * inter + n / 2] = __float2bfloat16_rn(v[t] / (1.f + expf(-v[t])) * up);
    }
  } else if (ph.ekind == E_RESIDUAL) {
    const int quarter = r >> 5;
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      float sq = 0.f;
      if (t < p.T && n < ph.N) {
        float* cell = p.x + static_cast<int64_t>(t) * ph.N + n;
        const float now = __ldcg(cell) + v[t];
        *cell = now;
        sq = now * now;
        p.xn[static_cast<int64_t>(t) * ph.N + n] = __float2bfloat16_rn(now * ph.norm_weight[n]);
      }
      sq = warp_sum(sq);
      if (lane == 0) p.ss[(tile * 4 + quarter) * kTok + t] = sq;
    }
  } else if (ph.ekind == E_LOGITS) {
    float* logits = static_cast<float*>(ph.out);
#pragma unroll
    for (int t = 0; t < kTok; ++t)
      if (t < p.T && n < ph.N) logits[static_cast<int64_t>(t) * ph.N + n] = v[t];
  } else {
    // q/k/v: the tile is one head. Bias, then through shared memory to pair dim i with i + 64.
    const float b = ph.bias != nullptr ? ph.bias[n] : 0.f;
#pragma unroll
    for (int t = 0; t < kTok; ++t) stage[t * kRows + r] = v[t] + b;
    named_sync(2, kEpiThreads);
    const int e = threadIdx.x - 64;  // 0..127
    const int head = tile;
    const bool is_q = head < p.q_heads, is_k = !is_q && head < p.q_heads + p.kv_heads;
    const int kv_head = is_k ? head - p.q_heads : head - p.q_heads - p.kv_heads;
    if (is_q || is_k) {
      const int i = e & 63, half = e >> 6;
      const float freq = p.inv_freq[i];
      for (int t = half * 8; t < half * 8 + 8 && t < p.T; ++t) {
        const int pos = p.positions[t];
        float sn, cs;
        sincosf(static_cast<float>(pos) * freq, &sn, &cs);
        const float x0 = stage[t * kRows + i], x1 = stage[t * kRows + i + 64];
        const float y0 = x0 * cs - x1 * sn, y1 = x1 * cs + x0 * sn;
        __nv_bfloat16* dst = nullptr;
        if (is_q) {
          dst = p.q_buf + (static_cast<int64_t>(t) * p.q_heads + head) * kHeadDim;
        } else {
          const int logical = pos >> p.page_shift;
          if (pos < 0 || logical >= p.max_pages) {
            if (i == 0) atomicOr(p.err, ERRBIT_BAD_POSITION);
          } else {
            const int page = ph.block_table[static_cast<int64_t>(t) * p.max_pages + logical];
            if (page < 0 || page >= ph.num_pages) {
              if (i == 0) atomicOr(p.err, ERRBIT_BAD_PAGE);
            } else {
              dst = ph.k_arena + kv_row_offset(page, kv_head, pos & (p.page_size - 1), p.kv_heads, p.page_size, kHeadDim);
            }
          }
        }
        if (dst != nullptr) {
          dst[i] = __float2bfloat16_rn(y0);
          dst[i + 64] = __float2bfloat16_rn(y1);
        }
      }
    } else {
      for (int t = 0; t < p.T; ++t) {
        const int pos = p.positions[t];
        const int logical = pos >> p.page_shift;
        if (pos < 0 || logical >= p.max_pages) {
          if (e == 0) atomicOr(p.err, ERRBIT_BAD_POSITION);
          continue;
        }
        const int page = ph.block_table[static_cast<int64_t>(t) * p.max_pages + logical];
        if (page < 0 || page >= ph.num_pages) {
          if (e == 0) atomicOr(p.err, ERRBIT_BAD_PAGE);
          continue;
        }
        ph.v_arena[kv_row_offset(page, kv_head, pos & (p.page_size - 1), p.kv_heads, p.page_size, kHeadDim) + e] =
            __float2bfloat16_rn(stage[t * kRows + e]);
      }
    }
    if (!is_q) {
      // The token that starts a page clears the page's other rows (see rope_kv.cu): leftovers of
      // the page's last owner must not meet a probability of zero in a PV product.
      __nv_bfloat16* arena = is_k ? ph.k_arena : ph.v_arena;
      for (int t = 0; t < p.T; ++t) {
        const int pos = p.positions[t];
        const int logical = pos >> p.page_shift;
        if (pos < 0 || (pos & (p.page_size - 1)) != 0 || logical >= p.max_pages) continue;
        const int page = ph.block_table[static_cast<int64_t>(t) * p.max_pages + logical];
        if (page < 0 || page >= ph.num_pages) continue;
        uint4* tail = reinterpret_cast<uint4*>(arena + kv_row_offset(page, kv_head, 1, p.kv_heads, p.page_size, kHeadDim));
        const int chunks = (p.page_size - 1) * (kHeadDim * 2 / 16);
        for (int c = e; c < chunks; c += kEpiThreads) tail[c] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    named_sync(2, kEpiThreads);  // the staging area is free again
  }
}

// One attention item: request t, kv head, split; the four attention warps (threads 128..255).
// `rings` is 4 x kAttnStages x 8 KB (1024-byte aligned); `uses` counts this warp's uses of each
// of its ring slots since the launch (it decides the mbarrier phase to wait for).
__device__ __forceinline__ void attention_item(const StepParams& p, const Phase& ph, int t, int kv_head, int split,
                                               unsigned char* rings, uint64_t* full, uint32_t (&uses)[kAttnStages],
                                               const Abort& abort) {
  constexpr int kKSteps = kHeadDim / 16;
  constexpr int kDimTiles = kHeadDim / 8;
  const int aw = (threadIdx.x >> 5) - 4, lane = threadIdx.x & 31;
  const int at = threadIdx.x - 128;  // 0..127
  const int group = p.q_heads / p.kv_heads;
  const int kv_len = p.seq_kv_len[t];
  const int first_pos = kv_len - 1;
  const int* table = ph.block_table + static_cast<int64_t>(t) * p.max_pages;
  const int lo = ph.window > 0 ? max(0, first_pos - ph.window + 1) : 0;
  const int hi = first_pos;
  int tile_begin = lo / kTileKeys, tile_end = hi / kTileKeys + 1;
  if (p.splits > 1) {
    const int tiles = tile_end - tile_begin;
    const int per_split = max(1, (tiles + p.splits - 1) / p.splits);
    tile_begin = tile_begin + split * per_split;
    tile_end = min(tile_end, tile_begin + per_split);
  }
  const int num_tiles = max(0, tile_end - tile_begin);
  const int key_off = tile_begin * kTileKeys + aw * 16;
  int mine_begin = 0, mine_end = num_tiles;
  while (mine_begin < mine_end && key_off + mine_begin * kTileKeys + 15 < lo) ++mine_begin;
  while (mine_end > mine_begin && key_off + (mine_end - 1) * kTileKeys > hi) --mine_end;
  const int mine = mine_end - mine_begin;

  unsigned char* my_ring = rings + aw * kAttnStages * kWarpStageBytes;
  uint64_t* my_full = full + aw * kAttnStages;
  auto request = [&](int j) {  // lane 0 only
    const int it = mine_begin + j;
    const int tile_start = (tile_begin + it) * kTileKeys;
    int page = __ldg(table + (tile_start >> p.page_shift));
    if (page < 0 || page >= ph.num_pages) {
      atomicOr(p.err, ERRBIT_BAD_PAGE);
      page = 0;
    }
    const int arena_row = (page * p.kv_heads + kv_head) * p.page_size + (tile_start & (p.page_size - 1)) + aw * 16;
    const int s = j % kAttnStages;
    unsigned char* dst = my_ring + s * kWarpStageBytes;
    mbar_expect_tx(&my_full[s], kWarpStageBytes);
    tma_load_2d(dst, &ph.k_map, &my_full[s], 0, arena_row);
    tma_load_2d(dst + 2048, &ph.k_map, &my_full[s], 64, arena_row);
    tma_load_2d(dst + 4096, &ph.v_map, &my_full[s], 0, arena_row);
    tma_load_2d(dst + 6144, &ph.v_map, &my_full[s], 64, arena_row);
  };
  int requested = 0;
  if (lane == 0) {
    // The newest keys were written with ordinary stores by other blocks before the barrier; the
    // TMA unit reads through another proxy.
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  while (requested < kAttnStages && requested < mine) {
    if (lane == 0) request(requested);
    ++requested;
  }

  const int r0 = lane >> 2, r1 = r0 + 8;
  const bool live0 = r0 < group, live1 = r1 < group;
  uint32_t qf[kKSteps][4];
  {
    const __nv_bfloat16* q0 = p.q_buf + (static_cast<int64_t>(t) * p.q_heads + kv_head * group + r0) * kHeadDim;
    const __nv_bfloat16* q1 = p.q_buf + (static_cast<int64_t>(t) * p.q_heads + kv_head * group + r1) * kHeadDim;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      qf[ks][0] = live0 ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + col)) : 0u;
      qf[ks][1] = live1 ? __ldcg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + col)) : 0u;
      qf[ks][2] = live0 ? __ldcg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + col)) : 0u;
      qf[ks][3] = live1 ? __ldcg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + col)) : 0u;
    }
  }
  float o[kDimTiles][4];
#pragma unroll
  for (int i = 0; i < kDimTiles; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int mi = lane >> 3;

  for (int j = 0; j < mine; ++j) {
    const int slot = j % kAttnStages;
    mbar_wait(&my_full[slot], uses[slot] & 1u, abort);
    ++uses[slot];
    const uint32_t k_base = saddr(my_ring + slot * kWarpStageBytes);
    const uint32_t v_base = k_base + kWarpStageBytes / 2;
    const int key_base = key_off + (mine_begin + j) * kTileKeys;
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

  // The four warps hold partial results for disjoint keys of the same <= 16 rows: merge them
  // through shared memory (the rings are no longer read) and write the split's partial result.
  named_sync(3, 128);
  float* merge_o = reinterpret_cast<float*>(rings);       // [4][16][128]
  float* merge_ml = merge_o + 4 * 16 * kHeadDim;          // [4][16][2]
  {
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < kDimTiles; ++i) {
      float* a = merge_o + (aw * 16 + r0) * kHeadDim + i * 8 + col;
      float* b = merge_o + (aw * 16 + r1) * kHeadDim + i * 8 + col;
      a[0] = o[i][0];
      a[1] = o[i][1];
      b[0] = o[i][2];
      b[1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      merge_ml[(aw * 16 + r0) * 2 + 0] = m0;
      merge_ml[(aw * 16 + r0) * 2 + 1] = l0;
      merge_ml[(aw * 16 + r1) * 2 + 0] = m1;
      merge_ml[(aw * 16 + r1) * 2 + 1] = l1;
    }
  }
  named_sync(3, 128);
  for (int item = at; item < group * kHeadDim; item += 128) {
    const int row = item / kHeadDim, d = item - row * kHeadDim;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * 16 + row) * 2]);
    const float use = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(merge_ml[(w * 16 + row) * 2] - use);
      l += merge_ml[(w * 16 + row) * 2 + 1] * f;
      acc += merge_o[(w * 16 + row) * kHeadDim + d] * f;
    }
    const int64_t out_row = static_cast<int64_t>(t) * p.q_heads + kv_head * group + row;
    p.part_o[(out_row * p.splits + split) * kHeadDim + d] = acc;
    if (d == 0) {
      p.part_ml[(out_row * p.splits + split) * 2 + 0] = m;
      p.part_ml[(out_row * p.splits + split) * 2 + 1] = l;
    }
  }
  // The merge area is the rings: the next item's copies must not land before everyone has read
  // it, and they come through the other proxy.
  named_sync(3, 128);
}

__global__ void __launch_bounds__(kThreads, 1) resident_decode_kernel(const StepParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = base;                                   // stages x 16 KB
  unsigned char* region = ring + p.stages * kStageBytes;        // 64 KB
  float* stage_f32 = reinterpret_cast<float*>(region + kRegionBytes);  // [16][128]
  __shared__ __align__(8) uint64_t w_full[kMaxStages], w_empty[kMaxStages];
  __shared__ __align__(8) uint64_t x_ready, acc_full[2], acc_empty[2];
  __shared__ __align__(8) uint64_t attn_full[4 * kAttnStages];
  __shared__ float rstd[kTok];
  __shared__ uint32_t tmem_base_shared;
  __shared__ int abort_flag;
  __shared__ int last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blocks = gridDim.x, block = blockIdx.x;
  const int stages = p.stages;
  Abort abort{&abort_flag, p.err};

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&w_full[s], 1);
      mbar_init(&w_empty[s], 1);
    }
    mbar_init(&x_ready, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    for (int i = 0; i < 4 * kAttnStages; ++i) mbar_init(&attn_full[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_shared)), "r"(32u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_shared;

  if (warp == 0) {
    // ---- weight producer: every unit of every product of the step, in order ----------------------
    if (lane == 0) {
      long long issued = 0;
      for (int i = 0; i < p.num_phases; ++i) {
        const Phase& ph = p.phases[i];
        if (ph.kind != PH_GEMM) continue;
        const Deal deal = deal_of(ph, blocks);
        const long long begin = deal.begin(block), end = deal.begin(block + 1);
        for (long long u = begin; u < end; ++u, ++issued) {
          const int s = static_cast<int>(issued % stages);
          if (issued >= stages) mbar_wait(&w_empty[s], static_cast<uint32_t>((issued / stages) - 1) & 1u, abort);
          if (abort.set()) break;
          const int tile = static_cast<int>(u / deal.kbs), kb = static_cast<int>(u - static_cast<long long>(tile) * deal.kbs);
          mbar_expect_tx(&w_full[s], kStageBytes);
          tma_load_2d(ring + s * kStageBytes, &ph.w_map, &w_full[s], kb * kBK, tile * kRows);
        }
        if (abort.set()) break;
      }
      if (abort.set()) {
        // Give copies still on their way time to land before the block's memory is given up.
        const long long start = clock64();
        while (clock64() - start < 4000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------------------
    uint32_t chosen;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    const bool leader = chosen != 0;
    const uint32_t idesc = umma_instr_desc();
    const uint64_t a_first = umma_smem_desc(saddr(ring));
    const uint64_t b_first = umma_smem_desc(saddr(region));
    long long consumed = 0;
    uint32_t acc_uses[2] = {0u, 0u};
    uint32_t x_uses = 0;  // products in which this block had units (the workers signal only those)
    int segment = 0;
    for (int i = 0; i < p.num_phases; ++i) {
      const Phase& ph = p.phases[i];
      if (ph.kind != PH_GEMM) continue;
      const Deal deal = deal_of(ph, blocks);
      const long long begin = deal.begin(block), end = deal.begin(block + 1);
      if (begin < end) {
        mbar_wait(&x_ready, x_uses & 1u, abort);
        ++x_uses;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int kb_base = (end - begin >= deal.kbs) ? 0 : static_cast<int>(begin % deal.kbs);
        long long u = begin;
        while (u < end) {
          const int kb0 = static_cast<int>(u % deal.kbs);
          const int count = static_cast<int>(min(end - u, static_cast<long long>(deal.kbs - kb0)));
          const int buf = segment & 1;
          if (acc_uses[buf] > 0) mbar_wait(&acc_empty[buf], (acc_uses[buf] - 1) & 1u, abort);
          ++acc_uses[buf];
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          for (int j = 0; j < count; ++j, ++consumed) {
            const int s = static_cast<int>(consumed % stages);
            mbar_wait(&w_full[s], static_cast<uint32_t>(consumed / stages) & 1u, abort);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // The X tile of this K block: slot (kb - kb_base), wrapping when the run crosses a row
            // tile's end with fewer than kbs units (then kb_base > 0 and slots wrap modulo kbs).
            int slot = kb0 + j - kb_base;
            if (slot < 0) slot += deal.kbs;
            const uint64_t a_desc = a_first + static_cast<uint64_t>(s) * (kStageBytes >> 4);
            const uint64_t b_desc = b_first + static_cast<uint64_t>(slot) * (kXTileBytes >> 4);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              if (leader) umma_bf16(tmem_base + buf * kTok, a_desc + k * 2, b_desc + k * 2, idesc, j > 0 || k > 0);
            if (leader) umma_commit(&w_empty[s]);
            __syncwarp();
          }
          if (leader) umma_commit(&acc_full[buf]);
          __syncwarp();
          ++segment;
          u += count;
        }
      }
    }
  } else {
    // ---- workers: X tiles, epilogues, attention, barriers ----------------------------------------
    const int wt = threadIdx.x - 64;
    const bool epi = warp < 6;  // warps 2..5 read the accumulator: TMEM lanes 32 * (warp % 4) ..
    const int quarter = warp & 3;
    uint32_t acc_uses[2] = {0u, 0u};
    uint32_t attn_uses[kAttnStages] = {0u, 0u};
    int segment = 0, barrier_index = 0;
    const bool tracing = p.trace != nullptr && block == 0 && wt == 0;
    const bool tracing_all = p.trace != nullptr && wt == 0;  // slowest block per phase: maxima over all blocks
    for (int i = 0; i < p.num_phases; ++i) {
      const Phase& ph = p.phases[i];
      if (tracing) p.trace[i * 4 + 0] = global_ns();
      if (ph.kind == PH_EMBED) {
        embed_phase(p, ph);
      } else if (ph.kind == PH_ATTN) {
        if (warp >= 4) {
          const int items = p.T * p.kv_heads * p.splits;
          for (int item = block; item < items; item += blocks) {
            const int t = item / (p.kv_heads * p.splits);
            const int rest = item - t * (p.kv_heads * p.splits);
            attention_item(p, ph, t, rest / p.splits, rest % p.splits, region, attn_full, attn_uses, abort);
          }
        }
      } else {
        const Deal deal = deal_of(ph, blocks);
        const long long begin = deal.begin(block), end = deal.begin(block + 1);
        if (begin < end) {
          // Which K blocks this block's run touches: all of them, or a range that may wrap
          // around a row tile's end (slot = (kb - kb_base) mod kbs).
          int kb_base = 0, count = deal.kbs;
          if (end - begin < deal.kbs) {
            kb_base = static_cast<int>(begin % deal.kbs);
            count = static_cast<int>(end - begin);
          }
          const int first = min(count, deal.kbs - kb_base);  // a wrapping range comes in two pieces
          if (ph.xkind == X_MERGE) {
            build_x_merge(p, region, kb_base, first);
            if (count > first) build_x_merge(p, region + first * kXTileBytes, 0, count - first);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            named_sync(1, kWorkers);
            if (wt == 32) mbar_arrive(&x_ready);
          } else {
            // The operand rows lie in global memory as bfloat16 (x times the norm's scale, or the
            // SwiGLU outputs): one thread asks the TMA unit for this block's K blocks. They were
            // written with ordinary stores by other blocks before the barrier.
            if (wt == 32) {
              asm volatile("fence.proxy.async;" ::: "memory");
              mbar_expect_tx(&x_ready, static_cast<uint32_t>(count) * kXTileBytes);
              for (int slot = 0; slot < count; ++slot) {
                const int kb = slot < first ? kb_base + slot : slot - first;
                tma_load_2d(region + slot * kXTileBytes, &ph.x_map, &x_ready, kb * kBK, 0);
              }
            }
            if (ph.xkind == X_NORM && wt < kTok) {
              // 1 / rms of each token from the partial sums of squares, added in index order.
              const int parts = ph.K / 32;
              float total = 0.f;
              for (int j0 = 0; j0 < parts; j0 += 8) {
                float part[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) part[j] = j0 + j < parts ? __ldcg(p.ss + (j0 + j) * kTok + wt) : 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) total += part[j];
              }
              rstd[wt] = rsqrtf(total / static_cast<float>(ph.K) + ph.eps);
            }
            named_sync(1, kWorkers);
          }
          if (tracing_all) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + i * 4 + 1), static_cast<unsigned long long>(global_ns()));
          if (epi) {
            long long u = begin;
            while (u < end) {
              const int tile = static_cast<int>(u / deal.kbs), kb0 = static_cast<int>(u % deal.kbs);
              const int n_units = static_cast<int>(min(end - u, static_cast<long long>(deal.kbs - kb0)));
              const int buf = segment & 1;
              mbar_wait(&acc_full[buf], acc_uses[buf] & 1u, abort);
              ++acc_uses[buf];
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              float v[16];
              tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kTok, v);
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[buf]);
              const int r = quarter * 32 + lane;
              bool finish = true;
              if (n_units < deal.kbs) {
                // Part of the tile's K: through scratch; whoever arrives last adds the parts.
                // The tile's parts are the runs of the blocks that own its units: consecutive blocks
                // when every block has units, else (fewer units than blocks) one block per unit.
                const long long tile_first = static_cast<long long>(tile) * deal.kbs;
                const bool dense = deal.units >= deal.blocks;
                const int first_owner = deal.owner(tile_first);
                const int parts = dense ? deal.owner(tile_first + deal.kbs - 1) - first_owner + 1 : deal.kbs;
                float* mine = p.scratch + static_cast<int64_t>(tile + block) * (kTok * kRows);
#pragma unroll
                for (int t = 0; t < kTok; ++t) mine[t * kRows + r] = v[t];
                __threadfence();
                named_sync(2, kEpiThreads);
                if (wt == 0) {
                  const int arrived = atomicAdd(p.counters + tile, 1);
                  last_flag = arrived == parts - 1;
                  if (last_flag) p.counters[tile] = 0;  // ready for the next phase
                }
                named_sync(2, kEpiThreads);
                finish = last_flag != 0;
                if (finish) {
                  __threadfence();
#pragma unroll
                  for (int t = 0; t < kTok; ++t) v[t] = 0.f;
                  // Four parts' values are requested before the first is added (they come from L2);
                  // the additions run in part order.
                  for (int part0 = 0; part0 < parts; part0 += 4) {
                    float theirs[4][kTok];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const int part = part0 + j;
                      const int owner = dense ? first_owner + part : deal.owner(tile_first + min(part, parts - 1));
                      const float* src = p.scratch + static_cast<int64_t>(tile + owner) * (kTok * kRows);
#pragma unroll
                      for (int t = 0; t < kTok; ++t) theirs[j][t] = part < parts ? __ldcg(src + t * kRows + r) : 0.f;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                      for (int t = 0; t < kTok; ++t) v[t] += theirs[j][t];
                  }
                }
                named_sync(2, kEpiThreads);  // last_flag may be rewritten by the next segment
              }
              if (finish) apply_epilogue(p, ph, tile, r, v, stage_f32, rstd);
              ++segment;
              u += n_units;
            }
          }
        }
      }
      if (p.trace != nullptr) {
        // Warp-uniform: a named barrier must not be reached from two sides of a branch inside a warp.
        named_sync(1, kWorkers);  // the whole block's work of the phase, attention included
        if (tracing_all)
          atomicMax(reinterpret_cast<unsigned long long*>(p.trace + i * 4 + 2), static_cast<unsigned long long>(global_ns()));
      }
      if (i + 1 < p.num_phases) grid_barrier(p, barrier_index++, abort);
      if (tracing) p.trace[i * 4 + 3] = global_ns();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
  }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(ptr);
  }
  return fn;
}

// A [rows, cols] bfloat16 row-major matrix cut into boxes of 64 columns x box_rows rows, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return b200_fail("resident_decode: the driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return b200_fail("resident_decode: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(status));
  return 0;
}

size_t smem_bytes(int stages) { return 1024 + static_cast<size_t>(stages) * kStageBytes + kRegionBytes + kTok * kRows * sizeof(float); }

}  // namespace

// ---- host interface ---------------------------------------------------------------------------------
//
// A plan is an array of phases in device memory, built once per model and cache (weights, norm
// scales, arenas and block-table addresses never move) and reused by every step.

constexpr int kPhaseFields = 18;

B200_API int b200_resident_phase_bytes() { return static_cast<int>(sizeof(Phase)); }
B200_API int b200_resident_phase_fields() { return kPhaseFields; }
B200_API int b200_resident_max_tokens() { return kTok; }

// Whether the kernel takes a model of these sizes (the caller keeps the chain of kernels otherwise).
// hidden and intermediate are K of some product: multiples of 64, and a block's run of units
// must fit the 32 X tiles of shared memory for every product (checked against `blocks`).
B200_API int b200_resident_supported(int hidden, int intermediate, int q_heads, int kv_heads, int head_dim, int vocab,
                                     int page_size, int blocks) {
  if (head_dim != kHeadDim || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || q_heads / kv_heads > 16) return 0;
  if (hidden % kRows || hidden < kRows || intermediate % kBK || intermediate < kBK) return 0;
  if (page_size < kTileKeys || (page_size & (page_size - 1))) return 0;
  if (vocab < 1 || blocks < 1) return 0;
  struct Shape { long long n, k; };
  const Shape shapes[] = {
      {static_cast<long long>(q_heads + 2 * kv_heads) * head_dim, hidden}, {hidden, static_cast<long long>(q_heads) * head_dim},
      {2LL * intermediate, hidden}, {hidden, intermediate}, {vocab, hidden}};
  for (const Shape& s : shapes) {
    const long long tiles = (s.n + kRows - 1) / kRows, kbs = (s.k + kBK - 1) / kBK;
    const long long most = (tiles * kbs + blocks - 1) / blocks + 1;  // units of the longest run
    const long long needed = deal_whole_tiles(tiles, blocks) ? kbs : (most < kbs ? most : kbs);
    if (needed > kMaxXTiles) return 0;
  }
  return 1;
}

// Fills `device_phases` (num_phases * b200_resident_phase_bytes() bytes of device memory) from
// `fields`, kPhaseFields 64-bit values per phase:
//   0 kind, 1 xkind, 2 ekind, 3 N, 4 K, 5 W, 6 norm weight, 7 eps (float bits), 8 bias, 9 k arena,
//   10 v arena, 11 block table, 12 arena rows (pages * kv_heads * page_size), 13 window, 14 out, 15 pages,
//   16 the product's operand rows [16, K] bfloat16 (xn or the SwiGLU outputs; 0 for the merge), 17 unused.
B200_API int b200_resident_build(const long long* fields, int num_phases, void* device_phases, cudaStream_t stream) {
  B200_REQUIRE(num_phases > 0 && fields != nullptr && device_phases != nullptr, "resident_decode: empty plan");
  std::vector<Phase> phases(num_phases);
  for (int i = 0; i < num_phases; ++i) {
    const long long* f = fields + static_cast<size_t>(i) * kPhaseFields;
    Phase& ph = phases[i];
    std::memset(&ph, 0, sizeof(Phase));
    ph.kind = static_cast<int>(f[0]);
    ph.xkind = static_cast<int>(f[1]);
    ph.ekind = static_cast<int>(f[2]);
    ph.N = static_cast<int>(f[3]);
    ph.K = static_cast<int>(f[4]);
    ph.norm_weight = reinterpret_cast<const float*>(f[6]);
    const uint32_t eps_bits = static_cast<uint32_t>(f[7]);
    std::memcpy(&ph.eps, &eps_bits, sizeof(float));
    ph.bias = reinterpret_cast<const float*>(f[8]);
    ph.k_arena = reinterpret_cast<__nv_bfloat16*>(f[9]);
    ph.v_arena = reinterpret_cast<__nv_bfloat16*>(f[10]);
    ph.block_table = reinterpret_cast<const int*>(f[11]);
    ph.window = static_cast<int>(f[13]);
    ph.out = reinterpret_cast<void*>(f[14]);
    ph.num_pages = static_cast<int>(f[15]);
    if (ph.kind == PH_GEMM) {
      B200_REQUIRE(ph.N > 0 && ph.K > 0 && ph.K % 8 == 0, "resident_decode: bad product %d x %d", ph.N, ph.K);
      B200_REQUIRE(f[5] != 0 && f[5] % 16 == 0, "resident_decode: weights must be 16-byte aligned");
      if (make_map(&ph.w_map, reinterpret_cast<const void*>(f[5]), ph.N, ph.K, kRows) != 0) return -1;
      if (ph.xkind != X_MERGE) {
        B200_REQUIRE(f[16] != 0 && f[16] % 16 == 0, "resident_decode: a product without its operand rows");
        if (make_map(&ph.x_map, reinterpret_cast<const void*>(f[16]), kTok, ph.K, kTok) != 0) return -1;
      }
    } else if (ph.kind == PH_ATTN) {
      B200_REQUIRE(f[9] != 0 && f[10] != 0 && f[12] > 0, "resident_decode: attention phase without arenas");
      if (make_map(&ph.k_map, reinterpret_cast<const void*>(f[9]), f[12], kHeadDim, 16) != 0) return -1;
      if (make_map(&ph.v_map, reinterpret_cast<const void*>(f[10]), f[12], kHeadDim, 16) != 0) return -1;
    } else {
      B200_REQUIRE(ph.kind == PH_EMBED, "resident_decode: unknown phase kind %d", ph.kind);
    }
  }
  const cudaError_t status =
      cudaMemcpyAsync(device_phases, phases.data(), sizeof(Phase) * num_phases, cudaMemcpyHostToDevice, stream);
  if (status != cudaSuccess) return b200_fail("resident_decode: copying the plan failed: %s", cudaGetErrorString(status));
  // The host vector goes away when this returns.
  if (cudaStreamSynchronize(stream) != cudaSuccess) return b200_fail("resident_decode: copying the plan failed");
  return 0;
}

// How many blocks a launch uses (one per SM) and the ring depth that fits beside them.
B200_API int b200_resident_blocks() { return b200_sm_count_host(); }

// Scratch the step needs: `floats` 32-bit words of partial accumulators (one slot per row tile
// and block), `counters` ints that must be zero before the first launch (each phase leaves them zero).
B200_API void b200_resident_scratch(int max_n, int blocks, long long* floats, int* counters) {
  const long long tiles = (static_cast<long long>(max_n) + kRows - 1) / kRows;
  *floats = (tiles + blocks) * kTok * kRows;
  *counters = static_cast<int>(tiles);
}

// One decode step. `bar` is one 32-bit word that this call zeroes on the stream first.
B200_API int b200_resident_decode(const void* device_phases, int num_phases, int tokens, int hidden, int q_heads,
                                  int kv_heads, int page_size, int max_pages, int vocab, int splits, float scale,
                                  const float* inv_freq, const int* token_ids, const int* positions,
                                  const int* seq_kv_len, float* x, void* xn, float* ss, void* q_buf, float* part_o, float* part_ml,
                                  float* scratch, int* counters, unsigned int* bar, int* err, long long* trace,
                                  cudaStream_t stream) {
  B200_REQUIRE(tokens >= 1 && tokens <= kTok, "resident_decode: %d tokens (at most %d)", tokens, kTok);
  B200_REQUIRE(splits >= 1 && splits <= kMaxSplits, "resident_decode: %d splits (at most %d)", splits, kMaxSplits);
  B200_REQUIRE(page_size >= kTileKeys && (page_size & (page_size - 1)) == 0, "resident_decode: page size %d", page_size);
  StepParams p;
  p.phases = static_cast<const Phase*>(device_phases);
  p.num_phases = num_phases;
  p.T = tokens;
  p.hidden = hidden;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.max_pages = max_pages;
  p.vocab = vocab;
  p.splits = splits;
  p.table_dtype = DTYPE_BF16;
  p.scale_log2 = scale * kLog2e;
  p.inv_freq = inv_freq;
  p.token_ids = token_ids;
  p.positions = positions;
  p.seq_kv_len = seq_kv_len;
  p.x = x;
  p.xn = static_cast<__nv_bfloat16*>(xn);
  p.ss = ss;
  p.q_buf = static_cast<__nv_bfloat16*>(q_buf);
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.scratch = scratch;
  p.counters = counters;
  p.bar = bar;
  p.err = err;
  p.trace = trace;
  p.stages = kMaxStages;
  while (p.stages > 2 && smem_bytes(p.stages) > 227 * 1024) --p.stages;
  const size_t smem = smem_bytes(p.stages);
  constexpr int kMaxDevices = 64;
  static bool configured[kMaxDevices] = {};
  int device = 0;
  B200_REQUIRE(cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < kMaxDevices, "resident_decode: no device");
  if (!configured[device]) {
    B200_REQUIRE(cudaFuncSetAttribute(resident_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem_bytes(kMaxStages))) == cudaSuccess,
                 "resident_decode: cannot size shared memory");
    configured[device] = true;
  }
  int per_sm = 0;
  B200_REQUIRE(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, resident_decode_kernel, kThreads, smem) == cudaSuccess &&
                   per_sm >= 1,
               "resident_decode: the kernel does not fit an SM");
  cudaError_t status = cudaMemsetAsync(bar, 0, sizeof(unsigned int), stream);
  if (status != cudaSuccess) return b200_fail("resident_decode: clearing the barrier failed: %s", cudaGetErrorString(status));
  void* args[] = {&p};
  status = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(resident_decode_kernel), dim3(b200_sm_count_host()),
                                       dim3(kThreads), args, smem, stream);
  if (status != cudaSuccess) return b200_fail("resident_decode: %s", cudaGetErrorString(status));
  return 0;
}
