// Paged causal attention for prompt portions on the 5th-generation tensor cores (head_dim 128).
//
// One block owns up to 128 query rows of one (request, kv head) pair - every (new token, query
// head of the group) combination, as in attention_flash.cu - and walks the request's keys 128
// at a time:
//   S = Q K^T      tcgen05.mma, both operands in shared memory (128-byte swizzle), S in TMEM
//   P = softmax    two groups of four warps, one thread per row, the groups taking the key
//                  tiles in turn: tcgen05.ld S, running max / sum in 32-bit
//                  (python/instinct/backends/portable.py:173-188), P back to TMEM as bfloat16
//   O += P V       tcgen05.mma with P read from TMEM and V from shared memory, O in TMEM
// Keys and values come straight from the arena's pages: one thread walks the block table and
// issues TMA tile loads (cp.async.bulk.tensor) of whole page pieces into rings (three key tiles,
// two value tiles, each with a loader thread of its own, so that a tile is on its way long
// before its product is issued), and no thread computes addresses row by row. Three S buffers
// let the tensor core run two tiles ahead of each softmax group. Masking follows
// python/instinct/batches.py:110-113: key <= query position and, with a window,
// key > position - window.
//
// Every wait (mbarriers, and the shared-memory word the two softmax threads of a row pass the
// turn with) is bounded; on a timeout the block records ERRBIT_TIMEOUT, skips its further waits,
// runs out and frees its TMEM. Shapes the kernel does not take (other head sizes, pages under 16 rows,
// block tables beyond kMaxChunks page pieces) go to attention_flash.cu.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int kDim = 128;        // head_dim
constexpr int kRows = 128;       // query rows per block (MMA M)
constexpr int kKeys = 128;       // keys per tile (MMA N of S, K of PV)
constexpr int kStagesK = 3;      // key tiles in flight: a slot is free once its S product retired
constexpr int kStagesV = 2;      // value tiles in flight: a slot is free once its PV product retired
constexpr int kThreadsA = 352;   // warp 0: K loads, warp 1: MMA, warps 2-5 and 6-9: softmax, warp 10: V loads
constexpr int kSoftmaxThreads = 256;
constexpr int kScoreBuffers = 3;  // S tiles in TMEM (3 x 128 columns, plus 128 for O: all 512)
constexpr int kHalfBytes = kKeys * 128;  // one 64-column half of a 128-row tile: 16 KB
constexpr int kTileBytesA = 2 * kHalfBytes;
constexpr int kMaxChunks = 1024;  // page pieces a block may walk (block-table entries cached in smem)
constexpr long long kWaitCyclesA = 4000000000LL;  // about two seconds
constexpr int ERRBIT_TIMEOUT_A = 8;
constexpr float kLog2eA = 1.4426950408889634f;

struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* block_table;
  const int* seq_q_start;
  const int* seq_q_len;
  const int* seq_kv_len;
  int* err;
  int first_seq;
  int max_pages, num_pages;
  int q_heads, kv_heads, group;
  int page_size, page_shift;
  int piece_rows;  // rows per TMA box: min(page_size, 128)
  int window;
  float scale_log2;
};

__device__ __forceinline__ uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = saddr(bar);
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - start > kWaitCyclesA) return false;
  }
}
__device__ __forceinline__ void tma_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(saddr(dst)), "l"(map), "r"(saddr(bar)), "r"(x), "r"(y)
      : "memory");
}

// K-major operand, 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
// MN-major operand (V: head dims contiguous, keys along K): 64-dim halves kHalfBytes apart
// (leading offset), 8-key groups 1024 bytes apart (stride offset), 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(kHalfBytes >> 4) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
// bf16 x bf16 -> fp32, M = 128, N = 128; `b_mn_major` for the PV product.
__device__ __forceinline__ uint32_t idesc(bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(kKeys >> 3) << 17) |
         (static_cast<uint32_t>(kRows >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t id, bool acc) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d),
               "l"(a), "l"(b), "r"(id), "r"(acc ? 1u : 0u)
               : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t id, bool acc) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d),
               "r"(a_tmem), "l"(b), "r"(id), "r"(acc ? 1u : 0u)
               : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
      "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
      "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 2^x on the special-function unit; 2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
  return chosen != 0;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreadsA, 1)
flash_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             const PrefillParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_tile = base;                                   // 32 KB: two halves of [128 rows][64 dims]
  unsigned char* k_ring = q_tile + kTileBytesA;                   // kStagesK x 32 KB
  unsigned char* v_ring = k_ring + kStagesK * kTileBytesA;        // kStagesV x 32 KB
  int* pages = reinterpret_cast<int*>(v_ring + kStagesV * kTileBytesA);  // [kMaxChunks]
  __shared__ __align__(8) uint64_t k_full[kStagesK], k_empty[kStagesK], v_full[kStagesV], v_empty[kStagesV];
  // o_done[t & 3] completes when PV[t] has retired (and with it every earlier product). A ring of
  // four, because its waiters are not in step with it: a phase bit tells "done" from "not yet"
  // only while the barrier is less than two phases from the one asked for, and every softmax
  // thread checks PV[t - 2] at each of its tiles, which keeps all its questions within that.
  __shared__ __align__(8) uint64_t s_full[kScoreBuffers], p_ready[kScoreBuffers], o_done[4];
  // What a row's two softmax threads (one per group) tell each other: the exponent offset after
  // the last tile decided, which tile is next to decide, and at the end their sums.
  __shared__ float row_m[kRows], row_l[2][kRows];
  __shared__ int row_next[kRows];
  __shared__ uint32_t tmem_base_shared;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.first_seq + blockIdx.z;
  const int kv_head = blockIdx.y;
  const int q_len = p.seq_q_len[seq];
  const int kv_len = p.seq_kv_len[seq];
  const int q_start = p.seq_q_start[seq];
  const int first_pos = kv_len - q_len;
  const int rows_total = q_len * p.group;
  // Later rows attend to more keys: they go first, so the longest blocks do not form the tail.
  const int row_base = static_cast<int>(gridDim.x - 1 - blockIdx.x) * kRows;
  // A block with nothing to do still waits for the kernel in front before it ends: the kernel
  // behind may pass its own wait once every block of this grid has ended, and must not do so
  // while this kernel's predecessor still runs.
  if (row_base >= rows_total) {
    wait_for_predecessor();
    let_successor_start();
    return;
  }
  const int* table = p.block_table + static_cast<int64_t>(seq) * p.max_pages;

  const int first_token = row_base / p.group;
  const int last_token = min(q_len - 1, (row_base + kRows - 1) / p.group);
  const int lo = p.window > 0 ? max(0, first_pos + first_token - p.window + 1) : 0;
  const int hi = first_pos + last_token;  // inclusive
  const int tile_begin = lo / kKeys, tile_end = hi / kKeys + 1;
  const int num_tiles = tile_end - tile_begin;
  const int pieces_per_tile = kKeys / p.piece_rows;
  if (num_tiles * pieces_per_tile > kMaxChunks) {
    // The launcher sized the walk from the host's lengths; lengths on the device that exceed
    // them are an error of the caller, reported rather than walked.
    wait_for_predecessor();
    let_successor_start();
    if (threadIdx.x == 0) atomicOr(p.err, ERRBIT_BAD_POSITION);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesK; ++s) {
      bar_init(&k_full[s], 1);
      bar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < kStagesV; ++s) {
      bar_init(&v_full[s], 1);
      bar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < kScoreBuffers; ++i) {
      bar_init(&s_full[i], 1);
      bar_init(&p_ready[i], 128);
    }
    for (int i = 0; i < 4; ++i) bar_init(&o_done[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_shared)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Block-table entries of every page piece this block walks: like the lengths above they are
  // part of the step's metadata, on the device before any kernel of the step ran, so all of
  // this may precede the wait for the kernel in front (which wrote the queries and the newest
  // keys).
  for (int i = threadIdx.x; i < num_tiles * pieces_per_tile; i += kThreadsA) {
    const int key = tile_begin * kKeys + i * p.piece_rows;
    // Pieces past the request's last key are read too (the table pads them with a page that
    // exists): their scores are masked, and their values only ever meet a probability of zero.
    pages[i] = (key >> p.page_shift) < p.max_pages ? table[key >> p.page_shift] : -1;
  }
  for (int i = threadIdx.x; i < kRows; i += kThreadsA) {
    row_m[i] = -INFINITY;
    row_next[i] = 0;
  }
  wait_for_predecessor();
  let_successor_start();
  if (p.window > 0 || tile_end * kKeys > p.max_pages * p.page_size) {
    // Pieces whose page the request no longer holds, or that lie past the block table, are
    // skipped by the loader; their rows must still hold finite numbers, since a masked
    // probability of zero times garbage may be NaN.
    for (int i = threadIdx.x; i < (kStagesK + kStagesV) * kTileBytesA / 16; i += kThreadsA)
      reinterpret_cast<uint4*>(k_ring)[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  // The loaders go ahead; the other nine warps bring the query tile in meanwhile (swizzled by
  // hand: chunk c of row r goes to chunk c ^ (r & 7) of its 128-byte row) and meet the issuing
  // warp at a barrier of their own.
  constexpr int kFillThreads = 9 * 32;
  if (warp >= 1 && warp <= 9) {
    for (int i = threadIdx.x - 32; i < kRows * 16; i += kFillThreads) {
      const int r = i >> 4, c = i & 15;
      const int row = row_base + r;
      uint4 value = make_uint4(0u, 0u, 0u, 0u);
      if (row < rows_total) {
        const int tok = row / p.group;
        const int head = kv_head * p.group + (row - tok * p.group);
        value = *reinterpret_cast<const uint4*>(p.q + (static_cast<int64_t>(q_start + tok) * p.q_heads + head) * kDim + c * 8);
      }
      *reinterpret_cast<uint4*>(q_tile + (c >> 3) * kHalfBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = value;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) asm volatile("bar.sync 2, %0;" ::"n"(kFillThreads) : "memory");
    else asm volatile("bar.arrive 2, %0;" ::"n"(kFillThreads) : "memory");
  }
  const uint32_t tmem = tmem_base_shared;
  // TMEM: three score buffers of 128 columns, then the output. Tile t's scores live in buffer
  // t % 3 and its probabilities (two bfloat16 per column) over their first 64 columns. With three
  // buffers and two softmax groups, a group that hands in tile t finds the scores of tile t + 2
  // computed already: their buffer was released when PV[t - 1] was issued.
  const uint32_t tmem_o = tmem + kScoreBuffers * 128;

  if (warp == 0 || warp == 10) {
    // ---- loaders: one TMA box per page piece and 64-column half; warp 0 keys, warp 10 values ---
    // (a converged warp with one elected lane issuing, as for the products below)
    const bool leader = elect_one();
    const bool keys = warp == 0;
    const int stages = keys ? kStagesK : kStagesV;
    uint64_t* full = keys ? k_full : v_full;
    uint64_t* empty = keys ? k_empty : v_empty;
    unsigned char* ring = keys ? k_ring : v_ring;
    const CUtensorMap* map = keys ? &k_map : &v_map;
    for (int it = 0; it < num_tiles; ++it) {
      const int s = it % stages;
      if (it >= stages && !bar_wait(&empty[s], ((it / stages) - 1) & 1)) {
        if (leader) atomicOr(p.err, ERRBIT_TIMEOUT_A);
        break;
      }
      uint32_t bytes = 0;
      for (int piece = 0; piece < pieces_per_tile; ++piece) {
        const int page = pages[it * pieces_per_tile + piece];
        if (page >= 0 && page < p.num_pages) bytes += 2u * p.piece_rows * 128u;
      }
      if (leader) bar_expect_tx(&full[s], bytes);
      for (int piece = 0; piece < pieces_per_tile; ++piece) {
        const int page = pages[it * pieces_per_tile + piece];
        if (page < 0) continue;
        if (page >= p.num_pages) {
          if (leader) atomicOr(p.err, ERRBIT_BAD_PAGE);
          continue;
        }
        const int key = (tile_begin + it) * kKeys + piece * p.piece_rows;
        const int arena_row = (page * p.kv_heads + kv_head) * p.page_size + (key & (p.page_size - 1));
        const int offset = piece * p.piece_rows * 128;
        if (leader) {
          tma_tile(ring + s * kTileBytesA + offset, map, &full[s], 0, arena_row);
          tma_tile(ring + s * kTileBytesA + kHalfBytes + offset, map, &full[s], 64, arena_row);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---- tensor-core issuer -----------------------------------------------------------------------
    // One thread issues every product, so the instructions between two tcgen05.mma are on the
    // critical path (with a descriptor built from an address each time they cost about 110
    // cycles per product, twice what the tensor core needs for it): the descriptors of the
    // query tile and of the first ring slots are built once, and a product's descriptor is
    // that plus a constant. The address field is 14 bits of 16-byte units and the whole of
    // shared memory fits it, so the additions never carry out of the field.
    // The whole warp walks the loop, so that everything the products take (descriptors,
    // addresses) is uniform across the warp and can live in uniform registers; one elected lane
    // issues. Inside a single-lane branch every operand had to be moved over first.
    const bool leader = elect_one();
    const uint32_t id_s = idesc(false), id_o = idesc(true);
    const uint64_t q_desc = desc_k_major(saddr(q_tile));
    const uint64_t k_desc = desc_k_major(saddr(k_ring));
    const uint64_t v_desc = desc_mn_major(saddr(v_ring));
    auto scores = [&](int it) -> bool {  // S[it % 3] = Q K^T for tile `it`
      const int s = it % kStagesK;
      if (!bar_wait(&k_full[s], (it / kStagesK) & 1)) {
        return false;
      }
      fence_after();
      const uint64_t k_here = k_desc + static_cast<uint64_t>(s * (kTileBytesA >> 4));
      const uint32_t d = (tmem + (it % kScoreBuffers) * 128);
#pragma unroll
      for (int ks = 0; ks < kDim / 16; ++ks) {
        constexpr int kHalf16 = kHalfBytes >> 4;
        const uint64_t off = static_cast<uint64_t>((ks >> 2) * kHalf16 + (ks & 3) * 2);  // 32 bytes per 16 dims
        if (leader) mma_ss(d, q_desc + off, k_here + off, id_s, ks > 0);
      }
      if (leader) {
        mma_commit(&k_empty[s]);  // K[it] is no longer read
        mma_commit(&s_full[it % kScoreBuffers]);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    for (int it = 0; it < kScoreBuffers && it < num_tiles && ok; ++it) ok = scores(it);
    for (int it = 0; it < num_tiles && ok; ++it) {
      const int s = it % kStagesV;
      // O += P V once the softmax warps have written P[it] and V[it] has landed.
      if (!bar_wait(&p_ready[it % kScoreBuffers], (it / kScoreBuffers) & 1)) {
        ok = false;
        break;
      }
      if (!bar_wait(&v_full[s], (it / kStagesV) & 1)) {
        ok = false;
        break;
      }
      fence_after();
      const uint64_t v_here = v_desc + static_cast<uint64_t>(s * (kTileBytesA >> 4));
      const uint32_t p_addr = (tmem + (it % kScoreBuffers) * 128);
#pragma unroll
      for (int ks = 0; ks < kKeys / 16; ++ks)  // 16 keys: 8 columns of P, 2,048 bytes of V
        if (leader) mma_ts(tmem_o, p_addr + ks * 8, v_here + static_cast<uint64_t>(ks * (2048 >> 4)), id_o, it > 0 || ks > 0);
      if (leader) {
        mma_commit(&v_empty[s]);      // V[it] is no longer read
        mma_commit(&o_done[it & 3]);  // nor P[it]; O holds tiles 0..it
      }
      __syncwarp();
      // The buffer P[it] lives in takes the scores of tile it + 3 (products run in issue order).
      if (it + kScoreBuffers < num_tiles && !scores(it + kScoreBuffers)) {
        ok = false;
        break;
      }
    }
    if (!ok && leader) {
      atomicOr(p.err, ERRBIT_TIMEOUT_A);
    }
  } else if (warp >= 2 && warp < 10) {
    // ---- softmax: one thread per query row and group; group 0 takes the even tiles, group 1 the odd
    // A tile's exponentials keep a quarter of the SM's special-function units busy for 1,024
    // cycles, its maximum pass and the waits take as long again: with two groups of warps one
    // group's maximum pass hides behind the other's exponentials. The two threads of a row
    // (same TMEM lane, warps w and w + 4) share the row's offset m through shared memory: a
    // tile's maximum is computed freely, but deciding whether it moves m waits until every
    // earlier tile has decided (row_next), so m changes as if one thread walked the tiles.
    const int quarter = warp & 3, group = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;  // row of the block = TMEM lane
    const int row = row_base + r;
    const bool live = row < rows_total;
    const int tok = min(row / p.group, q_len - 1);
    const int pos = first_pos + tok;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    volatile int* next_tile = &row_next[r];
    volatile float* shared_m = &row_m[r];
    float l = 0.f;            // this thread's sum, relative to the offset `seen`
    float seen = -INFINITY;
    bool ok = true;           // false after a wait gave up: later waits are skipped, the block runs out
    auto turn_of = [&](int tile) -> bool {  // spins until every tile before `tile` has decided
      if (!ok) return false;
      const long long start = clock64();
      while (*next_tile != tile) {
        if (clock64() - start > kWaitCyclesA) return false;
      }
      return true;
    };
    for (int it = group; it < num_tiles; it += 2) {
      if (ok && !__all_sync(0xffffffffu, bar_wait(&s_full[it % kScoreBuffers], (it / kScoreBuffers) & 1))) ok = false;
      fence_after();
      const int tile_start = (tile_begin + it) * kKeys;
      const uint32_t s_addr = (tmem + (it % kScoreBuffers) * 128) + lane_addr;
      // Keys [rel_lo, rel_hi] of this tile are the ones this row attends to.
      const int rel_hi = live ? pos - tile_start : -1;
      const int rel_lo = p.window > 0 ? pos - p.window + 1 - tile_start : 0;
      const bool needs_mask = __any_sync(0xffffffffu, rel_hi < kKeys - 1 || rel_lo > 0);
      // Two passes over the scores, 32 columns at a time (rolled loops: fully unrolled, this code
      // outgrew the instruction cache and the warps starved on fetches). Pass 1: the maximum.
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kKeys; c0 += 32) {
        uint32_t raw[32];
        tmem_ld32(s_addr + c0, raw);
        if (needs_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i > rel_hi || c0 + i < rel_lo) raw[i] = 0xff800000u;  // -inf
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(raw[i]));
          mx1 = fmaxf(mx1, __uint_as_float(raw[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(raw[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(raw[i + 3]));
        }
      }
      const float tile_max = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      // The offset m is only moved when this tile's maximum exceeds it by more than kSlack (in
      // log2 units): probabilities may then be as large as 2^kSlack, which bfloat16 and the
      // 32-bit sums take easily, and in exchange most tiles need no rescaling of the running
      // output, so a tile's softmax overlaps the previous tile's PV product.
      constexpr float kSlack = 8.f;
      if (!turn_of(it)) ok = false;
      float m = *shared_m;
      if (m != seen) {  // the other group moved the offset since this thread's last tile
        l *= seen == -INFINITY ? 0.f : exp2f(seen - m);
        seen = m;
      }
      float alpha = 1.f;
      const bool move = tile_max > m + kSlack;  // also the first finite maximum after m = -inf
      if (move) {
        alpha = exp2f(m - tile_max);
        m = tile_max;
        seen = m;
        l *= alpha;
        *shared_m = m;
      }
      __threadfence_block();
      *next_tile = it + 1;  // the next tile may decide; if it moves m too, it first waits for this tile's PV
      __syncwarp();
      if (__any_sync(0xffffffffu, move) && it > 0) {
        // The running output must be at rest to be rescaled: every earlier PV product retired.
        if (ok && !__all_sync(0xffffffffu, bar_wait(&o_done[(it - 1) & 3], ((it - 1) >> 2) & 1))) ok = false;
        fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < kDim; c0 += 32) {
          uint32_t raw[32];
          tmem_ld32(tmem_o + lane_addr + c0, raw);
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
          tmem_st32(tmem_o + lane_addr + c0, raw);
        }
        tmem_st_wait();
      }
      // Pass 2: P = 2^(s * scale - m) as bfloat16 pairs, written over the front of the S buffer
      // (columns c0/2.. of P replace scores that this thread has already read). The look at
      // PV[it - 2] first is what keeps this thread's view of the o_done ring current (see there).
      if (it >= 2 && ok && !__all_sync(0xffffffffu, bar_wait(&o_done[(it - 2) & 3], ((it - 2) >> 2) & 1))) ok = false;
      fence_after();
      const float offset = m == -INFINITY ? 0.f : m;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kKeys; c0 += 32) {
        uint32_t raw[32];
        tmem_ld32(s_addr + c0, raw);
        if (needs_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i > rel_hi || c0 + i < rel_lo) raw[i] = 0xff800000u;
        }
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(raw[i]), p.scale_log2, -offset));
          const float p1 = fast_exp2(fmaf(__uint_as_float(raw[i + 1]), p.scale_log2, -offset));
          const float p2 = fast_exp2(fmaf(__uint_as_float(raw[i + 2]), p.scale_log2, -offset));
          const float p3 = fast_exp2(fmaf(__uint_as_float(raw[i + 3]), p.scale_log2, -offset));
          sum0 += p0;
          sum1 += p1;
          sum2 += p2;
          sum3 += p3;
          packed[i >> 1] = pack2(p0, p1);
          packed[(i >> 1) + 1] = pack2(p2, p3);
        }
        tmem_st16((tmem + (it % kScoreBuffers) * 128) + lane_addr + (c0 >> 1), packed);
      }
      tmem_st_wait();
      l += (sum0 + sum1) + (sum2 + sum3);
      fence_before();
      bar_arrive(&p_ready[it % kScoreBuffers]);
    }
    // The finished row: O / l as bfloat16, l being both groups' sums brought to the final offset.
    if (!turn_of(num_tiles)) ok = false;
    {
      const float m = *shared_m;
      if (m != seen) l *= seen == -INFINITY ? 0.f : exp2f(seen - m);
    }
    row_l[group][r] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(kSoftmaxThreads) : "memory");
    l = row_l[0][r] + row_l[1][r];
    if (ok && num_tiles > 0) ok = bar_wait(&o_done[(num_tiles - 1) & 3], ((num_tiles - 1) >> 2) & 1);
    if (!ok && lane == 0) atomicOr(p.err, ERRBIT_TIMEOUT_A);
    fence_after();
    // Every lane takes part in the warp-wide TMEM loads (they are .sync.aligned); only lanes
    // whose row exists store. After a timeout the loads are skipped by all lanes together.
    // Group 0 stores the first half of the head's dims, group 1 the second.
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (all_ok) {
      const int token = min(row / p.group, q_len - 1);
      const int head = kv_head * p.group + (row - (row / p.group) * p.group);
      __nv_bfloat16* dst = p.out + (static_cast<int64_t>(q_start + token) * p.q_heads + head) * kDim;
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c0 = group * (kDim / 2); c0 < (group + 1) * (kDim / 2); c0 += 32) {
        uint32_t raw[32];
        tmem_ld32(tmem_o + lane_addr + c0, raw);
        if (live) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            packed[i >> 1] = pack2(__uint_as_float(raw[i]) * inv, __uint_as_float(raw[i + 1]) * inv);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(dst + c0)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        }
      }
    }
  }
  __syncwarp();
  fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

using EncodeTiledA = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledA encode_tiled_a() {
  static EncodeTiledA fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledA>(ptr);
  }
  return fn;
}

// One layer's K or V arena [pages, kv_heads, page_size, 128] as rows of 128 bfloat16; boxes of
// 64 columns x piece_rows rows.
int arena_map(CUtensorMap* map, const void* arena, int64_t rows, int piece_rows) {
  EncodeTiledA encode = encode_tiled_a();
  if (encode == nullptr) return b200_fail("flash_prefill_tcgen05: the driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {kDim, static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {kDim * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(piece_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(arena), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return b200_fail("flash_prefill_tcgen05: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(status));
  return 0;
}

}  // namespace

// Shapes the tcgen05 prefill kernel takes; the caller uses attention_flash.cu otherwise.
B200_API int b200_flash_prefill_tcgen05_supported(int q_heads, int kv_heads, int head_dim, int page_size, int max_kv_len) {
  if (head_dim != kDim || q_heads % kv_heads) return 0;
  if (page_size < 16 || (page_size & (page_size - 1))) return 0;
  const int piece = page_size < kKeys ? page_size : kKeys;
  if ((static_cast<int64_t>(max_kv_len) + kKeys) / piece + 2 > kMaxChunks) return 0;
  if (kv_heads > 65535) return 0;
  return 1;
}

// Attention of requests [first_seq, first_seq + num_seqs): each feeds `seq_q_len` new tokens
// whose keys and values are already in the arena. Query and output rows are the step's rows.
B200_API int b200_flash_prefill_tcgen05(const void* q, const void* k_arena, const void* v_arena, void* out,
                                        const int* block_table, const int* seq_q_start, const int* seq_q_len,
                                        const int* seq_kv_len, int first_seq, int num_seqs, int max_q_len,
                                        int max_kv_len, int max_pages, int num_pages, int q_heads, int kv_heads,
                                        int head_dim, int page_size, int window, float scale, int* err,
                                        cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  B200_REQUIRE(b200_flash_prefill_tcgen05_supported(q_heads, kv_heads, head_dim, page_size, max_kv_len),
               "flash_prefill_tcgen05: unsupported shape (heads %d/%d, head_dim %d, page %d, %d keys)", q_heads, kv_heads,
               head_dim, page_size, max_kv_len);
  B200_REQUIRE(num_seqs > 0 && num_seqs <= 65535 && max_q_len >= 1, "flash_prefill_tcgen05: bad batch");
  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_table = block_table;
  p.seq_q_start = seq_q_start;
  p.seq_q_len = seq_q_len;
  p.seq_kv_len = seq_kv_len;
  p.err = err;
  p.first_seq = first_seq;
  p.max_pages = max_pages;
  p.num_pages = num_pages;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = q_heads / kv_heads;
  p.page_size = page_size;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  p.page_shift = shift;
  p.piece_rows = page_size < kKeys ? page_size : kKeys;
  p.window = window;
  p.scale_log2 = scale * kLog2eA;
  CUtensorMap k_map, v_map;
  const int64_t rows = static_cast<int64_t>(num_pages) * kv_heads * page_size;
  if (arena_map(&k_map, k_arena, rows, p.piece_rows) != 0) return -1;
  if (arena_map(&v_map, v_arena, rows, p.piece_rows) != 0) return -1;
  const size_t smem = (1 + kStagesK + kStagesV) * static_cast<size_t>(kTileBytesA) + kMaxChunks * sizeof(int) + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return b200_fail("flash_prefill_tcgen05: cannot size shared memory (%zu bytes)", smem);
    configured = true;
  }
  const int row_blocks = (max_q_len * p.group + kRows - 1) / kRows;
  const dim3 grid(row_blocks, kv_heads, num_seqs);
  const cudaError_t status =
      launch_kernel(flash_prefill_tcgen05_kernel, grid, dim3(kThreadsA), smem, stream, k_map, v_map, p);
  if (status != cudaSuccess) return b200_fail("flash_prefill_tcgen05: %s", cudaGetErrorString(status));
  return 0;
}
