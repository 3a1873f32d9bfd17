// Weight-streaming matrix product on the 5th-generation tensor cores:
//   Y[M,N] = X[M,K] * W[N,K]^T  for up to 256 rows of X (decode steps and short portions).
//
// The operands swap roles so the weights fill the tensor core's wide side: a block owns 128
// rows of W (the MMA's M) and all tokens (the MMA's N, padded to a multiple of 16). One
// thread feeds a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte
// swizzle): a 128 x 64 tile of W and a tokens x 64 tile of X per stage. One thread issues
// tcgen05.mma (cta_group::1, kind::f16, bf16 in, fp32 accumulate) from those stages into a
// TMEM accumulator of 128 lanes x tokens columns and releases each stage with
// tcgen05.commit. Four warps read the accumulator back with tcgen05.ld and write Y.
// The weight tiles of the first stages are requested before the kernel waits for its
// predecessor on the stream (programmatic dependent launch), since weights never depend on it.
//
// When W has too few rows to give every SM a block, the blocks that share rows form a
// thread-block cluster and split K among them. Every member finishes a slice of the rows, adding
// the members' partial sums in rank order through distributed shared memory, so the sum does
// not depend on timing and no global scratch is needed: with up to 16 tokens the members write
// their partial sums into the owners' shared memory and the cluster meets once, with more they
// keep their tiles, meet, fetch their slices from each other and meet again (see the kernel).
//
// Every wait on an mbarrier is bounded: on a timeout the block records ERRBIT_TIMEOUT in the
// error word, stops issuing work, frees its TMEM and returns.
//
// Linear layers are x W^T with W stored [out, in] (python/instinct/backends/base.py:83-101);
// the reference sends them to cuBLASLt (cuda/execution_context.cu:95-110). Epilogues as in
// gemm_skinny.cu: bfloat16 or float32 rows, or SwiGLU over interleaved gate/up rows
// (python/instinct/backends/dense.py:124-128).
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace {

constexpr int kBlockRows = 128;  // rows of W per block = MMA M
constexpr int kBlockK = 64;      // k per stage: 128 bytes of bf16 = one swizzle row
constexpr int kMmaK = 16;
constexpr int kMaxMembers = 16;  // blocks of a cluster that share rows of W
constexpr int kMaxStages = 12;    // the launcher picks the depth from how many blocks share an SM
constexpr int kPushTokens = 16;  // up to this many (padded) tokens a cluster's partial sums are pushed to their owners
// Rows of a block that one cluster member finishes: gate/up pairs stay together, and where up to
// kWideSliceMembers members fetch their slices from each other, four rows to a load, a slice
// starts on a multiple of four rows.
constexpr int kWideSliceMembers = 4;
__host__ __device__ constexpr int slice_rows(int members, int tokens_pad) {
  const int even = ((kBlockRows + members - 1) / members + 1) & ~1;
  return tokens_pad > kPushTokens && members <= kWideSliceMembers ? (even + 3) & ~3 : even;
}
static_assert(kPushTokens >= kFoldTokens, "a product around a folded norm always takes the push form");
constexpr int kThreadsT = 192;   // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds
constexpr int ERRBIT_TIMEOUT = 8;

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - start > kWaitCycles) return false;
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle:
// groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);   // start address
  desc |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused for swizzled K-major)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                  // descriptor version (sm_100)
  desc |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
  return desc;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kBlockRows >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
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

struct StreamParams {
  void* y;
  int* err;
  int stages;
  int M, N, K;
  int tokens_pad;  // MMA N: M rounded up to a multiple of 16
  int tmem_cols;   // power of two >= max(32, tokens_pad)
  long long* trace;  // kTraceStamps timestamps per block when a sweep asked for them, else null
  NormFold fold;   // RMSNorm folded into this product (common.cuh); all null when unused
};

// The kernel is compiled once per (epilogue, way the cluster adds up, folded norm or not, traced or
// not): a block runs its epilogue once, from a cold instruction cache, and every form that shares
// the kernel's code with the others makes each of them slower (the one-for-all kernel had 85 KB
// of code; with the timestamps compiled in but switched off, 110 KB and 1.2 us more per product
// inside a decode step of 64 requests).
enum : int { MODE_SINGLE = 0, MODE_PUSH = 1, MODE_PULL = 2 };

template <int EPI>
__device__ __forceinline__ void write_output(const StreamParams& p, int m, int n, float v) {
  if constexpr (EPI == EPI_F32) static_cast<float*>(p.y)[static_cast<int64_t>(m) * p.N + n] = v;
  else static_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(m) * p.N + n] = __float2bfloat16_rn(v);
}

// A cluster member's slice of the rows, added up over the members' partial tiles
// ([tokens_pad][128 rows] in each member's shared memory) and written out; the sums run in member
// order. Two forms, chosen by the cluster's width from measurements (gate/up of 64 tokens, two
// members: 18.8 us with one 4-byte load per value and one item per round trip, 14.6 us in the wide
// form; down of 64 tokens, sixteen members: 10.9 us in the narrow form, 12.1 and 13.7 us with 8-
// and 16-byte loads).
//
// Wide, for up to kWideSliceMembers members: an item is four consecutive rows of one token (two
// gate/up pairs), fetched from each member with one 16-byte load; the slice starts on a multiple
// of four rows. A thread takes ITEMS items at a time and asks for all their values before it
// uses the first: one round trip through the cluster's shared memory per ITEMS items.
template <int EPI, int RANKS, int ITEMS>
__device__ __forceinline__ void pull_slices_wide(const StreamParams& p, const float* partial, int members, int tid,
                                                 int rows, int r_begin, int n0) {
  const int columns = (rows + 3) / 4;
  const int total = columns * p.M;
  constexpr bool swiglu = EPI == EPI_SWIGLU;
  for (int base = tid; base < total; base += 128 * ITEMS) {
    float4 part[ITEMS][RANKS];
#pragma unroll
    for (int q = 0; q < ITEMS; ++q) {
      const int item = base + q * 128;
      const int m = item / columns, r = r_begin + (item - m * columns) * 4;
#pragma unroll
      for (int rank = 0; rank < RANKS; ++rank)
        if (item < total && rank < members) part[q][rank] = load_peer_f32x4(partial + m * kBlockRows + r, rank);
    }
#pragma unroll
    for (int q = 0; q < ITEMS; ++q) {
      const int item = base + q * 128;
      if (item >= total) break;
      const int m = item / columns, r = r_begin + (item - m * columns) * 4;
      float values[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int rank = 0; rank < RANKS; ++rank) {
        if (rank < members) {
          values[0] += part[q][rank].x;
          values[1] += part[q][rank].y;
          values[2] += part[q][rank].z;
          values[3] += part[q][rank].w;
        }
      }
      const int n = n0 + r;
      const int live = min(4, min(r_begin + rows - r, p.N - n));  // rows of the item inside the slice and the matrix
      if (swiglu) {
#pragma unroll
        for (int i = 0; i < 4; i += 2)
          if (i + 1 < live)
            static_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(m) * (p.N / 2) + (n + i) / 2] =
                __float2bfloat16_rn(values[i] / (1.f + expf(-values[i])) * values[i + 1]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < live) write_output<EPI>(p, m, n + i, values[i]);
      }
    }
  }
}

// Narrow, for wider clusters: an item is one row of one token (a gate/up pair for the SwiGLU
// epilogue), every member's value asked for with a 4-byte load before the first is used.
template <int EPI>
__device__ __forceinline__ void pull_slices_narrow(const StreamParams& p, const float* partial, int members, int tid,
                                                   int rows, int r_begin, int n0) {
  if constexpr (EPI == EPI_SWIGLU) {
    const int pairs = rows / 2;
    for (int item = tid; item < pairs * p.M; item += 128) {
      const int m = item / pairs, r = r_begin + 2 * (item - m * pairs);
      float gates[kMaxMembers], ups[kMaxMembers];
#pragma unroll
      for (int rank = 0; rank < kMaxMembers; ++rank) {
        if (rank < members) {
          gates[rank] = load_peer_f32(partial + m * kBlockRows + r, rank);
          ups[rank] = load_peer_f32(partial + m * kBlockRows + r + 1, rank);
        }
      }
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int rank = 0; rank < kMaxMembers; ++rank) {
        if (rank < members) {
          gate += gates[rank];
          up += ups[rank];
        }
      }
      const int n = n0 + r;
      if (n < p.N)
        static_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(m) * (p.N / 2) + n / 2] =
            __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
    }
  } else {
    for (int item = tid; item < rows * p.M; item += 128) {
      const int m = item / rows, r = r_begin + (item - m * rows);
      float values[kMaxMembers];
#pragma unroll
      for (int rank = 0; rank < kMaxMembers; ++rank)
        if (rank < members) values[rank] = load_peer_f32(partial + m * kBlockRows + r, rank);
      float sum = 0.f;
#pragma unroll
      for (int rank = 0; rank < kMaxMembers; ++rank)
        if (rank < members) sum += values[rank];
      const int n = n0 + r;
      if (n < p.N) write_output<EPI>(p, m, n, sum);
    }
  }
}

// Where a block is in its life, for cli/microbench.py's trace: the nanosecond timer at eight
// points, one writer each. The kernel that records them is an instantiation of its own: even
// switched off at run time the stamps cost the products 0.2 to 0.8 us each (the branches around
// them sit in the loops that issue the MMAs and in the epilogue).
constexpr int kTraceStamps = 8;
template <bool TRACED>
__device__ __forceinline__ void stamp(const StreamParams& p, int which) {
  if constexpr (!TRACED) return;
  if (p.trace == nullptr) return;
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  p.trace[(static_cast<int64_t>(blockIdx.y) * gridDim.x + blockIdx.x) * kTraceStamps + which] = t;
}

template <int EPI, int MODE, bool FOLDED, bool TRACED>
__global__ void __launch_bounds__(kThreadsT)
stream_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                   const StreamParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // Stage s: W tile (128 x 128 B) then X tile (tokens_pad x 128 B), each 1024-byte aligned.
  const uint32_t w_bytes = kBlockRows * kBlockK * 2;
  const uint32_t x_bytes = static_cast<uint32_t>(p.tokens_pad) * kBlockK * 2;
  const uint32_t x_stride = (x_bytes + 1023u) & ~1023u;
  const uint32_t stage_bytes = w_bytes + x_stride;
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ uint32_t tmem_base_shared;
  __shared__ float rstd_s[kFoldTokens];
  __shared__ float squares[FOLDED ? kFoldTokens * kBlockRows : 1];  // [m][row of this member's slice]
  constexpr bool clustered = MODE != MODE_SINGLE, push = MODE == MODE_PUSH;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int n0 = blockIdx.x * kBlockRows;
  const int members = gridDim.y;  // blocks of this cluster; blockIdx.y is the rank
  const int k_blocks = (p.K + kBlockK - 1) / kBlockK;
  const int per_block = (k_blocks + members - 1) / members;
  const int kb_begin = blockIdx.y * per_block;
  const int kb_end = min(k_blocks, kb_begin + per_block);
  const int num_kb = max(0, kb_end - kb_begin);

  if (threadIdx.x == 0) {
    let_successor_start();
    stamp<TRACED>(p, 0);  // the block is resident
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // The thread that made the barriers also loads: the weights of the first stages are on
    // their way before the block has even met (they depend on nothing that runs before).
    const int first = min(num_kb, stages);
    for (int i = 0; i < first; ++i) {
      mbar_expect_tx(&full_bar[i], w_bytes + x_bytes);
      tma_load_2d(tiles + i * stage_bytes, &w_map, &full_bar[i], (kb_begin + i) * kBlockK, n0);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_shared)),
                 "r"(static_cast<uint32_t>(p.tmem_cols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_shared;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer -----------------------------------------------------------------------
    // The weights of the first stages went out above; X follows the dependency wait.
    const int first = min(num_kb, stages);
    wait_for_predecessor();
    let_successor_start();
    stamp<TRACED>(p, 1);  // the kernel in front is complete
    for (int i = 0; i < first; ++i)
      tma_load_2d(tiles + i * stage_bytes + w_bytes, &x_map, &full_bar[i], (kb_begin + i) * kBlockK, 0);
    for (int i = first; i < num_kb; ++i) {
      const int s = i % stages;
      const uint32_t parity = ((i / stages) - 1) & 1;
      if (!mbar_wait(&empty_bar[s], parity)) {
        atomicOr(p.err, ERRBIT_TIMEOUT);
        break;
      }
      mbar_expect_tx(&full_bar[s], w_bytes + x_bytes);
      tma_load_2d(tiles + s * stage_bytes, &w_map, &full_bar[s], (kb_begin + i) * kBlockK, n0);
      tma_load_2d(tiles + s * stage_bytes + w_bytes, &x_map, &full_bar[s], (kb_begin + i) * kBlockK, 0);
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------------
    // The whole warp walks the loop and one elected lane issues: what the products take
    // (descriptors, addresses) is then uniform across a converged warp and can stay in uniform
    // registers, where inside a single-lane branch every operand had to be moved over for
    // every product. A stage's descriptors are the first stage's plus a constant: the address
    // field counts 16-byte units and all of shared memory fits it, so nothing carries out.
    uint32_t chosen;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(chosen));
    const bool leader = chosen != 0;
    const uint32_t idesc = umma_instr_desc(p.tokens_pad);
    const uint64_t a_first = umma_smem_desc(smem_addr(tiles));
    const uint64_t b_first = umma_smem_desc(smem_addr(tiles) + w_bytes);
    bool alive = true;
    for (int i = 0; i < num_kb && alive; ++i) {
      const int s = i % stages;
      if (!mbar_wait(&full_bar[s], (i / stages) & 1)) {
        if (leader) atomicOr(p.err, ERRBIT_TIMEOUT);
        alive = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (leader && i == 0) stamp<TRACED>(p, 2);           // the first stage has landed
      if (leader && i == num_kb - 1) stamp<TRACED>(p, 3);  // the last one has
      const uint64_t stage_units = static_cast<uint64_t>(s) * (stage_bytes >> 4);
#pragma unroll
      for (int k = 0; k < kBlockK / kMmaK; ++k) {
        const uint64_t step = stage_units + static_cast<uint64_t>(k * (kMmaK * 2 >> 4));
        if (leader) umma_bf16(tmem_base, a_first + step, b_first + step, idesc, i > 0 || k > 0);
      }
      if (leader) umma_commit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
      __syncwarp();
    }
    if (leader) umma_commit(&accum_bar);  // the accumulator is complete once every MMA has retired
  }
  __syncwarp();

  // ---- epilogue: TMEM -> registers -> global, or -> shared memory when the cluster splits K ----
  // A cluster's members each hold a partial tile; member r finishes rows [r * slice, (r + 1) * slice).
  // With up to kPushTokens tokens every member writes its values straight into the shared memory
  // of the row's owner (an inbox behind the ring, which a member that is still streaming does
  // not touch), the cluster meets once, and each owner adds up what lies in its own memory and
  // may leave when it is done. With more tokens the inboxes would cost the ring its depth: the
  // members then put their tiles into their own rings, meet, fetch their slices from each other
  // with several items' loads in flight at once, and meet again before any of them leaves.
  const int slice = slice_rows(members, p.tokens_pad);
  float* partial = reinterpret_cast<float*>(tiles);  // [tokens_pad][128 rows]; the stages are idle by then
  float* inbox = reinterpret_cast<float*>(tiles + static_cast<size_t>(stages) * stage_bytes);  // [members][M][slice]
  const bool scaled = FOLDED && p.fold.ss_in != nullptr;
  const bool residual = FOLDED && p.fold.x != nullptr;  // the product is added into the residual stream
  if (warp >= 2) {
    wait_for_predecessor();
    if (scaled) {
      // The operand is the stream times a norm's scale: each token's 1 / rms from the partial sums
      // of squares, while the products run. Four tokens per epilogue warp.
      for (int m = warp - 2; m < p.M; m += 4) {
        const float r = fold_rstd(p.fold, m);
        if (lane == 0) rstd_s[m] = r;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const int quarter = warp & 3;  // TMEM lanes 32 * quarter .. + 31 belong to this warp
    const int row = quarter * 32 + lane;
    const int n = n0 + row;
    bool have = num_kb > 0;
    if (have && !mbar_wait(&accum_bar, 0)) {
      if (lane == 0) atomicOr(p.err, ERRBIT_TIMEOUT);
      have = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (threadIdx.x == 64) stamp<TRACED>(p, 4);  // the accumulator is complete
    for (int c0 = 0; c0 < p.tokens_pad; c0 += 16) {
      float v[16];
      if (have) {
        tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      if (push) {
        const int owner = row / slice;
        const uint32_t mine =
            peer_address(inbox + (static_cast<int>(blockIdx.y) * p.M + c0) * slice + (row - owner * slice), owner);
        const uint32_t pitch = static_cast<uint32_t>(slice) * sizeof(float);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c0 + i < p.M) store_peer_f32(mine + i * pitch, v[i]);
      } else if (clustered) {
#pragma unroll
        for (int i = 0; i < 16; ++i) partial[(c0 + i) * kBlockRows + row] = v[i];
      } else if (residual) {
        // Into the residual stream; partial sums of squares per (block, quarter of its rows).
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = c0 + i;
          float sq = 0.f;
          if (m < p.M && n < p.N) {
            const int64_t at = static_cast<int64_t>(m) * p.N + n;
            const float now = p.fold.x[at] + v[i];
            p.fold.x[at] = now;
            p.fold.xn[at] = __float2bfloat16_rn(now * p.fold.next_weight[n]);
            sq = now * now;
          }
          sq = warp_sum(sq);
          if (lane == 0 && m < kFoldTokens)
            p.fold.ss_out[(static_cast<int64_t>(blockIdx.x) * 4 + quarter) * kFoldTokens + m] = sq;
        }
      } else if (EPI == EPI_SWIGLU) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = c0 + i;
          const float gate = scaled && m < p.M ? v[i] * rstd_s[m] : v[i];
          const float up = __shfl_down_sync(0xffffffffu, gate, 1);
          if ((lane & 1) == 0 && m < p.M && n < p.N)
            static_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(m) * (p.N / 2) + n / 2] =
                __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c0 + i < p.M && n < p.N) write_output<EPI>(p, c0 + i, n, scaled ? v[i] * rstd_s[c0 + i] : v[i]);
      }
    }
  }
  if (clustered) {
    // Every thread of every member meets here; then each member finishes its slice of the rows.
    cluster_sync_all();
    if (threadIdx.x == 64) stamp<TRACED>(p, 5);  // every member's partial sums are where their owner reads them
    const int r_begin = blockIdx.y * slice, r_end = min(kBlockRows, r_begin + slice);
    const int rows = max(0, r_end - r_begin);
    if (warp >= 2 && push) {
      // The sums run in member order over this block's own inbox.
      const int tid = threadIdx.x - 64;
      const int plane = p.M * slice;
      if (EPI == EPI_SWIGLU) {
        const int pairs = rows / 2;
        for (int item = tid; item < pairs * p.M; item += 128) {
          const int m = item / pairs, j = item - m * pairs;
          const float* at = inbox + m * slice + 2 * j;
          float gate = 0.f, up = 0.f;
          for (int rank = 0; rank < members; ++rank) {
            const float2 both = *reinterpret_cast<const float2*>(at + rank * plane);
            gate += both.x;
            up += both.y;
          }
          if (scaled) {
            gate *= rstd_s[m];
            up *= rstd_s[m];
          }
          const int n = n0 + r_begin + 2 * j;
          if (n < p.N)
            static_cast<__nv_bfloat16*>(p.y)[static_cast<int64_t>(m) * (p.N / 2) + n / 2] =
                __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
      } else {
        for (int item = tid; item < rows * p.M; item += 128) {
          const int m = item / rows, r = item - m * rows;
          const float* at = inbox + m * slice + r;
          float sum = 0.f;
          for (int rank = 0; rank < members; ++rank) sum += at[rank * plane];
          if (scaled) sum *= rstd_s[m];
          const int n = n0 + r_begin + r;
          if (residual) {
            float sq = 0.f;
            if (n < p.N) {
              const int64_t to = static_cast<int64_t>(m) * p.N + n;
              const float now = p.fold.x[to] + sum;
              p.fold.x[to] = now;
              p.fold.xn[to] = __float2bfloat16_rn(now * p.fold.next_weight[n]);
              sq = now * now;
            }
            squares[m * kBlockRows + r] = sq;
          } else if (n < p.N) {
            write_output<EPI>(p, m, n, sum);
          }
        }
        if (residual) {
          // This member's partial sums of squares, one per token, added in row order.
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (tid < p.M && tid < kFoldTokens) {
            float total = 0.f;
            for (int r = 0; r < rows; ++r) total += squares[tid * kBlockRows + r];
            p.fold.ss_out[(static_cast<int64_t>(blockIdx.x) * members + blockIdx.y) * kFoldTokens + tid] = total;
          }
        }
      }
      if (threadIdx.x == 64) stamp<TRACED>(p, 6);  // this member's slice is stored
    } else if (!push) {
      if (warp >= 2) {
        const int tid = threadIdx.x - 64;
        if (members <= 2) pull_slices_wide<EPI, 2, 4>(p, partial, members, tid, rows, r_begin, n0);
        else if (members <= kWideSliceMembers) pull_slices_wide<EPI, kWideSliceMembers, 2>(p, partial, members, tid, rows, r_begin, n0);
        else pull_slices_narrow<EPI>(p, partial, members, tid, rows, r_begin, n0);
        if (threadIdx.x == 64) stamp<TRACED>(p, 6);  // this member's slice is stored
      }
      cluster_sync_all();  // nobody leaves while its shared memory is still being read
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0) stamp<TRACED>(p, 7);  // about to leave
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(p.tmem_cols))
                 : "memory");
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

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of 64 k x box_rows rows.
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return b200_fail("stream_gemm: the driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {kBlockK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) return b200_fail("stream_gemm: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(status));
  return 0;
}

struct StreamPlan {
  int blocks;
  int members;  // blocks per cluster: they share rows of W and split K
  int stages;
  size_t smem;
};

// The kernel's instantiations. A product around a folded norm is never traced and never has more
// than kPushTokens tokens (so its cluster never takes the pull form).
using StreamKernel = void (*)(const CUtensorMap, const CUtensorMap, const StreamParams);

template <int EPI, int MODE>
StreamKernel pick_form(bool folded, bool traced) {
  if constexpr (MODE != MODE_PULL) {
    if (folded) return stream_gemm_kernel<EPI, MODE, true, false>;
  }
  return traced ? stream_gemm_kernel<EPI, MODE, false, true> : stream_gemm_kernel<EPI, MODE, false, false>;
}
template <int EPI>
StreamKernel pick_mode(int mode, bool folded, bool traced) {
  switch (mode) {
    case MODE_SINGLE: return pick_form<EPI, MODE_SINGLE>(folded, traced);
    case MODE_PUSH: return pick_form<EPI, MODE_PUSH>(folded, traced);
    default: return pick_form<EPI, MODE_PULL>(folded, traced);
  }
}
StreamKernel pick_kernel(int epilogue, int mode, bool folded, bool traced) {
  switch (epilogue) {
    case EPI_F32: return pick_mode<EPI_F32>(mode, folded, traced);
    case EPI_SWIGLU: return pick_mode<EPI_SWIGLU>(mode, folded, traced);
    default: return pick_mode<EPI_BF16>(mode, folded, traced);
  }
}
int cluster_mode(int members, int tokens_pad) {
  return members <= 1 ? MODE_SINGLE : (tokens_pad <= kPushTokens ? MODE_PUSH : MODE_PULL);
}

// An instantiation's opt-ins, asked for when it is first used: as much dynamic shared memory as
// any plan wants, and clusters of more than eight blocks.
constexpr size_t kMaxDynamicSmem = 200 * 1024;
bool prepare_kernel(StreamKernel kernel) {
  static std::mutex guard;
  static std::vector<StreamKernel> ready;
  std::lock_guard<std::mutex> lock(guard);
  for (StreamKernel known : ready)
    if (known == kernel) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxDynamicSmem)) !=
          cudaSuccess ||
      cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  ready.push_back(kernel);
  return true;
}

// What a parameter sweep (cli/microbench.py) forces instead of the planner's own choices; zeros
// in normal use. Set through b200_stream_gemm_plan_override, never from the environment.
struct PlanOverride { int stages = 0, target = 0, members = 0; };
PlanOverride g_plan_override;

void size_ring(StreamPlan& plan, int k_blocks, int tokens_pad) {
  const size_t x_stride = (static_cast<size_t>(tokens_pad) * kBlockK * 2 + 1023) & ~size_t(1023);
  const size_t stage = static_cast<size_t>(kBlockRows) * kBlockK * 2 + x_stride;
  const int total = plan.blocks * plan.members;
  const size_t budget = total <= 2 * b200_sm_count_host() ? 100 * 1024 : 66 * 1024;
  const int per_block = (k_blocks + plan.members - 1) / plan.members;
  int stages = static_cast<int>(budget / stage);
  if (g_plan_override.stages > 0) stages = g_plan_override.stages;
  stages = stages > kMaxStages ? kMaxStages : stages;
  stages = stages > per_block ? per_block : stages;
  plan.stages = stages < 2 ? 2 : stages;
  const size_t partial = static_cast<size_t>(tokens_pad) * kBlockRows * sizeof(float);
  const size_t ring = plan.stages * stage;
  if (plan.members > 1 && tokens_pad <= kPushTokens) {
    // The inbox lies behind the ring: [members][M][slice] partial sums.
    const int slice = slice_rows(plan.members, tokens_pad);
    plan.smem = ring + static_cast<size_t>(plan.members) * tokens_pad * slice * sizeof(float) + 1024;
  } else {
    plan.smem = (ring > partial ? ring : partial) + 1024;
  }
}

// How many clusters of `members` blocks the device holds at once when every SM takes one
// block (clusters do not straddle GPCs, so this is less than SMs / members); 0 if the question
// cannot be answered. Plans are remembered, so this runs once per shape.
int clusters_one_per_sm(int members) {
  const StreamKernel kernel = pick_kernel(EPI_BF16, MODE_PULL, false, false);  // the forms differ by a few registers only
  if (!prepare_kernel(kernel)) return 0;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1, members * 64);
  config.blockDim = dim3(kThreadsT);
  config.dynamicSmemBytes = 48 * 1024;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 1;
  attribute.val.clusterDim.y = members;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

// A lower bound on the clusters of `members` blocks of `smem` bytes that run at once. The
// occupancy call answers for one block per SM whatever the block's size, while the profiler's
// launch statistics and the timings say that blocks of 93 KB run two to an SM. With s blocks
// per SM a GPC of g SMs takes floor(s g / members) clusters, which is what one block per SM
// gives for clusters of members / s blocks; rounding that size up keeps the bound safe.
int clusters_in_flight(int members, size_t smem) {
  int per_sm = static_cast<int>((227 * 1024) / (smem + 2048));
  per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
  return clusters_one_per_sm((members + per_sm - 1) / per_sm);
}

StreamPlan plan_stream_uncached(int N, int K, int tokens_pad) {
  StreamPlan plan;
  plan.blocks = (N + kBlockRows - 1) / kBlockRows;
  const int k_blocks = (K + kBlockK - 1) / kBlockK;
  const int sms = b200_sm_count_host();
  int target = 2 * sms;  // blocks aimed at: two per SM, so that neighbouring kernels' blocks can share SMs
  if (g_plan_override.target > 0) target = g_plan_override.target;
  // Clusters of up to 8 blocks are portable; 16 (which sm_100 schedules when asked) are used
  // when 8 would leave SMs without a block: the 1.5B down product (12 row blocks) went from
  // 10.6 to 8.6 us with them.
  int widest = plan.blocks * 8 < sms ? 16 : 8;
  if (g_plan_override.members > 0) widest = g_plan_override.members;
  int members = max(1, min(min(widest, kMaxMembers), target / plan.blocks));
  while (members > 1 && k_blocks / members < 3) --members;  // every block keeps a few stages to stream
  plan.members = members;
  size_ring(plan, k_blocks, tokens_pad);
  // All clusters should run at once: one that has to wait for a place starts when the others
  // are done, and the product takes half as long again (40 row blocks in clusters of 7 took
  // 16.5 us where clusters of 6 took 11.6 us; 36 in clusters of 8 12.0 us, of 6 8.7 us).
  // Narrow the clusters until they do.
  if (members > 1 && g_plan_override.members <= 0) {
    StreamPlan narrower = plan;
    while (narrower.members > 1) {
      const int room = clusters_in_flight(narrower.members, narrower.smem);
      if (room == 0 || narrower.blocks <= room) break;
      --narrower.members;
      size_ring(narrower, k_blocks, tokens_pad);
    }
    // Clusters of one block never all fit when wider ones did not; then width is not the matter.
    if (narrower.members > 1) plan = narrower;
  }
  return plan;
}

// Where the next launches record their blocks' timestamps (b200_stream_gemm_trace): launch i of
// the `launches` that follow writes kTraceStamps values per block from `buffer + i * stride`.
struct TraceTarget { long long* buffer = nullptr; int launches = 0, stride = 0, next = 0; };
TraceTarget g_trace;

// The plan is a function of N, K and the padded token count only (see gemm_skinny.cu for why
// not of M): about two blocks per SM, each with a ring of at most half an SM's shared memory,
// so that the blocks of the next kernel on the stream can move in and request their weights
// while this one drains (measured on a B200: 6% off a whole decode step against one block of
// 200 KB). Plans are remembered: the occupancy question costs more than a launch.
StreamPlan plan_stream(int N, int K, int tokens_pad) {
  struct Entry { int n, k, tokens; StreamPlan plan; };
  static std::mutex guard;
  static std::vector<Entry> known;
  std::lock_guard<std::mutex> lock(guard);
  if (g_plan_override.stages > 0 || g_plan_override.target > 0 || g_plan_override.members > 0)
    return plan_stream_uncached(N, K, tokens_pad);  // a sweep in progress: nothing is remembered
  for (const Entry& e : known)
    if (e.n == N && e.k == K && e.tokens == tokens_pad) return e.plan;
  const StreamPlan plan = plan_stream_uncached(N, K, tokens_pad);
  known.push_back({N, K, tokens_pad, plan});
  return plan;
}

}  // namespace

constexpr int kStreamMaxRows = 256;

// Shapes the kernel takes: at most 256 rows of X, K a multiple of 8 (row pitch a multiple of 16
// bytes, which TMA needs), N even for the SwiGLU epilogue.
B200_API int b200_stream_gemm_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > kStreamMaxRows || N < 1 || K < 8 || K % 8) return 0;
  if (epilogue == EPI_SWIGLU && N % 2) return 0;
  return 1;
}

// For parameter sweeps only: force the ring depth, the number of blocks aimed at or the cluster
// width of every later plan (0 = the planner's own choice). Plans made meanwhile are not remembered.
// A sweep's timeline (cli/microbench.py): the next `launches` launches of the kernel write eight
// timestamps per block into `buffer` (device memory, zeroed by the caller), `stride` values
// apart; launches whose blocks do not fit a stride, and all later ones, record nothing. Null
// switches it off. A launch captured in a graph keeps its place at every replay.
B200_API void b200_stream_gemm_trace(long long* buffer, int launches, int stride) {
  g_trace.buffer = buffer;
  g_trace.launches = buffer != nullptr ? launches : 0;
  g_trace.stride = stride;
  g_trace.next = 0;
}
B200_API int b200_stream_gemm_trace_stamps() { return kTraceStamps; }

B200_API void b200_stream_gemm_plan_override(int stages, int target, int members) {
  g_plan_override.stages = stages;
  g_plan_override.target = target;
  g_plan_override.members = members;
}

static int stream_gemm_run(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, int* err,
                           const NormFold& fold, cudaStream_t stream);

B200_API int b200_stream_gemm(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, int* err,
                              cudaStream_t stream) {
  return stream_gemm_run(W, X, Y, M, N, K, epilogue, err, NormFold{}, stream);
}

// With a folded norm behind it (NormFold in common.cuh): how many rows of partial sums of squares a
// launch with the residual epilogue writes: one per cluster member, or per quarter of a block
// that shares its rows with nobody.
B200_API int b200_stream_gemm_fold_parts(int M, int N, int K) {
  const StreamPlan plan = plan_stream(N, K, (M + 15) / 16 * 16);
  return plan.members > 1 ? plan.blocks * plan.members : plan.blocks * 4;
}

// The same product around a folded RMSNorm; the arguments are those of b200_skinny_gemm_fold.
B200_API int b200_stream_gemm_fold(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, int* err,
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
  B200_REQUIRE(M <= kFoldTokens, "stream_gemm_fold: at most %d tokens", kFoldTokens);
  B200_REQUIRE(ss_in == nullptr || (ss_parts > 0 && width > 0), "stream_gemm_fold: partial sums without their count");
  B200_REQUIRE(x == nullptr || (next_weight != nullptr && xn != nullptr && ss_out != nullptr && epilogue == EPI_BF16),
               "stream_gemm_fold: the residual epilogue needs the next norm's scale, xn and ss_out");
  B200_REQUIRE(x != nullptr || Y != nullptr, "stream_gemm_fold: no output");
  return stream_gemm_run(W, X, Y, M, N, K, epilogue, err, fold, stream);
}

static int stream_gemm_run(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue, int* err,
                           const NormFold& fold, cudaStream_t stream) {
  B200_REQUIRE(b200_stream_gemm_supported(M, N, K, epilogue), "stream_gemm: unsupported shape %d x %d x %d", M, N, K);
  B200_REQUIRE(epilogue >= EPI_BF16 && epilogue <= EPI_SWIGLU, "stream_gemm: unknown epilogue %d", epilogue);
  B200_REQUIRE(reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0,
               "stream_gemm: operands must be 16-byte aligned");
  StreamParams p;
  p.y = Y;
  p.err = err;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tokens_pad = (M + 15) / 16 * 16;
  p.tmem_cols = 32;
  while (p.tmem_cols < p.tokens_pad) p.tmem_cols *= 2;
  p.fold = fold;
  const StreamPlan plan = plan_stream(N, K, p.tokens_pad);
  p.stages = plan.stages;
  const bool folded = fold.ss_in != nullptr || fold.x != nullptr;
  p.trace = nullptr;
  if (!folded && g_trace.next < g_trace.launches && plan.blocks * plan.members * kTraceStamps <= g_trace.stride)
    p.trace = g_trace.buffer + static_cast<int64_t>(g_trace.next++) * g_trace.stride;
  CUtensorMap w_map, x_map;
  if (make_map(&w_map, W, N, K, kBlockRows) != 0) return -1;
  if (make_map(&x_map, X, M, K, p.tokens_pad) != 0) return -1;
  const int mode = cluster_mode(plan.members, p.tokens_pad);
  B200_REQUIRE(!(folded && (mode == MODE_PULL || p.trace != nullptr)), "stream_gemm: a folded norm with %d tokens", M);
  B200_REQUIRE(plan.smem <= kMaxDynamicSmem, "stream_gemm: the plan wants %zu bytes of shared memory", plan.smem);
  const StreamKernel kernel = pick_kernel(epilogue, mode, folded, p.trace != nullptr);
  if (!prepare_kernel(kernel)) return b200_fail("stream_gemm: the kernel's attributes could not be set");
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.blocks, plan.members);
  config.blockDim = dim3(kThreadsT);
  // The plan reserves an inbox for a full padded step; a launch asks for its own tokens' worth, so
  // that short steps leave more of the SM to the blocks of the kernels around them.
  size_t smem = plan.smem;
  if (plan.members > 1 && p.tokens_pad <= kPushTokens)
    smem -= static_cast<size_t>(plan.members) * (p.tokens_pad - M) * slice_rows(plan.members, p.tokens_pad) * sizeof(float);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int count = 0;
  if (plan.members > 1) {
    attributes[count].id = cudaLaunchAttributeClusterDimension;
    attributes[count].val.clusterDim.x = 1;
    attributes[count].val.clusterDim.y = plan.members;
    attributes[count].val.clusterDim.z = 1;
    ++count;
  }
  if (b200_overlap_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  const cudaError_t status = cudaLaunchKernelEx(&config, kernel, w_map, x_map, p);
  if (status != cudaSuccess) return b200_fail("stream_gemm: %s", cudaGetErrorString(status));
  return 0;
}
