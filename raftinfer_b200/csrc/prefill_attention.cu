// Causal GQA prefill attention with online softmax and a sigmoid output gate, head_dim 256, BF16 head-major KV
// cache, any number of query heads that is a multiple of the KV heads (replaces
// cpp/kernels/qwen35_online_attention.cu:296-322 append and :499-600 prefill; CPU form
// cpp/reference/qwen35.cpp:316-370).
//
// One persistent kernel, one CTA per SM, 320 threads.  The (128-query tile, head) items of the launch are sorted
// long-first and dealt to the CTAs in snake order; a CTA walks its items without leaving, and the first loads and
// score products of an item overlap the epilogue of the one before.
//   warp 8   producer (one lane).  TMA tiled loads with the 128-byte swizzle: the Q tile (64 KiB), then K and V
//            through a ring of five 32 KiB slots.  Key blocks that lie wholly inside this chunk come straight
//            from the BF16 key / value inputs; older blocks come from the cache (the tensor maps end at the live
//            context, so rows the cache has never held arrive as zeros).  The CTA that serves the first query head
//            of a KV group, on the tile whose last block it is, also writes such a block to the cache with TMA
//            stores once the MMAs have consumed it: that is this chunk's append (BF16 inputs are stored as they
//            are, which is what the reference's append writes).  A separate append kernel runs first only for
//            FP32 inputs (converted nearest-even) and for the rows that share a key block with the past; the
//            producer waits for it (programmatic dependent launch) before it reads such rows.  For FP32 inputs
//            that kernel also rounds the queries to BF16 and parks each Q tile in the rows of the output buffer
//            that the same tile will overwrite with its result, which is where the producer loads it from.
//   warp 9   MMA issue.  The whole warp walks the loops and one elected lane issues tcgen05.mma (BF16 in, FP32
//            accumulate in tensor memory), so ring positions and descriptors stay warp-uniform.  Tensor memory holds
//            the output tile O (128 lanes x 256 columns) and two score tiles S (128 x 128 each): 512 columns in all.
//            S = Q K^T takes both operands from shared memory (K-major); O += P V takes P from tensor memory
//            (written over the S tile it came from, as BF16) and V from shared memory (dim-major).
//            The issue order QK(j+1), PV(j) keeps the tensor pipe busy while the softmax of block j runs.
//   warps 0-7 softmax, two groups of four warps: a thread owns one query row (its tensor-memory lane) and 64 of
//            the 128 score columns, FP32, ex2.  Two warps per scheduler hide each other's latencies; with one
//            the softmax, not the tensor pipe, set the pace.  The running maximum used for the exponentials only
//            moves when it falls more than 8 (base-2) behind, at which point the threads rescale their rows of
//            O in tensor memory; this is rare after the first blocks.  The same threads normalise, gate and
//            store the tile at the end.
// Pair form (GQA group even): the two CTAs of a cluster take two query heads of one KV head at the same tile and
// run as one tcgen05 cta_group::2 unit (M = 256); each CTA loads half of every K block and half of every V block.
// Split form (few items, many key blocks each: a 512-token chunk against a long past, or the long tiles of a few
// heads of a long prompt): a second CTA (or pair) of the cluster takes the second half of an item's key blocks and
// hands its partial tile over through distributed shared memory at the end; items too short to be worth the
// hand-over are walked by the first CTA (or pair) alone.
//
// Work per launch: 4 * heads * 256 * (T * P + T (T + 1) / 2) flops for T new tokens after P past tokens.
// Every wait on an mbarrier is bounded; when one runs out the CTA records RIB200_DEVICE_WAIT_TIMED_OUT, nothing
// waits any more, tensor memory is released and the kernel returns.

#include "common.hpp"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <type_traits>

namespace rib200 {
namespace {

constexpr int kHeadDim = 256;
// Head counts are run-time values (the reference's prefill takes any query_heads that is a multiple of kv_heads,
// cpp/kernels/qwen35_online_attention.cu:33-44), which is also what a head-sharded rank passes: its own slice.
constexpr int kTileRows = 128;  // query rows per CTA
constexpr int kBlockKeys = 128; // keys per score tile
constexpr int kHalfKeys = 64;   // keys per ring slot
constexpr int kSlots = 5;
constexpr int kBoxCols = 64;                              // 64 BF16 = one 128-byte swizzle row
constexpr int kQBoxBytes = kTileRows * 128;               // 16 KiB
constexpr int kQBytes = 4 * kQBoxBytes;                   // 64 KiB
constexpr int kSlotBoxBytes = kHalfKeys * 128;            // 8 KiB
constexpr int kSlotBytes = 4 * kSlotBoxBytes;             // 32 KiB
constexpr int kKeyBoxBytes = kBlockKeys * 128;            // K slot: two boxes of 128 keys x 64 dims, 16 KiB each
constexpr int kRingOffset = kQBytes;
constexpr int kBarrierOffset = kRingOffset + kSlots * kSlotBytes;
constexpr int kExchangeOffset = kBarrierOffset + 256;     // row maxima / row sums passed between the two softmax groups
constexpr int kSmemBytes = kExchangeOffset + 2 * 2 * kTileRows * 4;
constexpr int kSoftmaxThreads = 256;                      // two groups of four warps, 64 score columns per thread
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr long long kWaitLimitCycles = 1LL << 30;
constexpr float kScaleLog2e = 0.0625F * 1.4426950408889634F; // (1 / sqrt(256)) * log2(e)
constexpr float kRescaleThreshold = 8.0F;
// Split form: an item shares its key blocks between two CTAs (or pairs) when it has at least this many.  The
// hand-over of the partial tile costs about as much as five blocks, so where only part of a launch's items are long
// (a rank's slice of the heads of a long prompt, tiles of 1 .. 32 blocks) the bar is higher.
constexpr std::uint32_t kSplitMinBlocks = 4;
constexpr std::uint32_t kSplitMinBlocksLate = 20;

// barrier indices (8 bytes each) inside the barrier block
enum : int {
  kBarQFull = 0,
  kBarFull = 1,             // kSlots
  kBarEmpty = 1 + kSlots,   // kSlots
  kBarSFull = 1 + 2 * kSlots,  // 2
  kBarPFull = 3 + 2 * kSlots,  // 2
  kBarPvDone = 5 + 2 * kSlots, // 2
  kBarQFree = 7 + 2 * kSlots,  // the tile's last score product has read Q
  kBarOFree = 8 + 2 * kSlots,  // the tile's epilogue has read O
  kBarDrain = 9 + 2 * kSlots,  // used once, by a CTA that has given up: its MMAs have drained
  kBarPeerFull = 10 + 2 * kSlots, // split form: the partner's partial result has landed in this CTA's ring
  kBarPeerFree = 11 + 2 * kSlots, // split form: the partner's ring may be written
  kBarStoresDone = 12 + 2 * kSlots, // split form: the producer's write-backs to the cache have read their slots
  kBarCount = 13 + 2 * kSlots
};

// Optional timeline probe (compile with -DRIB200_TRACE): the first CTA of the grid stamps clock64() at the
// points named below, 16 stamps per key block, into a device array that rib200_debug_read_trace copies out.
#ifdef RIB200_TRACE
__device__ long long g_trace[128 * 16];
__device__ long long g_cta_trace[1024 * 4]; // per CTA: start ns, end ns, key blocks, SM id
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define RIB200_STAMP(block, slot)                                                   \
  do {                                                                              \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (block) < 128) {                      \
      g_trace[(block) * 16 + (slot)] = clock64();                                   \
    }                                                                               \
  } while (0)
#define RIB200_STAMP_CTA2(slot)                                                     \
  do {                                                                              \
    if (blockIdx.x == 2 && blockIdx.y == 0) {                                       \
      g_trace[120 * 16 + (slot)] = global_ns();                                     \
    }                                                                               \
  } while (0)
#define RIB200_STAMP_NS(slot)                                                       \
  do {                                                                              \
    if (blockIdx.x == 0 && blockIdx.y == 0) {                                       \
      g_trace[121 * 16 + (slot)] = global_ns();                                     \
    }                                                                               \
  } while (0)
#else
#define RIB200_STAMP_NS(slot)                                                       \
  do {                                                                              \
  } while (0)
#define RIB200_STAMP(block, slot)                                                   \
  do {                                                                              \
  } while (0)
#define RIB200_STAMP_CTA2(slot)                                                     \
  do {                                                                              \
  } while (0)
#endif

struct PrefillParams {
  const void *gate;
  void *output;                // this GPU's output buffer
  void *peers[7];              // head-sharded form: the other ranks' buffers, which receive a copy of every tile
  std::uint32_t peer_count;
  std::uint32_t output_heads;  // heads per row of a destination buffer
  std::uint32_t output_head_offset;
  std::uint32_t tokens;
  std::uint32_t past;
  std::uint32_t tiles;
  std::uint32_t query_heads;
  std::uint32_t group; // query heads per KV head
  std::uint32_t split_min_blocks; // split form: items with fewer key blocks are left to the first CTA (or pair) alone
  unsigned int *status;
};

__device__ __forceinline__ std::uint32_t smem_u32(const void *p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(std::uint32_t bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(std::uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(std::uint32_t bar, std::uint32_t parity) {
  std::uint32_t done;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0;
}

// Bounded wait.  Returns false when the wait ran out or another role has already given up.
__device__ __forceinline__ bool mbar_wait(std::uint32_t bar, std::uint32_t parity, volatile std::uint32_t *abort_flag) {
  if (mbar_try_wait(bar, parity)) {
    return true;
  }
  const long long started = clock64();
  std::uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255U) == 0) {
      if (*abort_flag != 0) {
        return false;
      }
      if (clock64() - started > kWaitLimitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Bounded wait that never makes its caller leave: when it runs out it flags the CTA, and once the CTA is flagged it
// returns at once.
__device__ __forceinline__ void mbar_wait_through(std::uint32_t bar, std::uint32_t parity,
                                                  volatile std::uint32_t *abort_flag) {
  if (mbar_try_wait(bar, parity) || *abort_flag != 0) {
    return;
  }
  const long long started = clock64();
  std::uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255U) == 0) {
      if (*abort_flag != 0) {
        return;
      }
      if (clock64() - started > kWaitLimitCycles) {
        *abort_flag = 1;
        return;
      }
    }
  }
}

// One lane of the (converged) warp, the same one every time.
__device__ __forceinline__ bool elect_one() {
  std::uint32_t chosen;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "elect.sync _|p, 0xFFFFFFFF;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(chosen));
  return chosen != 0;
}

__device__ __forceinline__ void tma_load_2d(std::uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                            std::uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                   "r"(dst),
               "l"(reinterpret_cast<std::uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tma_load_3d(std::uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            std::uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::
          "r"(dst),
      "l"(reinterpret_cast<std::uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

// ---- two-CTA (cta_group::2) helpers: the pair's even CTA leads -------------------------------------------
__device__ __forceinline__ std::uint32_t cluster_rank() {
  std::uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}

// shared::cluster address of `addr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster
__device__ __forceinline__ std::uint32_t map_to_rank(std::uint32_t addr, std::uint32_t rank) {
  std::uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void mbar_arrive_cluster(std::uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}

// arrive that publishes this thread's earlier writes (also those into the partner's shared memory) to the cluster
__device__ __forceinline__ void mbar_arrive_cluster_release(std::uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;\n" ::: "memory"); }

// bulk copy from this CTA's shared memory into another CTA of the cluster; the bytes count on a barrier there
__device__ __forceinline__ void bulk_copy_to_cluster(std::uint32_t cluster_dst, std::uint32_t cta_src,
                                                     std::uint32_t bytes, std::uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   cluster_dst),
               "r"(cta_src), "r"(bytes), "r"(cluster_bar)
               : "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// TMA tiled store shared -> global (bulk async group of the issuing thread)
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int c0, int c1, int c2, std::uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];\n" ::"l"(
                   reinterpret_cast<std::uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// the stores of this thread have read their shared-memory source
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// the stores of this thread are complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

// TMA tiled load issued by either CTA of a pair into its own shared memory; the bytes are counted on the
// leader's barrier (`leader_bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(std::uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 std::uint32_t leader_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
               "%3}], [%4];\n" ::"r"(dst),
               "l"(reinterpret_cast<std::uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar)
               : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(std::uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2,
                                                 std::uint32_t leader_bar) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
               "%3, %4}], [%5];\n" ::"r"(dst),
               "l"(reinterpret_cast<std::uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(leader_bar)
               : "memory");
}

__device__ __forceinline__ void umma_ss_pair(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                             std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void umma_ts_pair(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint64_t b_desc,
                                             std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}

// completion of all earlier pair MMAs arrives on a barrier given by its shared::cluster address
__device__ __forceinline__ void umma_commit_pair(std::uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(cluster_bar)
               : "memory");
}

// 32-byte global load (sm_100) into two 16-byte halves
__device__ __forceinline__ void ld_global_v8(const void *src, uint4 &lo, uint4 &hi) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
               : "l"(src));
}
// 32-byte global store (sm_100): one instruction per sector instead of two
__device__ __forceinline__ void st_global_v8(void *dst, const std::uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
// lbo / sbo in bytes (the field drops the low four bits).
__device__ __forceinline__ std::uint64_t smem_desc(std::uint32_t addr, std::uint32_t lbo, std::uint32_t sbo) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((addr & 0x3FFFFU) >> 4);
  d |= static_cast<std::uint64_t>((lbo >> 4) & 0x3FFFU) << 16;
  d |= static_cast<std::uint64_t>((sbo >> 4) & 0x3FFFU) << 32;
  d |= static_cast<std::uint64_t>(1) << 46; // version
  d |= static_cast<std::uint64_t>(2) << 61; // SWIZZLE_128B
  return d;
}

// Instruction descriptor: BF16 x BF16 -> FP32; M = 128 for one CTA, 256 for a pair.
__host__ __device__ constexpr std::uint32_t instr_desc(int m, int n, bool b_mn_major) {
  return (1U << 4) | (1U << 7) | (1U << 10) | (b_mn_major ? (1U << 16) : 0U) |
         (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_ss(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                        std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void umma_ts(std::uint32_t d_tmem, std::uint32_t a_tmem, std::uint64_t b_desc,
                                        std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
               : "memory");
}

__device__ __forceinline__ void umma_commit(std::uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(std::uint32_t taddr, std::uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                 "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                 "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                 "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_st32(std::uint32_t taddr, const std::uint32_t (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
               "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
               "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]),
               "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
               "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// 1 / (1 + e^-x) = 0.5 tanh(x / 2) + 0.5 through one tanh.approx (absolute error about 2.5e-4): half the
// special-function work of the form below, for outputs that are rounded to BF16 (spacing 4e-3 near 1) anyway
__device__ __forceinline__ float sigmoid_for_bf16(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(t) : "f"(0.5F * x));
  return fmaf(0.5F, t, 0.5F);
}

// 1 / (1 + e^-x) through ex2 and an approximate reciprocal (relative error ~1e-6, far below BF16 resolution)
__device__ __forceinline__ float fast_sigmoid(float x) {
  return __fdividef(1.0F, 1.0F + fast_exp2(x * -1.4426950408889634F));
}

__device__ __forceinline__ std::uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const std::uint32_t *>(&v);
}

// ---- append: K and V of this chunk into the cache -----------------------------------------------------
// For FP32 activations it also rounds the queries to BF16.  There is no workspace on this path, so the BF16 copy of
// the Q tile of (tile, head) is parked in the first half of that tile's own rows of the output buffer: the attention
// kernel loads it from there with TMA at the start of the tile and overwrites it with the FP32 result at its end.
template <bool F32>
__global__ void __launch_bounds__(256) prefill_append_kernel(const void *key, const void *value,
                                                             __nv_bfloat16 *cache, std::uint32_t tokens,
                                                             std::uint32_t past, std::uint32_t max_ctx,
                                                             std::uint32_t kv_heads, const float *query,
                                                             void *q_parking, std::uint32_t q_tokens,
                                                             std::uint32_t q_heads, std::uint32_t out_heads,
                                                             std::uint32_t out_head_offset) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  // one thread per 8 elements: [plane][token][kv head][32 pieces of 8]
  const std::size_t pieces = static_cast<std::size_t>(tokens) * kv_heads * 32;
  const std::size_t id = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= 2 * pieces) {
    if constexpr (F32) {
      const std::size_t q_id = id - 2 * pieces;
      if (q_id < static_cast<std::size_t>(q_tokens) * q_heads * 32) {
        const std::uint32_t piece = static_cast<std::uint32_t>(q_id % 32);
        const std::uint32_t head = static_cast<std::uint32_t>((q_id / 32) % q_heads);
        const std::size_t token = q_id / (32 * static_cast<std::size_t>(q_heads));
        const float *src = query + (token * q_heads + head) * kHeadDim + piece * 8;
        const float4 a = *reinterpret_cast<const float4 *>(src);
        const float4 b = *reinterpret_cast<const float4 *>(src + 4);
        uint4 raw;
        raw.x = pack_bf16(a.x, a.y);
        raw.y = pack_bf16(a.z, a.w);
        raw.z = pack_bf16(b.x, b.y);
        raw.w = pack_bf16(b.z, b.w);
        unsigned char *row = static_cast<unsigned char *>(q_parking) +
                             (token * out_heads + out_head_offset + head) * (kHeadDim * 4);
        *reinterpret_cast<uint4 *>(row + piece * 16) = raw;
      }
    }
    return;
  }
  const bool is_value = id >= pieces;
  const std::size_t local = is_value ? id - pieces : id;
  const std::uint32_t piece = static_cast<std::uint32_t>(local % 32);
  const std::uint32_t head = static_cast<std::uint32_t>((local / 32) % kv_heads);
  const std::uint32_t token = static_cast<std::uint32_t>(local / (32 * kv_heads));
  const std::size_t src = (static_cast<std::size_t>(token) * kv_heads + head) * kHeadDim + piece * 8;
  const void *base = is_value ? value : key;
  uint4 raw;
  if constexpr (F32) {
    const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + src);
    const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + src + 4);
    raw.x = pack_bf16(a.x, a.y);
    raw.y = pack_bf16(a.z, a.w);
    raw.z = pack_bf16(b.x, b.y);
    raw.w = pack_bf16(b.z, b.w);
  } else {
    raw = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(base) + src);
  }
  const std::size_t plane = static_cast<std::size_t>(kv_heads) * max_ctx * kHeadDim;
  const std::size_t dst = (is_value ? plane : 0) + (static_cast<std::size_t>(head) * max_ctx + past + token) * kHeadDim +
                          piece * 8;
  *reinterpret_cast<uint4 *>(cache + dst) = raw;
}

// ---- attention ----------------------------------------------------------------------------------------
// One persistent CTA per SM walks its share of the (query tile, head) list; the list is sorted by length and
// dealt out in a snake so that every CTA gets about the same number of key blocks.
struct TileWalk {
  std::uint32_t tiles, heads, total, stride, cta, iteration;
  __device__ TileWalk(std::uint32_t tiles_, std::uint32_t heads_, std::uint32_t stride_, std::uint32_t cta_)
      : tiles(tiles_), heads(heads_), total(tiles_ * heads_), stride(stride_), cta(cta_), iteration(0) {}
  // position in the length-sorted list, or total when the walk is over
  __device__ std::uint32_t position() const {
    const std::uint32_t p = iteration * stride + ((iteration & 1U) ? stride - 1 - cta : cta);
    return p < total ? p : total;
  }
  __device__ bool done() const { return position() >= total; }
  __device__ std::uint32_t head() const { return position() % heads; }
  __device__ std::uint32_t tile() const { return tiles - 1 - position() / heads; } // long tiles first
  __device__ void next() { ++iteration; }
};

// Pair == true runs two CTAs of a cluster as one tcgen05 cta_group::2 unit: they take two query heads of the same
// KV head at the same query tile, the even CTA issues every MMA for both (M = 256), and each CTA loads only half
// of every K and V block (the MMA reads the B operand from both CTAs' shared memory).  That halves the bytes an
// SM pulls from L2 per block.  Every TMA load has one destination CTA; the completion signals that both CTAs need
// are two plain tcgen05.commit instructions, one per CTA's barrier.
//
// Split == true is for launches with so few (tile, head) items that half of the SMs would idle (a 512-token chunk
// against a long past): the two CTAs of a cluster take the same item and each runs the ordinary single-CTA loop
// over half of its key blocks; at the end the second CTA ships its unnormalised O tile and its (maximum, row sum)
// into the first one's ring through distributed shared memory, and the first merges the two and writes the tile.
// One item per cluster, so the ring is free when the partial arrives.
constexpr int kLandingPitch = kHeadDim * 4 + 16;                 // bytes per row of a partial O tile in the ring
constexpr int kLandingMeta = kTileRows * kLandingPitch;          // then [group][row] maximum, [group][row] row sum
constexpr int kLandingBytes = kLandingMeta + 4 * kTileRows * 4;
static_assert(kLandingBytes <= kSlots * kSlotBytes && kLandingBytes % 16 == 0, "partial tile must fit in the ring");

template <bool F32, bool Pair, bool Split>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_attention_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                             const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap k_new_map,
                             const __grid_constant__ CUtensorMap v_new_map, const PrefillParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const std::uint32_t base = smem_u32(smem); // the 128-byte swizzle needs 1 KiB alignment; checked below
  const std::uint32_t q_smem = base;
  const std::uint32_t ring = base + kRingOffset;
  const std::uint32_t bars = base + kBarrierOffset;
  volatile std::uint32_t *tmem_slot = reinterpret_cast<volatile std::uint32_t *>(smem + kBarrierOffset + kBarCount * 8);
  volatile std::uint32_t *abort_flag = tmem_slot + 1;
  auto bar = [&](int index) { return bars + static_cast<std::uint32_t>(index) * 8U; };

#ifdef RIB200_TRACE
  const long long cta_started = global_ns();
  std::uint32_t traced_blocks = 0;
#endif
  const int warp = __shfl_sync(0xFFFFFFFFU, threadIdx.x >> 5, 0); // a value the compiler knows to be warp-uniform
  const int lane = threadIdx.x & 31;
  // A cluster is a pair of heads, a split of one item, or both: CTAs 0, 1 the pair that takes the first half of
  // the keys, CTAs 2, 3 the pair that takes the second half.
  constexpr bool kCluster = Pair || Split;
  constexpr std::uint32_t kClusterSize = (Pair ? 2U : 1U) * (Split ? 2U : 1U);
  const std::uint32_t cta = kCluster ? cluster_rank() : 0U;
  const std::uint32_t rank = Pair ? cta & 1U : 0U;                  // place in the pair: 0 leads it
  const std::uint32_t lead_cta = Pair ? cta & ~1U : cta;            // cluster rank of the pair's leader
  const std::uint32_t half = Split ? (Pair ? cta >> 1 : cta) : 0U;  // which half of the keys
  const std::uint32_t half_stride = Pair ? 2U : 1U;                 // cluster ranks between the two halves
  const std::uint32_t unit = blockIdx.x / kClusterSize;             // index of this cluster among its peers
  const std::uint32_t units = gridDim.x / kClusterSize;
  constexpr std::uint32_t kRowThreads = Pair ? 2 * kSoftmaxThreads : kSoftmaxThreads; // softmax threads per unit
  // barriers every softmax thread of the unit arrives on live in the leader
  auto arrive_on_leader = [&](int index) {
    if constexpr (Pair) {
      mbar_arrive_cluster(map_to_rank(bar(index), lead_cta));
    } else {
      mbar_arrive(bar(index));
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(bar(kBarQFull), 1);
    mbar_init(bar(kBarQFree), 1);
    mbar_init(bar(kBarDrain), 1);
    mbar_init(bar(kBarPeerFull), 1);
    mbar_init(bar(kBarPeerFree), kSoftmaxThreads);
    mbar_init(bar(kBarStoresDone), 1);
    mbar_init(bar(kBarOFree), kRowThreads);
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(bar(kBarFull + s), 1);
      mbar_init(bar(kBarEmpty + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(kBarSFull + b), 1);
      mbar_init(bar(kBarPFull + b), kRowThreads);
      mbar_init(bar(kBarPvDone + b), 1);
    }
    *abort_flag = (base & 1023U) != 0 ? 1U : 0U; // a misaligned window would scramble every tile: give up cleanly
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if constexpr (kCluster) {
    cluster_sync_all(); // the partner's barriers exist before anything arrives on them
  }
  // From here the producer warp starts its first loads; the other warps take the SM's tensor memory meanwhile
  // (the allocation takes about as long as those loads) and meet on a barrier of their own before they use it.
  if (warp != kProducerWarp) {
    if (warp == kMmaWarp) {
      // the whole tensor memory of the SM: O (256 columns) + two score tiles (128 each)
      if constexpr (Pair) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(
                         smem_u32(const_cast<std::uint32_t *>(tmem_slot)))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
      } else {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(
                         smem_u32(const_cast<std::uint32_t *>(tmem_slot)))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
      }
    }
    tcgen05_fence_before();
    asm volatile("bar.sync 3, %0;\n" ::"n"(kThreads - 32) : "memory");
    tcgen05_fence_after();
  }
  if constexpr (Split) {
    if (half == 0 && threadIdx.x == 0) {
      mbar_expect_tx(bar(kBarPeerFull), kLandingBytes); // the partner's partial tile, one bulk copy
    }
  }
  if (threadIdx.x == 0) {
    RIB200_STAMP(0, 14); // set-up done
    RIB200_STAMP_NS(3);
    RIB200_STAMP_CTA2(4);
  }
  const std::uint32_t tmem = *tmem_slot;
  const std::uint32_t tmem_o = tmem;         // columns [0, 256)
  const std::uint32_t tmem_s = tmem + 256;   // two tiles of 128 columns

  // geometry of one tile
  auto tile_rows = [&](std::uint32_t tile) {
    return min(static_cast<std::uint32_t>(kTileRows), p.tokens - tile * kTileRows);
  };
  auto tile_blocks = [&](std::uint32_t tile) {
    return (p.past + tile * kTileRows + tile_rows(tile) - 1) / kBlockKeys + 1; // newest visible key / 128 + 1
  };
  // the key blocks this CTA walks: all of them, or its half in the split form (the hand-over can only start when
  // both halves are done, so equal halves are best)
  // A short item is not worth the hand-over: the first CTA (or pair) of the cluster then walks all of its blocks and
  // the second one sits the item out (it has no other: the split form launches one cluster per item).
  auto split_item = [&](std::uint32_t tile) { return Split && tile_blocks(tile) >= p.split_min_blocks; };
  auto first_block = [&](std::uint32_t tile) {
    return split_item(tile) && half == 1 ? (tile_blocks(tile) + 1) / 2 : 0U;
  };
  auto my_blocks = [&](std::uint32_t tile) {
    const std::uint32_t all = tile_blocks(tile);
    if (!Split) {
      return all;
    }
    if (!split_item(tile)) {
      return half == 0 ? all : 0U;
    }
    return half == 0 ? (all + 1) / 2 : all - (all + 1) / 2;
  };

  if (warp == kProducerWarp) {
    // ================= producer =================
    if (lane == 0) {
      // Key blocks that lie wholly inside this chunk are read from the BF16 key / value inputs, so they need
      // nothing from the append kernel that precedes this launch; the first block that needs cache rows of this
      // chunk (a block that straddles the past, or any block when the inputs are FP32) waits for that kernel.
      bool append_done = false;
      auto wait_for_append = [&] {
        if (!append_done) {
          asm volatile("griddepcontrol.wait;\n" ::: "memory");
          append_done = true;
        }
      };
      // In-kernel append.  A key block read from the inputs is also this chunk's contribution to the cache: the
      // CTA that serves the first query head of the KV group, on the tile whose last block it is, writes the
      // slot back to the cache with a TMA store (same box, so the swizzled slot is exactly its source) once the
      // MMAs have consumed it, i.e. when the slot's turn to be refilled comes, or at the end of the walk.
      // pending[slot]: bit 31 set | bit 30 value | bit 29 half | bits 16-23 KV head | bits 0-15 block
      std::uint32_t pending[kSlots];
      for (std::uint32_t i = 0; i < kSlots; ++i) {
        pending[i] = 0;
      }
      auto store_slot = [&](std::uint32_t slot) {
        const std::uint32_t entry = pending[slot];
        pending[slot] = 0;
        const bool is_value = (entry >> 30) & 1U;
        const std::uint32_t half = (entry >> 29) & 1U;
        const int kv = static_cast<int>((entry >> 16) & 0xFFU);
        const int key0 = static_cast<int>((entry & 0xFFFFU) * kBlockKeys);
        const std::uint32_t src = ring + slot * kSlotBytes;
        if constexpr (Pair) {
          if (is_value) {
            for (int b = 0; b < 2; ++b) {
              tma_store_3d(&v_map, static_cast<int>(rank * 128 + b * kBoxCols), key0, kv, src + b * kKeyBoxBytes);
            }
          } else {
            for (int b = 0; b < 4; ++b) {
              tma_store_3d(&k_map, b * kBoxCols, key0 + static_cast<int>(rank * kHalfKeys), kv,
                           src + b * kSlotBoxBytes);
            }
          }
        } else {
          if (is_value) {
            for (int b = 0; b < 4; ++b) {
              tma_store_3d(&v_map, b * kBoxCols, key0 + static_cast<int>(half * kHalfKeys), kv,
                           src + b * kSlotBoxBytes);
            }
          } else {
            for (int b = 0; b < 2; ++b) {
              tma_store_3d(&k_map, static_cast<int>((half * 2 + b) * kBoxCols), key0, kv, src + b * kKeyBoxBytes);
            }
          }
        }
        tma_store_commit();
        tma_store_wait_read(); // the slot may be overwritten now
      };
      std::uint32_t n = 0; // running slot number; the MMA warp walks the same sequence
      bool ok = *abort_flag == 0;
      for (TileWalk walk(p.tiles, Pair ? p.query_heads / 2 : p.query_heads, units, unit); ok && !walk.done(); walk.next()) {
        const std::uint32_t head = Pair ? walk.head() * 2 + rank : walk.head();
        const std::uint32_t kv_head = head / p.group;
        const std::uint32_t row0 = walk.tile() * kTileRows;
        const std::uint32_t all_blocks = tile_blocks(walk.tile());
        const std::uint32_t block0 = first_block(walk.tile()); // this CTA walks blocks block0 .. block0 + blocks - 1
        const std::uint32_t blocks = my_blocks(walk.tile());
        if (Split && blocks == 0) {
          continue; // the item is left to the first half of the cluster
        }
        if (walk.iteration > 0) {
          // the previous tile's last score product has finished reading Q
          ok = mbar_wait(bar(kBarQFree), (walk.iteration - 1) & 1U, abort_flag);
          if (!ok) {
            break;
          }
        }
        if constexpr (F32) {
          // the BF16 queries wait in the output buffer, where the kernel in front of this one parked them:
          // q_map is [256][output heads][token] there
          wait_for_append();
          const int parked_head = static_cast<int>(p.output_head_offset + head);
          if constexpr (Pair) {
            if (rank == 0) {
              mbar_expect_tx(bar(kBarQFull), 2 * kQBytes);
            }
            const std::uint32_t leader_bar = map_to_rank(bar(kBarQFull), lead_cta);
            for (int b = 0; b < 4; ++b) {
              tma_load_3d_pair(q_smem + b * kQBoxBytes, &q_map, b * kBoxCols, parked_head, static_cast<int>(row0),
                               leader_bar);
            }
          } else {
            mbar_expect_tx(bar(kBarQFull), kQBytes);
            for (int b = 0; b < 4; ++b) {
              tma_load_3d(q_smem + b * kQBoxBytes, &q_map, b * kBoxCols, parked_head, static_cast<int>(row0),
                          bar(kBarQFull));
            }
          }
        } else {
          if constexpr (Pair) {
            if (rank == 0) {
              mbar_expect_tx(bar(kBarQFull), 2 * kQBytes); // both CTAs' Q tiles count on the leader's barrier
            }
            const std::uint32_t leader_bar = map_to_rank(bar(kBarQFull), lead_cta);
            for (int b = 0; b < 4; ++b) {
              tma_load_2d_pair(q_smem + b * kQBoxBytes, &q_map, static_cast<int>(head * kHeadDim + b * kBoxCols),
                               static_cast<int>(row0), leader_bar);
            }
          } else {
            mbar_expect_tx(bar(kBarQFull), kQBytes);
            for (int b = 0; b < 4; ++b) {
              tma_load_2d(q_smem + b * kQBoxBytes, &q_map, static_cast<int>(head * kHeadDim + b * kBoxCols),
                          static_cast<int>(row0), bar(kBarQFull));
            }
          }
        }
        // K travels as two slots per block split by head dims (128 keys x 128 dims each, so that one MMA spans
        // all 128 keys); V as two slots split by keys (64 keys x 256 dims each).
        const bool appends = !F32 && head % p.group == (Pair ? rank : 0U); // serves the group's first head
        auto load_half = [&](bool is_value, std::uint32_t block, std::uint32_t half) {
          const std::uint32_t slot = n % kSlots;
          if (n >= kSlots) {
            if (!mbar_wait(bar(kBarEmpty + slot), ((n / kSlots) - 1) & 1U, abort_flag)) {
              return false;
            }
            if (pending[slot] != 0) {
              store_slot(slot);
            }
          }
          const std::uint32_t dst = ring + slot * kSlotBytes;
          const bool from_inputs = !F32 && block * kBlockKeys >= p.past;
          if (!from_inputs && (block + 1) * kBlockKeys > p.past) {
            wait_for_append();
          }
          const CUtensorMap *k_src = from_inputs ? &k_new_map : &k_map;
          const CUtensorMap *v_src = from_inputs ? &v_new_map : &v_map;
          const int block_key0 = static_cast<int>(block * kBlockKeys - (from_inputs ? p.past : 0U));
          if (appends && from_inputs && block + 1 == all_blocks) {
            pending[slot] = 0x80000000U | (is_value ? 0x40000000U : 0U) | (half << 29) | (kv_head << 16) | block;
          }
          if constexpr (Pair) {
            // one slot per block and operand: this CTA's 64 keys of K (all dims), or its 128 dims of V (all keys)
            if (rank == 0) {
              mbar_expect_tx(bar(kBarFull + slot), 2 * kSlotBytes);
            }
            const std::uint32_t leader_bar = map_to_rank(bar(kBarFull + slot), lead_cta);
            const int key0 = block_key0;
            if (is_value) {
              for (int b = 0; b < 2; ++b) {
                tma_load_3d_pair(dst + b * kKeyBoxBytes, v_src, static_cast<int>(rank * 128 + b * kBoxCols), key0,
                                 static_cast<int>(kv_head), leader_bar);
              }
            } else {
              for (int b = 0; b < 4; ++b) {
                tma_load_3d_pair(dst + b * kSlotBoxBytes, k_src, b * kBoxCols,
                                 key0 + static_cast<int>(rank * kHalfKeys), static_cast<int>(kv_head), leader_bar);
              }
            }
            ++n;
            return true;
          }
          mbar_expect_tx(bar(kBarFull + slot), kSlotBytes);
          if (is_value) {
            const int key0 = block_key0 + static_cast<int>(half * kHalfKeys);
            for (int b = 0; b < 4; ++b) {
              tma_load_3d(dst + b * kSlotBoxBytes, v_src, b * kBoxCols, key0, static_cast<int>(kv_head),
                          bar(kBarFull + slot));
            }
          } else {
            const int key0 = block_key0;
            for (int b = 0; b < 2; ++b) {
              tma_load_3d(dst + b * kKeyBoxBytes, k_src, static_cast<int>((half * 2 + b) * kBoxCols), key0,
                          static_cast<int>(kv_head), bar(kBarFull + slot));
            }
          }
          ++n;
          return true;
        };
        constexpr std::uint32_t kParts = Pair ? 1 : 2; // ring slots per block and operand
        for (std::uint32_t h = 0; ok && h < kParts && blocks > 0; ++h) {
          ok = load_half(false, block0, h);
        }
        for (std::uint32_t j = 0; ok && j < blocks; ++j) {
          for (std::uint32_t h = 0; ok && h < kParts && j + 1 < blocks; ++h) {
            ok = load_half(false, block0 + j + 1, h);
          }
          for (std::uint32_t h = 0; ok && h < kParts; ++h) {
            ok = load_half(true, block0 + j, h);
          }
        }
      }
      // slots still waiting to be written back, oldest first (its MMAs finish first): the last fill of slot s was
      // number m, m % kSlots == s
      for (std::uint32_t back = std::min<std::uint32_t>(kSlots, n); ok && back >= 1; --back) {
        const std::uint32_t m = n - back;
        const std::uint32_t slot = m % kSlots;
        if (pending[slot] != 0) {
          ok = mbar_wait(bar(kBarEmpty + slot), (m / kSlots) & 1U, abort_flag);
          if (ok) {
            store_slot(slot);
          }
        }
      }
      if constexpr (Split) {
        mbar_arrive(bar(kBarStoresDone)); // every write-back has read its slot: the ring may hold the partial tile
      }
      tma_store_wait_all();
      // this grid never completes before the append kernel has: work queued behind it sees the cache rows
      wait_for_append();
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issue =================
    // The whole warp walks the loops, so that control flow, ring positions and descriptors are the same in every
    // lane and can live in uniform registers (where tcgen05.mma takes its operands from); one elected lane issues
    // the MMAs and the commits.  A wait that runs out flags the CTA, and from then on nothing waits: the warp runs
    // through its remaining tiles on stale operands rather than leave a loop early.
    if (!Pair || rank == 0) {
      const bool leader = elect_one();
      constexpr int kUnitRows = Pair ? 2 * kTileRows : kTileRows;
      constexpr std::uint32_t kIdescQk = instr_desc(kUnitRows, kBlockKeys, false);
      constexpr std::uint32_t kIdescPv = instr_desc(kUnitRows, kHeadDim, true);
      // Descriptors are built once; inside the loops only a constant is added to the address field.
      const std::uint64_t q_desc = smem_desc(q_smem, 16, 1024);
      const std::uint64_t k_desc = smem_desc(ring, 16, 1024); // K-major, 8-row groups 1 KiB apart
      // dim-major V: 64-dim boxes of 64 keys (8 KiB) in the single-CTA form, of 128 keys (16 KiB) in the pair form
      const std::uint64_t v_desc = smem_desc(ring, Pair ? kKeyBoxBytes : kSlotBoxBytes, 1024);
      const std::uint32_t remote_bars = Pair ? map_to_rank(bars, lead_cta + 1) : 0U;
      const std::uint32_t local_bars = Pair ? map_to_rank(bars, lead_cta) : bars;
      // completion of everything issued so far, signalled to this CTA and, in a pair, to the partner as well
      auto commit = [&](std::uint32_t index) {
        if (leader) {
          if constexpr (Pair) {
            umma_commit_pair(local_bars + index * 8U);
            umma_commit_pair(remote_bars + index * 8U);
          } else {
            umma_commit(bars + index * 8U);
          }
        }
      };
      auto wait = [&](std::uint32_t index, std::uint32_t parity) {
        mbar_wait_through(bars + index * 8U, parity, abort_flag);
        tcgen05_fence_after();
      };
      std::uint32_t slot = 0;       // ring position: the producer walks the same sequence
      std::uint32_t slot_parity = 0;
      auto next_slot = [&] {
        if (++slot == kSlots) {
          slot = 0;
          slot_parity ^= 1U;
        }
      };
      std::uint32_t g0 = 0; // running key-block number of the tile's first block (S buffer = block & 1)
      for (TileWalk walk(p.tiles, Pair ? p.query_heads / 2 : p.query_heads, units, unit); !walk.done(); walk.next()) {
        const std::uint32_t blocks = my_blocks(walk.tile());
        if (Split && blocks == 0) {
          continue;
        }
        wait(kBarQFull, walk.iteration & 1U);
        // S[g & 1] = Q K_block^T.  Pair form: one slot, each CTA holding 64 of the block's 128 keys with all 256
        // dims in four 64-dim boxes.  Single form: two slots, each holding all 128 keys for half of the dims.
        auto issue_qk = [&](std::uint32_t j) {
          const std::uint32_t g = g0 + j;
          if (walk.iteration == 0) {
            RIB200_STAMP(j, 0); // QK issue begins
          }
          const std::uint32_t d = tmem_s + (g & 1U) * kBlockKeys;
          if constexpr (Pair) {
            wait(kBarFull + slot, slot_parity);
            const std::uint64_t b0 = k_desc + ((slot * kSlotBytes) >> 4);
            if (leader) {
#pragma unroll
              for (int ks = 0; ks < 16; ++ks) {
                const std::uint32_t a_off = ((ks >> 2) * kQBoxBytes + (ks & 3) * 32) >> 4;
                const std::uint32_t b_off = ((ks >> 2) * kSlotBoxBytes + (ks & 3) * 32) >> 4;
                umma_ss_pair(d, q_desc + a_off, b0 + b_off, kIdescQk, ks > 0 ? 1U : 0U);
              }
            }
            commit(kBarEmpty + slot);
            next_slot();
          } else {
#pragma unroll
            for (std::uint32_t half = 0; half < 2; ++half) {
              wait(kBarFull + slot, slot_parity);
              const std::uint64_t a0 = q_desc + ((half * 2 * kQBoxBytes) >> 4);
              const std::uint64_t b0 = k_desc + ((slot * kSlotBytes) >> 4);
              if (leader) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                  const std::uint32_t a_off = ((ks >> 2) * kQBoxBytes + (ks & 3) * 32) >> 4;
                  const std::uint32_t b_off = ((ks >> 2) * kKeyBoxBytes + (ks & 3) * 32) >> 4;
                  umma_ss(d, a0 + a_off, b0 + b_off, kIdescQk, (half > 0 || ks > 0) ? 1U : 0U);
                }
              }
              commit(kBarEmpty + slot);
              next_slot();
            }
          }
          commit(kBarSFull + (g & 1U));
          if (j + 1 == blocks) {
            commit(kBarQFree); // the tile's last read of Q
          }
          if (walk.iteration == 0) {
            RIB200_STAMP(j, 1); // QK issued
          }
        };
        if (blocks > 0) {
          issue_qk(0);
        }
        for (std::uint32_t j = 0; j < blocks; ++j) {
          const std::uint32_t g = g0 + j;
          if (j + 1 < blocks) {
            issue_qk(j + 1);
          }
          if (walk.iteration == 0) {
            RIB200_STAMP(j, 2); // waiting for P
          }
          wait(kBarPFull + (g & 1U), (g >> 1) & 1U);
          if (j == 0 && walk.iteration > 0) {
            // the first PV of a tile overwrites O: the previous tile's epilogue must have read it
            wait(kBarOFree, (walk.iteration - 1) & 1U);
          }
          if (walk.iteration == 0) {
            RIB200_STAMP(j, 3); // P arrived
          }
          // O += P_j V_j, P from tensor memory (BF16 pairs: 16 keys = 8 columns), V dim-major from the ring
          if constexpr (Pair) {
            // one slot: each CTA holds 128 of the 256 dims for all 128 keys
            wait(kBarFull + slot, slot_parity);
            const std::uint64_t b0 = v_desc + ((slot * kSlotBytes) >> 4);
            if (leader) {
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {
                const std::uint32_t a = tmem_s + (g & 1U) * kBlockKeys + ks * 8;
                umma_ts_pair(tmem_o, a, b0 + ((ks * 2048) >> 4), kIdescPv, (j > 0 || ks > 0) ? 1U : 0U);
              }
            }
            commit(kBarEmpty + slot);
            next_slot();
          } else {
#pragma unroll
            for (std::uint32_t half = 0; half < 2; ++half) {
              wait(kBarFull + slot, slot_parity);
              const std::uint64_t b0 = v_desc + ((slot * kSlotBytes) >> 4);
              if (leader) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  const std::uint32_t a = tmem_s + (g & 1U) * kBlockKeys + half * 32 + ks * 8;
                  umma_ts(tmem_o, a, b0 + ((ks * 2048) >> 4), kIdescPv, (j > 0 || half > 0 || ks > 0) ? 1U : 0U);
                }
              }
              commit(kBarEmpty + slot);
              next_slot();
            }
          }
          commit(kBarPvDone + (g & 1U));
          if (walk.iteration == 0) {
            RIB200_STAMP(j, 4); // PV issued
          }
        }
        g0 += blocks;
      }
      if (*abort_flag != 0) {
        // after giving up: every MMA issued above has left the tensor pipe before tensor memory is freed
        commit(kBarDrain);
        mbar_wait_through(bars + kBarDrain * 8U, 0, abort_flag);
      }
    }
  } else {
    // ================= softmax, correction, epilogue =================
    // Two groups of four warps.  A thread owns one query row (tensor-memory lane 32 * (warp % 4) + lane) and the
    // 64 score columns of its group, so two threads share a row; they agree on the row maximum through shared
    // memory once per block and keep separate partial row sums until the end of the tile.
    const int group = warp >> 2;
    const std::uint32_t row = (warp & 3) * 32 + lane;
    const std::uint32_t lane_base = static_cast<std::uint32_t>((warp & 3) * 32) << 16;
    float *exchange = reinterpret_cast<float *>(smem + kExchangeOffset); // [parity][group][row]
    bool ok = *abort_flag == 0;
    std::uint32_t g0 = 0;

    for (TileWalk walk(p.tiles, Pair ? p.query_heads / 2 : p.query_heads, units, unit); ok && !walk.done(); walk.next()) {
      const std::uint32_t head = Pair ? walk.head() * 2 + rank : walk.head();
      const std::uint32_t row0 = walk.tile() * kTileRows;
      const std::uint32_t rows = tile_rows(walk.tile());
      const std::uint32_t blocks = my_blocks(walk.tile());
      const std::uint32_t block0 = first_block(walk.tile());
      const bool split_here = split_item(walk.tile());
      if (Split && blocks == 0) {
        continue;
      }
      const std::uint32_t q_pos = p.past + row0 + row; // position of this row's query (rows past the tile are idle)

      float m_used = -INFINITY; // maximum the exponentials are taken against (scaled, base 2); same in both groups
      float l_sum = 0.0F;       // this thread's share of the row sum
      for (std::uint32_t j = 0; j < blocks && ok; ++j) {
        const std::uint32_t g = g0 + j;
        const std::uint32_t buf = g & 1U;
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 8); // softmax waits for S
        }
        ok = mbar_wait(bar(kBarSFull + buf), (g >> 1) & 1U, abort_flag);
        ok = __all_sync(0xFFFFFFFFU, ok);
        if (!ok) {
          break;
        }
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 9); // S arrived
        }
        tcgen05_fence_after();
        const std::uint32_t s_addr = tmem_s + lane_base + buf * kBlockKeys;
        // raw scores (unscaled) of this group's 64 columns: both loads are in flight before the single wait
        std::uint32_t xr[2][32];
        tmem_ld32(s_addr + group * 64, xr[0]);
        tmem_ld32(s_addr + group * 64 + 32, xr[1]);
        tmem_wait_ld();
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 10); // S in registers
        }
        float x[64];
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          x[e] = __uint_as_float(xr[e >> 5][e & 31]);
        }
        // causal mask: key position j*128 + c is visible iff <= q_pos (also hides rows the context never held)
        const std::uint32_t key0 = (block0 + j) * kBlockKeys;
        if (key0 + kBlockKeys - 1 > p.past + row0) {
          const int visible = static_cast<int>(q_pos) - static_cast<int>(key0 + group * 64) + 1;
#pragma unroll
          for (int e = 0; e < 64; ++e) {
            if (e >= visible) {
              x[e] = -INFINITY;
            }
          }
        }
        float mx0 = fmaxf(x[0], x[1]);
        float mx1 = fmaxf(x[2], x[3]);
#pragma unroll
        for (int e = 4; e < 64; e += 4) {
          mx0 = fmaxf(mx0, fmaxf(x[e], x[e + 1]));
          mx1 = fmaxf(mx1, fmaxf(x[e + 2], x[e + 3]));
        }
        const float mine = fmaxf(mx0, mx1);
        exchange[(buf * 2 + group) * kTileRows + row] = mine;
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        const float theirs = exchange[(buf * 2 + (group ^ 1)) * kTileRows + row];
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 11); // maxima exchanged
        }
        // the scale is positive: it commutes with the maximum.  A row that sees no key of this block (possible only
        // for the second half of a split item) gets a large negative finite maximum, so that its weights are zeros.
        const float mx = fmaxf(fmaxf(mine, theirs) * kScaleLog2e, -1.0e30F);
        // move the reference maximum only when it fell far behind; block 0 always sets it
        const bool move = mx > m_used + kRescaleThreshold;
        if (__any_sync(0xFFFFFFFFU, move && j > 0)) {
          // rescale this warp's 32 rows of O (this group's 128 columns); PV(j-1) must have landed
          ok = mbar_wait(bar(kBarPvDone + ((g - 1) & 1U)), ((g - 1) >> 1) & 1U, abort_flag);
          ok = __all_sync(0xFFFFFFFFU, ok);
          if (!ok) {
            break;
          }
          tcgen05_fence_after();
          const float factor = move ? exp2f(m_used - mx) : 1.0F;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            std::uint32_t v[32];
            const std::uint32_t o_addr = tmem_o + lane_base + group * 128 + c * 32;
            tmem_ld32(o_addr, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
            }
            tmem_st32(o_addr, v);
          }
          tmem_wait_st();
          l_sum *= factor;
        }
        if (move) {
          m_used = mx;
        }
        // p = 2^(x * scale - m): one FMA and one ex2 per score; four partial sums
        const float neg_m = -m_used;
        float part0 = 0.0F;
        float part1 = 0.0F;
        float part2 = 0.0F;
        float part3 = 0.0F;
        std::uint32_t packed[32];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = fast_exp2(fmaf(x[2 * e], kScaleLog2e, neg_m));
          const float p1 = fast_exp2(fmaf(x[2 * e + 1], kScaleLog2e, neg_m));
          const float p2 = fast_exp2(fmaf(x[2 * e + 2], kScaleLog2e, neg_m));
          const float p3 = fast_exp2(fmaf(x[2 * e + 3], kScaleLog2e, neg_m));
          part0 += p0;
          part1 += p1;
          part2 += p2;
          part3 += p3;
          packed[e] = pack_bf16(p0, p1);
          packed[e + 1] = pack_bf16(p2, p3);
        }
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 12); // exponentials done
        }
        tmem_st32(s_addr + group * 32, packed); // keys 64*group .. +63 are BF16 pairs in columns 32*group .. +31
        l_sum += (part0 + part1) + (part2 + part3);
        tmem_wait_st();
        tcgen05_fence_before();
        arrive_on_leader(kBarPFull + buf);
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(j, 13); // P published
        }
      }
      if (!ok) {
        break;
      }

      // ---- epilogue: out = O / l * sigmoid(gate); each group writes its 128 of the 256 columns ----
      const std::uint32_t g_last = g0 + blocks - 1;
      g0 += blocks;
      const std::size_t out_base =
          (static_cast<std::size_t>(row0 + row) * p.query_heads + head) * kHeadDim + group * 128;
      const std::size_t dst_base =
          (static_cast<std::size_t>(row0 + row) * p.output_heads + p.output_head_offset + head) * kHeadDim +
          group * 128;
      const bool live = row < rows;
      uint4 gate_raw[16]; // BF16 gates of this thread's 128 columns, fetched while the last PV is still running
      if constexpr (!F32) {
        if (live) {
          const uint4 *gp = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.gate) + out_base);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            ld_global_v8(gp + i, gate_raw[i], gate_raw[i + 1]);
          }
        }
      }
      // FP32 gates cannot all wait in registers as the BF16 ones do: the first 32-column piece is fetched here, while
      // the last PV is still running, the other three are pulled into L2 and fetched one piece ahead further down
      float4 gate_now[F32 ? 8 : 1];
      if constexpr (F32) {
        if (live) {
          const float4 *gsrc = reinterpret_cast<const float4 *>(static_cast<const float *>(p.gate) + out_base);
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            ld_global_v8(gsrc + i, *reinterpret_cast<uint4 *>(&gate_now[i]), *reinterpret_cast<uint4 *>(&gate_now[i + 1]));
          }
#pragma unroll
          for (int piece = 1; piece < 4; ++piece) {
            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(gsrc + piece * 8));
          }
        }
      }
      ok = mbar_wait(bar(kBarPvDone + (g_last & 1U)), (g_last >> 1) & 1U, abort_flag);
      ok = __all_sync(0xFFFFFFFFU, ok);
      if (!ok) {
        break;
      }
      tcgen05_fence_after();
      if (threadIdx.x == 0 && walk.iteration == 0) {
        RIB200_STAMP(1, 14); // last PV landed
        RIB200_STAMP_NS(0);
      }
      if constexpr (Split) {
        if (half == 1) {
          // Second half of a split item: the unnormalised O rows, the maximum they are scaled against and the
          // row-sum shares go to this CTA's own ring (its MMAs have left it), and from there to the first CTA's
          // ring in one bulk copy through distributed shared memory, once that CTA's MMAs have left theirs.
          unsigned char *stage = smem + kRingOffset;
          if (threadIdx.x == 0) {
            RIB200_STAMP_CTA2(0); // last PV landed
          }
          ok = mbar_wait(bar(kBarStoresDone), walk.iteration & 1U, abort_flag); // the cache write-backs are out
          ok = __all_sync(0xFFFFFFFFU, ok);
          if (!ok) {
            break;
          }
          if (threadIdx.x == 0) {
            RIB200_STAMP_CTA2(1); // write-backs out
          }
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            std::uint32_t v[32];
            tmem_ld32(tmem_o + lane_base + group * 128 + c * 32, v);
            tmem_wait_ld();
            uint4 *dst = reinterpret_cast<uint4 *>(stage + row * kLandingPitch + (group * 128 + c * 32) * 4);
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              dst[e / 4] = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
            }
          }
          float *meta = reinterpret_cast<float *>(stage + kLandingMeta);
          meta[group * kTileRows + row] = m_used;
          meta[2 * kTileRows + group * kTileRows + row] = l_sum;
          if (threadIdx.x == 0) {
            RIB200_STAMP_CTA2(2); // staged
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
          asm volatile("bar.sync 1, 256;\n" ::: "memory");
          if (threadIdx.x == 0) {
            ok = mbar_wait(bar(kBarPeerFree), walk.iteration & 1U, abort_flag);
            RIB200_STAMP_CTA2(3); // partner's ring free
            if (ok) {
              bulk_copy_to_cluster(map_to_rank(ring, cta - half_stride), ring, kLandingBytes,
                                   map_to_rank(bar(kBarPeerFull), cta - half_stride));
            }
          }
          tcgen05_fence_before();
          arrive_on_leader(kBarOFree);
          continue;
        }
        // first half: every MMA of this CTA has completed, its ring is free for the partner's partial tile
        if (split_here) {
          mbar_arrive_cluster_release(map_to_rank(bar(kBarPeerFree), cta + half_stride));
        }
      }
      // The row sum is the two groups' shares.  They pass through the half of the exchange area that the next
      // block to run (the first of the next tile) does not use; the first barrier makes sure the partner has
      // finished reading this tile's last maximum from it.
      const std::uint32_t sums = ((g0 & 1U) ^ 1U) * 2;
      asm volatile("bar.sync 1, 256;\n" ::: "memory");
      exchange[(sums + group) * kTileRows + row] = l_sum;
      asm volatile("bar.sync 1, 256;\n" ::: "memory");
      float inv = 1.0F / (l_sum + exchange[(sums + (group ^ 1)) * kTileRows + row]);
      float own_weight = 1.0F;  // split form: factors that bring the two halves to a common maximum
      float peer_weight = 0.0F;
      const unsigned char *landed = smem + kRingOffset;
      if (Split && split_here) {
        ok = mbar_wait(bar(kBarPeerFull), walk.iteration & 1U, abort_flag);
        ok = __all_sync(0xFFFFFFFFU, ok);
        if (!ok) {
          break;
        }
        fence_cluster();
        if (threadIdx.x == 0 && walk.iteration == 0) {
          RIB200_STAMP(1, 15); // partner's partial tile landed
          RIB200_STAMP_NS(1);
        }
        const float *meta = reinterpret_cast<const float *>(landed + kLandingMeta);
        const float peer_max = meta[group * kTileRows + row];
        const float peer_sum = meta[2 * kTileRows + row] + meta[3 * kTileRows + row];
        const float both = fmaxf(m_used, peer_max);
        own_weight = exp2f(m_used - both);
        peer_weight = exp2f(peer_max - both);
        inv = 1.0F / (own_weight * (l_sum + exchange[(sums + (group ^ 1)) * kTileRows + row]) + peer_weight * peer_sum);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        std::uint32_t v[32];
        tmem_ld32(tmem_o + lane_base + group * 128 + c * 32, v);
        float4 gate_next[F32 ? 8 : 1];
        if constexpr (F32) {
          if (live && c < 3) {
            const float4 *gsrc =
                reinterpret_cast<const float4 *>(static_cast<const float *>(p.gate) + out_base + (c + 1) * 32);
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
              ld_global_v8(gsrc + i, *reinterpret_cast<uint4 *>(&gate_next[i]),
                           *reinterpret_cast<uint4 *>(&gate_next[i + 1]));
            }
          }
        }
        tmem_wait_ld();
        if (Split && split_here) {
          const float4 *peer = reinterpret_cast<const float4 *>(landed + row * kLandingPitch + (group * 128 + c * 32) * 4);
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float4 pv = peer[e / 4];
            v[e] = __float_as_uint(__uint_as_float(v[e]) * own_weight + pv.x * peer_weight);
            v[e + 1] = __float_as_uint(__uint_as_float(v[e + 1]) * own_weight + pv.y * peer_weight);
            v[e + 2] = __float_as_uint(__uint_as_float(v[e + 2]) * own_weight + pv.z * peer_weight);
            v[e + 3] = __float_as_uint(__uint_as_float(v[e + 3]) * own_weight + pv.w * peer_weight);
          }
        }
        if (c == 3) {
          // O has been read: the next tile's first PV may overwrite it
          tcgen05_fence_before();
          arrive_on_leader(kBarOFree);
        }
        if (live) {
          if constexpr (F32) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              const float4 ga = gate_now[e / 4];
              const float4 gb = gate_now[e / 4 + 1];
              const float gs[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
              std::uint32_t r[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                r[i] = __float_as_uint(__uint_as_float(v[e + i]) * inv * fast_sigmoid(gs[i]));
              }
              st_global_v8(static_cast<float *>(p.output) + dst_base + c * 32 + e, r);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 16) {
              const uint4 ga = gate_raw[c * 4 + e / 8];
              const uint4 gb = gate_raw[c * 4 + e / 8 + 1];
              const std::uint32_t gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
              std::uint32_t ow[8];
#pragma unroll
              for (int h = 0; h < 8; ++h) {
                const float g0f = __uint_as_float(gw[h] << 16);
                const float g1f = __uint_as_float(gw[h] & 0xFFFF0000U);
                const float r0 = __uint_as_float(v[e + 2 * h]) * inv * sigmoid_for_bf16(g0f);
                const float r1 = __uint_as_float(v[e + 2 * h + 1]) * inv * sigmoid_for_bf16(g1f);
                ow[h] = pack_bf16(r0, r1);
              }
              st_global_v8(static_cast<__nv_bfloat16 *>(p.output) + dst_base + c * 32 + e, ow);
            }
          }
        }
        if constexpr (F32) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            gate_now[i] = gate_next[i];
          }
        }
      }
      if (p.peer_count > 0) {
        // Head-sharded form: forward the tile to the other ranks' buffers.  A thread wrote one row's 128 columns;
        // the warp now re-reads its 32 rows (they are in L2) so that every store instruction covers whole
        // contiguous row segments, which is what peer stores over NVLink need to be efficient.
        __syncwarp();
        constexpr int kSegmentBytes = F32 ? 512 : 256;     // this group's share of a row
        constexpr int kChunksPerRow = kSegmentBytes / 16;  // 32 or 16
        constexpr int kRowsPerStep = 32 / kChunksPerRow;   // 1 or 2
        const std::size_t element = F32 ? 4 : 2;
        const std::size_t row_pitch = static_cast<std::size_t>(p.output_heads) * kHeadDim * element;
        const std::size_t column_offset =
            (static_cast<std::size_t>(p.output_head_offset + head) * kHeadDim + group * 128) * element;
        const std::uint32_t chunk = lane % kChunksPerRow;
        const unsigned char *own = static_cast<const unsigned char *>(p.output);
#pragma unroll 4
        for (int step = 0; step < 32 / kRowsPerStep; ++step) {
          const std::uint32_t r = (warp & 3) * 32 + step * kRowsPerStep + lane / kChunksPerRow;
          if (r < rows) {
            const std::size_t at = static_cast<std::size_t>(row0 + r) * row_pitch + column_offset + chunk * 16;
            const uint4 piece = *reinterpret_cast<const uint4 *>(own + at);
#pragma unroll
            for (std::uint32_t d = 0; d < 7; ++d) { // static indices: the pointers stay in the parameter bank
              if (d < p.peer_count) {
                *reinterpret_cast<uint4 *>(static_cast<unsigned char *>(p.peers[d]) + at) = piece;
              }
            }
          }
        }
      }
      if (threadIdx.x == 0 && walk.iteration == 0) {
        RIB200_STAMP(0, 15); // tile written
        RIB200_STAMP_NS(2);
      }
#ifdef RIB200_TRACE
      traced_blocks += blocks;
#endif
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCluster) {
    cluster_sync_all(); // neither CTA leaves (or frees tensor memory) while the other may still use it
  }
  if (threadIdx.x == 0 && *abort_flag != 0) {
    atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
  }
#ifdef RIB200_TRACE
  if (threadIdx.x == 0) {
    const std::uint32_t id = blockIdx.x;
    if (id < 1024) {
      std::uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      g_cta_trace[id * 4 + 0] = cta_started;
      g_cta_trace[id * 4 + 1] = global_ns();
      g_cta_trace[id * 4 + 2] = traced_blocks;
      g_cta_trace[id * 4 + 3] = smid;
    }
  }
#endif
  if (warp == kMmaWarp) {
    tcgen05_fence_after();
    if constexpr (Pair) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
    }
  }
}


// ---- host side ------------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled_entry() {
  static EncodeTiled fn = [] {
    void *entry = nullptr;
    cudaDriverEntryPointQueryResult result{};
    cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result),
            "cuTensorMapEncodeTiled lookup");
    require(entry != nullptr && result == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is unavailable",
            RIB200_STATUS_UNAVAILABLE);
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return fn;
}

CUtensorMap make_map(void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides_bytes,
                     const cuuint32_t *box) {
  CUtensorMap map;
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult rc =
      encode_tiled_entry()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), base, dims,
                           strides_bytes, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  require(rc == CUDA_SUCCESS, "tensor map encoding failed", RIB200_STATUS_CUDA_ERROR);
  return map;
}

template <bool F32, bool Pair, bool Split> void configure_once() {
  static std::once_flag flags[64];
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  std::call_once(flags[device], [] {
    cuda_ok(cudaFuncSetAttribute(prefill_attention_kernel<F32, Pair, Split>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemBytes),
            "prefill attention shared-memory opt-in");
  });
}

// Builds made with -DRIB200_TUNING read two switches from the environment, for A/B timing of the kernel forms:
// RIB200_PREFILL_PAIR=0 keeps every shape on the single-CTA form, RIB200_PREFILL_SPLIT=0 never splits an item
// over two CTA pairs.  The library as shipped has neither switch: both forms are chosen by shape alone.
#ifdef RIB200_TUNING
bool pair_form_enabled() {
  static const bool enabled = [] {
    const char *env = std::getenv("RIB200_PREFILL_PAIR");
    return env == nullptr || env[0] != '0';
  }();
  return enabled;
}
bool split_form_enabled() {
  static const bool enabled = [] {
    const char *env = std::getenv("RIB200_PREFILL_SPLIT");
    return env == nullptr || env[0] != '0';
  }();
  return enabled;
}
#else
constexpr bool pair_form_enabled() { return true; }
constexpr bool split_form_enabled() { return true; }
#endif

template <bool F32, bool Pair, bool Split> void launch(const PrefillArgs &a, cudaStream_t stream) {
  configure_once<F32, Pair, Split>();
  auto *cache = static_cast<__nv_bfloat16 *>(a.kv_cache);
  // The attention kernel itself writes the key blocks that lie wholly inside this chunk into the cache (BF16
  // inputs).  The append kernel covers the rest: every row for FP32 inputs, else the chunk's rows that share a key
  // block with the past.
  const std::uint32_t ragged = a.past_tokens % kBlockKeys == 0 ? 0U : kBlockKeys - a.past_tokens % kBlockKeys;
  const std::uint32_t append_rows = F32 ? a.tokens : std::min<std::uint32_t>(a.tokens, ragged);
  // where this GPU's output tiles go (the head-sharded form writes into a wider buffer at a head offset)
  void *own_output = a.output_count == 0 ? a.output : a.outputs[a.output_self];
  const std::uint32_t out_heads = a.output_count == 0 ? a.query_heads : a.output_heads;
  const std::uint32_t out_head_offset = a.output_count == 0 ? 0U : a.output_head_offset;
  if (append_rows > 0) {
    const std::size_t kv_pieces = static_cast<std::size_t>(append_rows) * a.kv_heads * 32 * 2;
    const std::size_t q_pieces = F32 ? static_cast<std::size_t>(a.tokens) * a.query_heads * 32 : 0; // parked queries
    prefill_append_kernel<F32><<<static_cast<unsigned int>((kv_pieces + q_pieces + 255) / 256), 256, 0, stream>>>(
        a.key, a.value, cache, append_rows, a.past_tokens, a.max_context_tokens, a.kv_heads,
        static_cast<const float *>(a.query), own_output, a.tokens, a.query_heads, out_heads, out_head_offset);
    cuda_ok(cudaGetLastError(), "prefill append launch");
  }

  const std::uint64_t context = static_cast<std::uint64_t>(a.past_tokens) + a.tokens;
  // K / V: [kv head][row < context][256], rows 512 bytes apart, heads max_ctx rows apart.  The single-CTA form
  // loads K in boxes of 128 keys and V in boxes of 64; the pair form the other way round (each CTA takes 64 keys
  // of K and all 128 keys of half of V's dims).
  const cuuint64_t kv_dims[3] = {kHeadDim, context, a.kv_heads};
  const cuuint64_t kv_strides[2] = {kHeadDim * 2, static_cast<cuuint64_t>(a.max_context_tokens) * kHeadDim * 2};
  const cuuint32_t tall_box[3] = {kBoxCols, kBlockKeys, 1};
  const cuuint32_t short_box[3] = {kBoxCols, kHalfKeys, 1};
  const CUtensorMap k_map = make_map(cache, 3, kv_dims, kv_strides, Pair ? short_box : tall_box);
  const CUtensorMap v_map =
      make_map(cache + static_cast<std::size_t>(a.kv_heads) * a.max_context_tokens * kHeadDim, 3, kv_dims, kv_strides,
               Pair ? tall_box : short_box);
  // BF16 key / value inputs, [token][kv head][256]: the same boxes over this chunk's own rows
  CUtensorMap k_new_map = k_map;
  CUtensorMap v_new_map = v_map;
  if (!F32) {
    const cuuint64_t new_dims[3] = {kHeadDim, a.tokens, a.kv_heads};
    const cuuint64_t new_strides[2] = {static_cast<cuuint64_t>(a.kv_heads) * kHeadDim * 2, kHeadDim * 2};
    k_new_map = make_map(const_cast<void *>(a.key), 3, new_dims, new_strides, Pair ? short_box : tall_box);
    v_new_map = make_map(const_cast<void *>(a.value), 3, new_dims, new_strides, Pair ? tall_box : short_box);
  }
  // Q: [token][query_heads * 256] for BF16 activations; for FP32 the BF16 copy parked in the output buffer,
  // [256][output heads][token] with 1024-byte head slots
  CUtensorMap q_map = k_map;
  if (F32) {
    const cuuint64_t q_dims[3] = {kHeadDim, out_heads, a.tokens};
    const cuuint64_t q_strides[2] = {kHeadDim * 4, static_cast<cuuint64_t>(out_heads) * kHeadDim * 4};
    const cuuint32_t q_box[3] = {kBoxCols, 1, kTileRows};
    q_map = make_map(own_output, 3, q_dims, q_strides, q_box);
  } else {
    const cuuint64_t q_dims[2] = {static_cast<cuuint64_t>(a.query_heads) * kHeadDim, a.tokens};
    const cuuint64_t q_strides[1] = {static_cast<cuuint64_t>(a.query_heads) * kHeadDim * 2};
    const cuuint32_t q_box[2] = {kBoxCols, kTileRows};
    q_map = make_map(const_cast<void *>(a.query), 2, q_dims, q_strides, q_box);
  }

  PrefillParams params{};
  params.gate = a.gate;
  if (a.output_count == 0) {
    params.output = a.output;
    params.peer_count = 0;
    params.output_heads = a.query_heads;
    params.output_head_offset = 0;
  } else {
    params.output = a.outputs[a.output_self];
    params.peer_count = 0;
    for (std::uint32_t d = 0; d < a.output_count; ++d) {
      if (d != a.output_self) {
        params.peers[params.peer_count++] = a.outputs[d];
      }
    }
    params.output_heads = a.output_heads;
    params.output_head_offset = a.output_head_offset;
  }
  params.tokens = a.tokens;
  params.past = a.past_tokens;
  params.tiles = (a.tokens + kTileRows - 1) / kTileRows;
  params.query_heads = a.query_heads;
  params.group = a.query_heads / a.kv_heads;
  {
    // every item when already the first tile is long enough to be worth a hand-over, else only the long ones
    const std::uint32_t first_tile_blocks =
        (a.past_tokens + std::min<std::uint32_t>(a.tokens, kTileRows) - 1) / kBlockKeys + 1;
    params.split_min_blocks = first_tile_blocks >= kSplitMinBlocks ? kSplitMinBlocks : kSplitMinBlocksLate;
  }
  params.status = device_status_word();

  cudaLaunchConfig_t config{};
  int device = 0;
  int sm_count = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  cuda_ok(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device), "SM count query");
  const std::uint32_t sms = static_cast<std::uint32_t>(sm_count);
  if (Split) {
    // one item (or pair of heads) per cluster
    config.gridDim = dim3(Pair ? 4 * params.tiles * (a.query_heads / 2) : 2 * params.tiles * a.query_heads, 1, 1);
  } else if (Pair) {
    const std::uint32_t pair_items = params.tiles * (a.query_heads / 2);
    config.gridDim = dim3(2 * std::min<std::uint32_t>(pair_items, sms / 2), 1, 1);
  } else {
    config.gridDim = dim3(std::min<std::uint32_t>(params.tiles * a.query_heads, sms), 1, 1);
  }
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2]{};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = (Pair ? 2 : 1) * (Split ? 2 : 1);
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = 1;
  // attribute 0 (overlap with the append kernel) only when that kernel was launched
  config.attrs = append_rows > 0 ? attributes : attributes + 1;
  config.numAttrs = (Pair || Split ? 1 : 0) + (append_rows > 0 ? 1 : 0);
  cuda_ok(cudaLaunchKernelEx(&config, prefill_attention_kernel<F32, Pair, Split>, q_map, k_map, v_map, k_new_map, v_new_map, params),
          "prefill attention launch");
}

} // namespace

void encode_f32_rows_map(void *map_out, void *base, std::uint64_t row_floats, std::uint64_t rows,
                         std::uint32_t box_floats, std::uint32_t box_rows) {
  static_assert(sizeof(CUtensorMap) == 128, "the opaque tensor-map type of common.hpp has the driver's size");
  const cuuint64_t dims[2] = {row_floats, rows};
  const cuuint64_t strides[1] = {row_floats * sizeof(float)};
  const cuuint32_t box[2] = {box_floats, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = encode_tiled_entry()(static_cast<CUtensorMap *>(map_out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base,
                                           dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  require(rc == CUDA_SUCCESS, "tensor map encoding failed", RIB200_STATUS_CUDA_ERROR);
}

void encode_plain_rows_map(void *map_out, const void *base, bool f32, std::uint64_t row_elements,
                           std::uint64_t row_stride_elements, std::uint64_t rows, std::uint32_t box_elements,
                           std::uint32_t box_rows) {
  const std::uint64_t element = f32 ? 4 : 2;
  require(reinterpret_cast<std::uintptr_t>(base) % 16 == 0 && (row_stride_elements * element) % 16 == 0,
          "rows read through a tensor map must start on 16-byte boundaries");
  const cuuint64_t dims[2] = {row_elements, rows};
  const cuuint64_t strides[1] = {row_stride_elements * element};
  const cuuint32_t box[2] = {box_elements, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = encode_tiled_entry()(
      static_cast<CUtensorMap *>(map_out), f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
      const_cast<void *>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  require(rc == CUDA_SUCCESS, "tensor map encoding failed", RIB200_STATUS_CUDA_ERROR);
}

#ifdef RIB200_TRACE
extern "C" int rib200_debug_read_trace(long long *host, std::size_t count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace, count * sizeof(long long)));
}
extern "C" int rib200_debug_read_cta_trace(long long *host, std::size_t count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_cta_trace, count * sizeof(long long)));
}
#endif

void launch_prefill_attention(const PrefillArgs &args, cudaStream_t stream) {
  require(args.tokens <= 65535U * kTileRows, "prefill attention: too many tokens for one launch");
  // Few items, each with many key blocks (a short chunk against a long past): two CTAs share an item's keys.
  // Otherwise two query heads of one KV head form a pair; an odd group size keeps the single-CTA form.
  int device = 0;
  int sm_count = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  cuda_ok(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device), "SM count query");
  const std::uint32_t tiles = (args.tokens + kTileRows - 1) / kTileRows;
  const std::uint32_t first_tile_blocks =
      (args.past_tokens + std::min<std::uint32_t>(args.tokens, kTileRows) - 1) / kBlockKeys + 1;
  // ... or few items of which only the late ones are long (a rank's slice of the heads of a long prompt): those are
  // split, the short ones are left to one CTA (or pair) of their cluster.
  const std::uint32_t last_tile_blocks = (args.past_tokens + args.tokens - 1) / kBlockKeys + 1;
  const bool split = split_form_enabled() && 2 * tiles * args.query_heads <= static_cast<std::uint32_t>(sm_count) &&
                     (first_tile_blocks >= kSplitMinBlocks || last_tile_blocks >= kSplitMinBlocksLate);
  const bool pair = pair_form_enabled() && (args.query_heads / args.kv_heads) % 2 == 0;
  auto dispatch = [&](auto f32) {
    constexpr bool kF32 = decltype(f32)::value;
    if (split && pair) {
      launch<kF32, true, true>(args, stream);
    } else if (split) {
      launch<kF32, false, true>(args, stream);
    } else if (pair) {
      launch<kF32, true, false>(args, stream);
    } else {
      launch<kF32, false, false>(args, stream);
    }
  };
  if (args.activations_f32) {
    dispatch(std::true_type{});
  } else {
    dispatch(std::false_type{});
  }
}

} // namespace rib200
