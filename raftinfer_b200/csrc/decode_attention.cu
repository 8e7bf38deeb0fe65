// Split-k GQA decode attention over the BF16 head-major KV cache, for 16 query heads / 4 KV heads /
// head_dim 256 (the only decode signature RAFTInfer accepts,
// cpp/kernels/qwen35_online_attention.cu:96-104).
//
// It replaces the four launches of cpp/kernels/qwen35_online_attention.cu:925-1015 (append, single
// block, partition, merge) by two: a partition kernel that also appends the new token, and a combine
// kernel whose sixteen-lane groups fold the split partials (shared memory and one pass of loads; the
// probabilities inside the partition kernel travel by warp shuffles).  The partial (max, sum, acc) contract
// and the workspace layout of cpp/kernels/qwen35_online_attention.cu:603-691,1111-1143 are kept.
//
// Bandwidth plan.  One CTA serves one (partition, KV head) and all four query heads of the group, so
// every K and V byte is read from HBM once (the reference streams each KV head four times).  Each warp
// owns 16-token steps of the partition.  Lane 0 of the warp is its producer: it moves the 512-byte K (or V)
// rows of a step, two at a time, from the cache into a private ring of shared-memory slots with TMA bulk
// copies (cp.async.bulk, completion counted on an mbarrier), several slots ahead of the consumer.  Row pairs sit
// at a 1040-byte pitch and the tensor-core row index is a permutation of the token order, which makes every
// ldmatrix of eight rows hit eight different bank groups.  Because ring, barriers and producer are private to
// the warp, no block-level barrier is needed while streaming.
//
// Arithmetic plan.  Tokens are the M dimension of mma.sync.m16n8k16 (BF16 in, FP32 accumulate) and the
// eight N columns carry the four query heads twice: column 2h holds the BF16 high part and column 2h+1
// the BF16 residual of head h, for q in the score product and for the probabilities in the value
// product.  Both products therefore see ~16 mantissa bits although the tensor cores run in BF16, at no
// extra cost (N = 8 is the minimum tile).  Softmax runs in FP32 with exp2f; accumulators are rescaled only
// when a running maximum moves.
//
// Every wait on an mbarrier is bounded: when it runs out the warp records RIB200_DEVICE_WAIT_TIMED_OUT in
// the device status word and leaves the streaming loop.

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

namespace rib200 {
namespace {

// Optional timeline probe (compile with -DRIB200_TRACE): every partition CTA records, in nanoseconds of the global
// timer, when it started, when its first slot had landed, when its stream ended and when it left; every combine CTA
// when it started, when the partition grid had completed and when it left.
#ifdef RIB200_TRACE
__device__ long long g_decode_trace[4096 * 4];
__device__ long long g_combine_trace[256 * 4];
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define RIB200_DECODE_STAMP(array, cta, slot)                          \
  do {                                                                 \
    if (threadIdx.x == 0 && (cta) < sizeof(array) / 32) {              \
      array[(cta) * 4 + (slot)] = global_ns();                         \
    }                                                                  \
  } while (0)
#else
#define RIB200_DECODE_STAMP(array, cta, slot) \
  do {                                        \
  } while (0)
#endif


constexpr int kHeadDim = 256;
constexpr int kQueryHeads = 16;
constexpr int kKvHeads = 4;
constexpr int kGroup = kQueryHeads / kKvHeads;
constexpr int kStepTokens = 16;
constexpr int kRowBytes = kHeadDim * 2;                // one cached K or V row
// A slot holds the 16 rows of a step as 8 pairs: rows 2p and 2p+1 back to back (1 KiB, one bulk copy) at a pitch of
// 1040 bytes.  The issue of a bulk copy costs the warp about as much for 1 KiB as for 512 bytes, so pairs halve the
// time a warp spends feeding its ring.  The MMA row index m stands for token 2 (m % 8) + m / 8 of the step: the
// eight rows of one ldmatrix then sit 1040 bytes apart, which is free of bank conflicts.
constexpr int kPairPitch = 2 * kRowBytes + 16;
constexpr int kSlotBytes = (kStepTokens / 2) * kPairPitch; // the K rows or the V rows of one step
__host__ __device__ constexpr std::uint32_t row_offset(std::uint32_t row) { // byte offset of a step's row in its slot
  return (row >> 1) * kPairPitch + (row & 1U) * kRowBytes;
}
constexpr int kMergePitch = kHeadDim + 8;              // floats per (warp, head) row of the merge area
constexpr long long kWaitLimitCycles = 1LL << 28;      // SM cycles an mbarrier wait may take before giving up

// Shape of one CTA: `Warps` warps, each with a private ring of `Slots` slots (K and V slots alternate).
template <int Warps, int Slots> struct Tile {
  static constexpr int kWarps = Warps;
  static constexpr int kRingSlots = Slots;
  static constexpr int kRingBytes = Warps * Slots * kSlotBytes;
  static constexpr int kBarrierBytes = (Warps * Slots * 8 + 15) / 16 * 16;
  // the cross-warp merge area reuses the ring once streaming is over
  static constexpr int kMergeFloats = Warps * (kGroup * kMergePitch + 2 * kGroup);
  static_assert(kMergeFloats * 4 <= kRingBytes, "merge area must fit in the ring");
  static constexpr int kSmemBytes = kRingBytes + kBarrierBytes;
  static constexpr int kCtasPerSm = (227 * 1024) / (kSmemBytes + 1024) > 0 ? (227 * 1024) / (kSmemBytes + 1024) : 1;
};
constexpr float kLog2e = 1.4426950408889634F;

struct DecodeParams {
  const void *query;
  const void *key;
  const void *value;
  const void *gate;
  void *output;
  __nv_bfloat16 *cache;               // single sequence
  void *const *caches;                // batched
  const std::uint32_t *max_ctx_array; // batched
  const std::uint32_t *pos_array;     // batched, or the device position of a single sequence
  std::uint32_t max_ctx;
  std::uint32_t host_pos;
  std::uint32_t partition_tokens;
  std::uint32_t threshold_tokens;
  std::uint32_t capacity;
  std::uint32_t max_partitions;
  float *partial_max;
  float *partial_sum;
  float *partial_value;
  std::size_t partial_stride; // floats between sequences in partial_max / partial_sum (batched)
  unsigned int *status;
  std::uint32_t early_kv; // single sequence, host position: the first ring slots are fetched before the wait below
  // Paged form of the batched kernel: `cache` is the page pool, a page holds one partition (256 tokens) in the
  // head-major layout of a 256-token cache, and block_tables[sequence][partition] names the page.
  const std::uint32_t *block_tables;
  std::uint32_t max_blocks;
  std::uint32_t pool_pages;
};

constexpr std::uint32_t kPageTokens = 256;
constexpr std::size_t kPageElems = static_cast<std::size_t>(2) * 4 * kPageTokens * 256;

__device__ __forceinline__ std::uint32_t smem_address(const void *p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbarrier_init(std::uint32_t bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbarrier_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(std::uint32_t bar, std::uint32_t parity) {
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

// L2 policy for the cache rows: a step reads each of them once, so they are the first to go.  What the step
// writes and reads again (the split-k partials) then stays in L2 between the two kernels.
__device__ __forceinline__ std::uint64_t evict_first_policy() {
  std::uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
  return policy;
}

// TMA bulk copy global -> shared, completion bytes counted on `bar`
__device__ __forceinline__ void bulk_copy_g2s(std::uint32_t dst, const void *src, std::uint32_t bytes,
                                              std::uint32_t bar, std::uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::"r"(
          dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(std::uint32_t addr, std::uint32_t &r0, std::uint32_t &r1,
                                            std::uint32_t &r2, std::uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(std::uint32_t addr, std::uint32_t &r0, std::uint32_t &r1,
                                                  std::uint32_t &r2, std::uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void sts128(std::uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], std::uint32_t a0, std::uint32_t a1, std::uint32_t a2,
                                         std::uint32_t a3, std::uint32_t b0, std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ std::uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const std::uint32_t *>(&v);
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// high part (part == 0) or residual (part == 1) of the two-term BF16 split of x
__device__ __forceinline__ float split_part(float x, int part) {
  const float hi = bf16_round(x);
  return part == 0 ? hi : x - hi;
}

template <bool F32> __device__ __forceinline__ void load8(const void *base, std::size_t index, float (&out)[8]) {
  if constexpr (F32) {
    const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + index);
    const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + index + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(base) + index);
    const std::uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000U);
    }
  }
}

template <bool F32> __device__ __forceinline__ void store8(void *base, std::size_t index, const float (&v)[8]) {
  if constexpr (F32) {
    *reinterpret_cast<float4 *>(static_cast<float *>(base) + index) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(static_cast<float *>(base) + index + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint4 raw;
    raw.x = pack_bf16(v[0], v[1]);
    raw.y = pack_bf16(v[2], v[3]);
    raw.z = pack_bf16(v[4], v[5]);
    raw.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(base) + index) = raw;
  }
}

template <bool F32> __device__ __forceinline__ uint4 load8_as_bf16(const void *base, std::size_t index) {
  float v[8];
  load8<F32>(base, index, v);
  uint4 raw;
  raw.x = pack_bf16(v[0], v[1]);
  raw.y = pack_bf16(v[2], v[3]);
  raw.z = pack_bf16(v[4], v[5]);
  raw.w = pack_bf16(v[6], v[7]);
  return raw;
}

// Partition kernel.  grid = (partition capacity, 4 KV heads, sequences), Warps * 32 threads.
template <bool F32, bool Batched, class T>
__global__ void __launch_bounds__(T::kWarps * 32, T::kCtasPerSm) decode_partition_kernel(const DecodeParams p) {
  constexpr int kWarps = T::kWarps;
  constexpr int kRingSlots = T::kRingSlots;
  constexpr int kRingBytes = T::kRingBytes;
  extern __shared__ __align__(128) unsigned char smem[];
  // Both kernels of a decode step are launched with programmatic stream serialisation.  This grid may have been
  // made resident early by the kernel before it (the combine kernel of a preceding step does that).  Unless the
  // caller has opted into the early cache fetch, nothing is read or written before that kernel has completed, so
  // the ordering is that of a plain launch, minus the launch latency.
  if (Batched || p.early_kv == 0) {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // Let the kernel behind this one become resident now; it blocks in its own griddepcontrol.wait until this
    // whole grid has finished and flushed.  (With the early cache fetch the release comes after the wait further
    // down, so that nothing launched behind this grid can start while the kernel in front of it still runs.)
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  }
  [[maybe_unused]] const unsigned int trace_cta = blockIdx.x + gridDim.x * blockIdx.y;
  RIB200_DECODE_STAMP(g_decode_trace, trace_cta, 0);

  const int seq = Batched ? static_cast<int>(blockIdx.z) : 0;
  const bool paged = Batched && p.block_tables != nullptr;
  const std::uint32_t max_ctx = (Batched && !paged) ? p.max_ctx_array[seq] : p.max_ctx;
  const std::uint32_t pos = p.pos_array != nullptr ? p.pos_array[seq] : p.host_pos;
  if (pos >= max_ctx) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
      atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_POSITION_OUT_OF_RANGE));
    }
    return;
  }
  const std::uint32_t ctx = pos + 1;
  const bool direct = p.partition_tokens == 0 || ctx < p.threshold_tokens;
  std::uint32_t begin = 0;
  std::uint32_t end = ctx;
  if (direct) {
    if (blockIdx.x != 0) {
      return;
    }
  } else {
    begin = blockIdx.x * p.partition_tokens;
    if (begin >= ctx) {
      return;
    }
    end = min(ctx, begin + p.partition_tokens);
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int kvh = blockIdx.y;
  // Token `tok` of a head's plane sits at row tok - origin: a contiguous cache holds the whole context, a page
  // only this CTA's partition.
  __nv_bfloat16 *cache = p.cache;
  std::uint32_t plane_tokens = max_ctx;
  std::uint32_t origin = 0;
  if constexpr (Batched) {
    if (paged) {
      const std::uint32_t page = p.block_tables[static_cast<std::size_t>(seq) * p.max_blocks + blockIdx.x];
      if (page >= p.pool_pages) {
        if (threadIdx.x == 0) {
          atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_PAGE_OUT_OF_RANGE));
        }
        return;
      }
      cache = p.cache + static_cast<std::size_t>(page) * kPageElems;
      plane_tokens = kPageTokens;
      origin = begin;
    } else {
      cache = static_cast<__nv_bfloat16 *>(p.caches[seq]);
    }
  }
  __nv_bfloat16 *k_plane = cache + static_cast<std::size_t>(kvh) * plane_tokens * kHeadDim;
  __nv_bfloat16 *v_plane = k_plane + static_cast<std::size_t>(kKvHeads) * plane_tokens * kHeadDim;
  const std::size_t act_seq = static_cast<std::size_t>(seq);
  const std::size_t kv_in_base = (act_seq * kKvHeads + kvh) * kHeadDim;

  const std::uint32_t total_steps = (end - begin + kStepTokens - 1) / kStepTokens;
  const std::uint32_t my_steps =
      total_steps > static_cast<std::uint32_t>(warp) ? (total_steps - warp + kWarps - 1) / kWarps : 0;
  const std::uint32_t my_slots = 2 * my_steps; // slot 2i = K rows of step i, slot 2i+1 = V rows of step i
  const std::uint32_t ring = smem_address(smem) + warp * kRingSlots * kSlotBytes;
  const std::uint32_t bars = smem_address(smem) + kRingBytes + warp * kRingSlots * 8;

  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kRingSlots; ++r) {
      mbarrier_init(bars + r * 8, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();

  const std::uint64_t stream_policy = evict_first_policy();
  // Producer (lane 0): slot n goes to ring position n % kRingSlots.  Only the live rows of the step are
  // copied; the consumer zero-fills the rest and patches in the row that is being appended.
  auto issue = [&](std::uint32_t n) {
    if (lane != 0) {
      return;
    }
    const std::uint32_t tok0 = begin + (warp + (n >> 1) * kWarps) * kStepTokens;
    const std::uint32_t rows = min(static_cast<std::uint32_t>(kStepTokens), end - tok0);
    const std::uint32_t slot = ring + (n % kRingSlots) * kSlotBytes;
    const std::uint32_t bar = bars + (n % kRingSlots) * 8;
    const __nv_bfloat16 *src =
        ((n & 1U) == 0 ? k_plane : v_plane) + static_cast<std::size_t>(tok0 - origin) * kHeadDim;
    fence_proxy_async(); // earlier reads of this ring position are ordered before the TMA write
    mbarrier_expect_tx(bar, rows * kRowBytes);
#pragma unroll
    for (int pair = 0; pair < kStepTokens / 2; ++pair) {
      if (static_cast<std::uint32_t>(2 * pair) < rows) {
        const std::uint32_t live = min(2U, rows - 2 * pair);
        bulk_copy_g2s(slot + pair * kPairPitch, src + 2 * pair * kHeadDim, live * kRowBytes, bar, stream_policy);
      }
    }
  };

  // Consumer side of slot n.  Returns false when the wait ran out.
  bool healthy = true;
  auto wait_slot = [&](std::uint32_t n) {
    const std::uint32_t bar = bars + (n % kRingSlots) * 8;
    const std::uint32_t parity = (n / kRingSlots) & 1U;
    if (!mbarrier_try_wait(bar, parity)) {
      const long long started = clock64();
      while (!mbarrier_try_wait(bar, parity)) {
        if (clock64() - started > kWaitLimitCycles) {
          healthy = false;
          break;
        }
      }
    }
    healthy = __all_sync(0xFFFFFFFFU, healthy);
    if (n == 0) {
      RIB200_DECODE_STAMP(g_decode_trace, trace_cta, 1);
    }
    return healthy;
  };

  // After the copy has landed: patch in the row being appended (it is not in the cache yet; its bytes come
  // from the key/value input and also go to the cache) and zero the rows past the live range.
  auto fix_rows = [&](std::uint32_t n, std::uint32_t tok0) {
    const std::uint32_t slot = ring + (n % kRingSlots) * kSlotBytes;
    const bool is_value = (n & 1U) != 0;
    bool touched = false;
    if (pos >= tok0 && pos < tok0 + kStepTokens && pos < end) {
      const uint4 raw = load8_as_bf16<F32>(is_value ? p.value : p.key, kv_in_base + 8 * lane);
      sts128(slot + row_offset(pos - tok0) + lane * 16, raw);
      __nv_bfloat16 *plane = is_value ? v_plane : k_plane;
      *reinterpret_cast<uint4 *>(plane + static_cast<std::size_t>(pos - origin) * kHeadDim + 8 * lane) = raw;
      touched = true;
    }
    if (tok0 + kStepTokens > end) {
      for (std::uint32_t r = end - tok0; r < kStepTokens; ++r) {
        sts128(slot + row_offset(r) + lane * 16, make_uint4(0U, 0U, 0U, 0U));
      }
      touched = true;
    }
    if (touched) {
      __syncwarp();
    }
  };

  // get the first slots moving before anything else is fetched
#pragma unroll
  for (int n = 0; n < kRingSlots - 1; ++n) {
    if (static_cast<std::uint32_t>(n) < my_slots) {
      issue(n);
    }
  }
  const bool whole_ring_early = !Batched && p.early_kv != 0;
  if (whole_ring_early && static_cast<std::uint32_t>(kRingSlots - 1) < my_slots) {
    issue(kRingSlots - 1); // nothing has been consumed yet: the last ring position can be filled now as well
  }
  if (!Batched && p.early_kv != 0) {
    // Early cache fetch: the copies above read cache rows only, with every address taken from kernel
    // parameters, and the caller has promised that no kernel in flight writes those rows.  Everything the
    // kernel in front may have produced (query, key, value, gate) and everything this grid writes comes
    // after this wait.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  }

  // Query fragments (the B operand of the score product): lane (g, t) holds, for k-step ks, dims
  // 16ks + 2t, +1 and 16ks + 8 + 2t, +1 of N column g = (head g>>1, split part g&1), pre-scaled by
  // 1/sqrt(256).
  std::uint32_t qf[32];
  {
    const int head = kvh * kGroup + (g >> 1);
    const int part = g & 1;
    const std::size_t q_base = (act_seq * kQueryHeads + head) * kHeadDim;
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const std::size_t index = q_base + 16 * ks + 8 * half + 2 * t;
        float x0;
        float x1;
        if constexpr (F32) {
          const float2 v = *reinterpret_cast<const float2 *>(static_cast<const float *>(p.query) + index);
          x0 = v.x;
          x1 = v.y;
        } else {
          const std::uint32_t raw =
              *reinterpret_cast<const std::uint32_t *>(static_cast<const __nv_bfloat16 *>(p.query) + index);
          x0 = __uint_as_float(raw << 16);
          x1 = __uint_as_float(raw & 0xFFFF0000U);
        }
        qf[2 * ks + half] = pack_bf16(split_part(x0 * 0.0625F, part), split_part(x1 * 0.0625F, part));
      }
    }
  }

  // ldmatrix lane addressing.  K (A operand, tokens x dims): matrix mi = lane>>3 covers MMA rows
  // (mi&1)*8.., 16-byte chunk (mi>>1) of the k-step.  V (A operand transposed, dims x tokens): matrix mi
  // covers MMA k indices (mi>>1)*8.., chunk (mi&1) of the 16-dim tile.  MMA index m is token 2 (m % 8) + m / 8.
  const int mi = lane >> 3;
  const std::uint32_t k_lane = (lane & 7) * kPairPitch + (mi & 1) * kRowBytes + (mi >> 1) * 16;
  const std::uint32_t v_lane = (lane & 7) * kPairPitch + (mi >> 1) * kRowBytes + (mi & 1) * 16;

  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0F;
  }
  float run_max = -INFINITY; // head t, identical in the eight lanes that share t
  float run_sum = 0.0F;      // this lane's share of the row sum of head t

  for (std::uint32_t i = 0; i < my_steps; ++i) {
    const std::uint32_t tok0 = begin + (warp + i * kWarps) * kStepTokens;

    // ---- K slot: scores and softmax ----
    fence_proxy_async();
    __syncwarp(); // all lanes are done with the ring position that is refilled next
    if (2 * i + kRingSlots - 1 < my_slots && !(whole_ring_early && i == 0)) {
      issue(2 * i + kRingSlots - 1);
    }
    if (!wait_slot(2 * i)) {
      break;
    }
    fix_rows(2 * i, tok0);
    const std::uint32_t k_slot = ring + ((2 * i) % kRingSlots) * kSlotBytes + k_lane;

    // S[token][column] = K[token][:] . Q[column][:], four independent accumulator chains
    float s0[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    float s1[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    float s2[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    float s3[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
    for (int ks = 0; ks < 16; ks += 4) {
      std::uint32_t a[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        ldmatrix_x4(k_slot + (ks + u) * 32, a[u][0], a[u][1], a[u][2], a[u][3]);
      }
      mma_bf16(s0, a[0][0], a[0][1], a[0][2], a[0][3], qf[2 * ks + 0], qf[2 * ks + 1]);
      mma_bf16(s1, a[1][0], a[1][1], a[1][2], a[1][3], qf[2 * ks + 2], qf[2 * ks + 3]);
      mma_bf16(s2, a[2][0], a[2][1], a[2][2], a[2][3], qf[2 * ks + 4], qf[2 * ks + 5]);
      mma_bf16(s3, a[3][0], a[3][1], a[3][2], a[3][3], qf[2 * ks + 6], qf[2 * ks + 7]);
    }
    // lane (g, t): head t, MMA rows g and g + 8 = tokens tok0 + 2g and tok0 + 2g + 1 (high part + residual columns)
    float score_a = ((s0[0] + s1[0]) + (s2[0] + s3[0])) + ((s0[1] + s1[1]) + (s2[1] + s3[1]));
    float score_b = ((s0[2] + s1[2]) + (s2[2] + s3[2])) + ((s0[3] + s1[3]) + (s2[3] + s3[3]));
    if (tok0 + 2 * g >= end) {
      score_a = -INFINITY;
    }
    if (tok0 + 2 * g + 1 >= end) {
      score_b = -INFINITY;
    }
    float step_max = fmaxf(score_a, score_b);
    step_max = fmaxf(step_max, __shfl_xor_sync(0xFFFFFFFFU, step_max, 4));
    step_max = fmaxf(step_max, __shfl_xor_sync(0xFFFFFFFFU, step_max, 8));
    step_max = fmaxf(step_max, __shfl_xor_sync(0xFFFFFFFFU, step_max, 16));
    if (__any_sync(0xFFFFFFFFU, step_max > run_max)) {
      // some head's running maximum moved: rescale what has been accumulated (rare after the first steps)
      const float new_max = fmaxf(run_max, step_max); // finite: the step holds at least one live token
      const float rescale = exp2f((run_max - new_max) * kLog2e);
      run_sum *= rescale;
      run_max = new_max;
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        oacc[m][0] *= rescale;
        oacc[m][1] *= rescale;
        oacc[m][2] *= rescale;
        oacc[m][3] *= rescale;
      }
    }
    const float prob_a = exp2f((score_a - run_max) * kLog2e);
    const float prob_b = exp2f((score_b - run_max) * kLog2e);
    run_sum += prob_a + prob_b;

    // probabilities as the B operand of the value product: lane (g, t) needs column g = (head g>>1,
    // part g&1) for tokens 2t, 2t+1, 2t+8, 2t+9; lane (token, head) holds them after the softmax.
    const int src0 = (2 * t) * 4 + (g >> 1);
    const int src1 = (2 * t + 1) * 4 + (g >> 1);
    const float p0 = __shfl_sync(0xFFFFFFFFU, prob_a, src0);
    const float p1 = __shfl_sync(0xFFFFFFFFU, prob_a, src1);
    const float p2 = __shfl_sync(0xFFFFFFFFU, prob_b, src0);
    const float p3 = __shfl_sync(0xFFFFFFFFU, prob_b, src1);
    const int part = g & 1;
    const std::uint32_t pb0 = pack_bf16(split_part(p0, part), split_part(p1, part));
    const std::uint32_t pb1 = pack_bf16(split_part(p2, part), split_part(p3, part));

    // ---- V slot: O[dim][column] += V[token][dim] * P[token][column] ----
    fence_proxy_async();
    __syncwarp();
    if (2 * i + kRingSlots < my_slots) {
      issue(2 * i + kRingSlots);
    }
    if (!wait_slot(2 * i + 1)) {
      break;
    }
    fix_rows(2 * i + 1, tok0);
    const std::uint32_t v_slot = ring + ((2 * i + 1) % kRingSlots) * kSlotBytes + v_lane;
#pragma unroll
    for (int mt = 0; mt < 16; mt += 4) {
      std::uint32_t a[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        ldmatrix_x4_trans(v_slot + (mt + u) * 32, a[u][0], a[u][1], a[u][2], a[u][3]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        mma_bf16(oacc[mt + u], a[u][0], a[u][1], a[u][2], a[u][3], pb0, pb1);
      }
    }
  }
  if (!healthy && lane == 0) {
    atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
  }

  run_sum += __shfl_xor_sync(0xFFFFFFFFU, run_sum, 4);
  run_sum += __shfl_xor_sync(0xFFFFFFFFU, run_sum, 8);
  run_sum += __shfl_xor_sync(0xFFFFFFFFU, run_sum, 16);

  // cross-warp combine through shared memory.  Lane (g, t) holds, for head t and every 16-dim tile mt,
  // dims 16mt + g and 16mt + g + 8 (high-part column + residual column).
  RIB200_DECODE_STAMP(g_decode_trace, trace_cta, 2);
  __syncthreads(); // every warp has left its ring: the merge area may now overwrite it
  float *merge = reinterpret_cast<float *>(smem);
  float *warp_max = merge;                       // [kWarps][4]
  float *warp_sum = merge + kWarps * kGroup;     // [kWarps][4]
  float *warp_out = merge + 2 * kWarps * kGroup; // [kWarps][4][kMergePitch]
  if (g == 0) {
    warp_max[warp * kGroup + t] = run_max;
    warp_sum[warp * kGroup + t] = run_sum;
  }
#pragma unroll
  for (int mt = 0; mt < 16; ++mt) {
    float *dst = warp_out + (warp * kGroup + t) * kMergePitch + 16 * mt + g;
    dst[0] = oacc[mt][0] + oacc[mt][1];
    dst[8] = oacc[mt][2] + oacc[mt][3];
  }
  __syncthreads();

  // 4 heads x 32 eight-dim pieces = 128 work items over the CTA's threads
  for (int item = threadIdx.x; item < kGroup * 32; item += kWarps * 32) {
    const int head_in_group = item >> 5;
    const int dim0 = (item & 31) * 8;
    float block_max = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      block_max = fmaxf(block_max, warp_max[w * kGroup + head_in_group]);
    }
    float block_sum = 0.0F;
    float acc[8] = {0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float weight = exp2f((warp_max[w * kGroup + head_in_group] - block_max) * kLog2e);
      block_sum += warp_sum[w * kGroup + head_in_group] * weight;
      const float *src = warp_out + (w * kGroup + head_in_group) * kMergePitch + dim0;
      const float4 a = *reinterpret_cast<const float4 *>(src);
      const float4 b = *reinterpret_cast<const float4 *>(src + 4);
      acc[0] += a.x * weight; acc[1] += a.y * weight; acc[2] += a.z * weight; acc[3] += a.w * weight;
      acc[4] += b.x * weight; acc[5] += b.y * weight; acc[6] += b.z * weight; acc[7] += b.w * weight;
    }

    const int head = kvh * kGroup + head_in_group;
    if (direct) {
      const std::size_t out_index = (act_seq * kQueryHeads + head) * kHeadDim + dim0;
      float gate[8];
      load8<F32>(p.gate, out_index, gate);
      float result[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        result[e] = (acc[e] / block_sum) / (1.0F + expf(-gate[e]));
      }
      store8<F32>(p.output, out_index, result);
      continue;
    }
    const std::size_t partial = static_cast<std::size_t>(head) * p.max_partitions + blockIdx.x;
    float *pmax = p.partial_max + act_seq * p.partial_stride;
    float *psum = p.partial_sum + act_seq * p.partial_stride;
    float *pval = p.partial_value + act_seq * p.partial_stride * kHeadDim;
    if ((item & 31) == 0) {
      pmax[partial] = block_max;
      psum[partial] = block_sum;
    }
    float *dst = pval + partial * kHeadDim + dim0;
    *reinterpret_cast<float4 *>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  RIB200_DECODE_STAMP(g_decode_trace, trace_cta, 3);
}

// Combine kernel.  grid = (16 query heads, 4 dim quarters, sequences), 256 threads: sixteen partition
// groups of sixteen lanes, a lane owning four consecutive dims of the quarter.
template <bool F32, bool Batched>
__global__ void __launch_bounds__(256) decode_combine_kernel(const DecodeParams p) {
  __shared__ float group_max[16];
  __shared__ float group_sum[16];
  __shared__ float group_acc[16][64];

  // wait until the partition grid has completed and its partials are visible
  [[maybe_unused]] const unsigned int trace_cta = blockIdx.x + gridDim.x * blockIdx.y;
  RIB200_DECODE_STAMP(g_combine_trace, trace_cta, 0);
  // a kernel launched behind this one with programmatic serialisation may become resident (it waits for this grid)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  // the gate does not come from the partition grid: fetch it while that grid is still running
  float gate_value = 0.0F;
  if (threadIdx.x < 64) {
    const std::size_t gate_index =
        ((Batched ? static_cast<std::size_t>(blockIdx.z) : 0) * kQueryHeads + blockIdx.x) * kHeadDim + blockIdx.y * 64 +
        threadIdx.x;
    if constexpr (F32) {
      gate_value = static_cast<const float *>(p.gate)[gate_index];
    } else {
      gate_value = __bfloat162float(static_cast<const __nv_bfloat16 *>(p.gate)[gate_index]);
    }
  }
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  RIB200_DECODE_STAMP(g_combine_trace, trace_cta, 1);

  const int seq = Batched ? static_cast<int>(blockIdx.z) : 0;
  const std::uint32_t max_ctx = (Batched && p.block_tables == nullptr) ? p.max_ctx_array[seq] : p.max_ctx;
  const std::uint32_t pos = p.pos_array != nullptr ? p.pos_array[seq] : p.host_pos;
  if (pos >= max_ctx) {
    return;
  }
  const std::uint32_t ctx = pos + 1;
  if (p.partition_tokens == 0 || ctx < p.threshold_tokens) {
    return; // served directly by the partition kernel
  }
  const std::uint32_t parts = (ctx + p.partition_tokens - 1) / p.partition_tokens;
  if (parts > p.capacity) {
    // The captured grid cannot cover this context.  Record it and leave the output untouched.
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
      atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_DECODE_CAPACITY_EXCEEDED));
    }
    return;
  }
  const std::size_t act_seq = static_cast<std::size_t>(seq);
  const int head = blockIdx.x;
  const int quarter = blockIdx.y;
  const float *pmax = p.partial_max + act_seq * p.partial_stride + static_cast<std::size_t>(head) * p.max_partitions;
  const float *psum = p.partial_sum + act_seq * p.partial_stride + static_cast<std::size_t>(head) * p.max_partitions;
  const float *pval = p.partial_value +
                      (act_seq * p.partial_stride + static_cast<std::size_t>(head) * p.max_partitions) * kHeadDim;

  // One pass: every thread folds its share of the partials into a running (max, sum, acc) - all loads of the
  // pass are independent, so they are in flight together - then the sixteen groups are folded in shared memory.
  const int group = threadIdx.x >> 4;
  const int sub = threadIdx.x & 15;
  float run_max = -INFINITY;
  float run_sum = 0.0F;
  float4 acc = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  // Eight partials at a time: first all their loads (so that they are in flight together, one round trip to L2 for
  // a 32K context), then the folding.
  constexpr int kBatch = 8;
  for (std::uint32_t first = group; first < parts; first += 16 * kBatch) {
    float part_max[kBatch];
    float part_sum[kBatch];
    float4 part_value[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const std::uint32_t i = first + 16 * j;
      if (i < parts) {
        part_max[j] = pmax[i];
        part_sum[j] = psum[i];
        part_value[j] =
            *reinterpret_cast<const float4 *>(pval + static_cast<std::size_t>(i) * kHeadDim + quarter * 64 + sub * 4);
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (first + 16 * j < parts) {
        const float4 v = part_value[j];
        const float new_max = fmaxf(run_max, part_max[j]);
        const float keep = exp2f((run_max - new_max) * kLog2e);
        const float take = exp2f((part_max[j] - new_max) * kLog2e);
        run_sum = run_sum * keep + part_sum[j] * take;
        acc.x = acc.x * keep + v.x * take;
        acc.y = acc.y * keep + v.y * take;
        acc.z = acc.z * keep + v.z * take;
        acc.w = acc.w * keep + v.w * take;
        run_max = new_max;
      }
    }
  }
  RIB200_DECODE_STAMP(g_combine_trace, trace_cta, 3);
  if (sub == 0) {
    group_max[group] = run_max;
    group_sum[group] = run_sum;
  }
  *reinterpret_cast<float4 *>(&group_acc[group][sub * 4]) = acc;
  __syncthreads();
  if (threadIdx.x < 64) {
    float total_max = group_max[0];
#pragma unroll
    for (int gidx = 1; gidx < 16; ++gidx) {
      total_max = fmaxf(total_max, group_max[gidx]);
    }
    float total_sum = 0.0F;
    float total = 0.0F;
#pragma unroll
    for (int gidx = 0; gidx < 16; ++gidx) {
      const float weight = exp2f((group_max[gidx] - total_max) * kLog2e); // 0 for a group that had no partial
      total_sum += group_sum[gidx] * weight;
      total += group_acc[gidx][threadIdx.x] * weight;
    }
    const std::size_t out_index = (act_seq * kQueryHeads + head) * kHeadDim + quarter * 64 + threadIdx.x;
    if constexpr (F32) {
      static_cast<float *>(p.output)[out_index] = (total / total_sum) / (1.0F + expf(-gate_value));
    } else {
      static_cast<__nv_bfloat16 *>(p.output)[out_index] =
          __float2bfloat16_rn((total / total_sum) / (1.0F + expf(-gate_value)));
    }
  }
  RIB200_DECODE_STAMP(g_combine_trace, trace_cta, 2);
}

// CTA shapes.  Shared memory bounds the bytes in flight per SM (the rings fill it either way), so the shape
// only decides how the partitions spread over the machine: with many partitions a CTA is a single warp (no
// cross-warp merge, most CTAs resident); with few, more warps share a partition so that every SM has work and
// each warp's chain of dependent steps is short.  All shapes are the same kernel template.
template <bool F32, bool Batched, class T> void configure_once() {
  static std::once_flag flags[64];
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  std::call_once(flags[device], [] {
    cuda_ok(cudaFuncSetAttribute(decode_partition_kernel<F32, Batched, T>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes),
            "decode attention shared-memory opt-in");
  });
}

template <bool F32, bool Batched, class T>
void launch_pair_tiled(const DecodeParams &params, dim3 partition_grid, dim3 combine_grid, bool combine,
                       cudaStream_t stream) {
  configure_once<F32, Batched, T>();
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = partition_grid;
  config.blockDim = dim3(T::kWarps * 32, 1, 1);
  config.dynamicSmemBytes = T::kSmemBytes;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  cuda_ok(cudaLaunchKernelEx(&config, decode_partition_kernel<F32, Batched, T>, params),
          "decode attention partition launch");
  if (!combine) {
    return;
  }
  config.gridDim = combine_grid;
  config.blockDim = dim3(256, 1, 1);
  config.dynamicSmemBytes = 0;
  cuda_ok(cudaLaunchKernelEx(&config, decode_combine_kernel<F32, Batched>, params),
          "decode attention combine launch");
}

template <bool F32, bool Batched>
void launch_pair(const DecodeParams &params, dim3 partition_grid, dim3 combine_grid, bool combine,
                 cudaStream_t stream) {
  const std::size_t ctas = static_cast<std::size_t>(partition_grid.x) * partition_grid.y * partition_grid.z;
  if (ctas <= 148) {
    launch_pair_tiled<F32, Batched, Tile<8, 3>>(params, partition_grid, combine_grid, combine, stream);
  } else if (ctas <= 296) {
    launch_pair_tiled<F32, Batched, Tile<4, 3>>(params, partition_grid, combine_grid, combine, stream);
  } else if (ctas <= 592) {
    launch_pair_tiled<F32, Batched, Tile<2, 3>>(params, partition_grid, combine_grid, combine, stream);
  } else {
    launch_pair_tiled<F32, Batched, Tile<1, 3>>(params, partition_grid, combine_grid, combine, stream);
  }
}

} // namespace

#ifdef RIB200_TRACE
extern "C" int rib200_debug_read_decode_trace(long long *partition, long long *combine) {
  const int first = static_cast<int>(cudaMemcpyFromSymbol(partition, g_decode_trace, sizeof(g_decode_trace)));
  const int second = static_cast<int>(cudaMemcpyFromSymbol(combine, g_combine_trace, sizeof(g_combine_trace)));
  return first != 0 ? first : second;
}
#endif

void launch_decode_attention(const DecodeArgs &a, cudaStream_t stream) {
  DecodeParams params{};
  params.query = a.query;
  params.key = a.key;
  params.value = a.value;
  params.gate = a.gate;
  params.output = a.output;
  params.cache = static_cast<__nv_bfloat16 *>(a.kv_cache);
  params.pos_array = a.device_position;
  params.max_ctx = a.max_context_tokens;
  params.host_pos = a.host_position;
  params.partition_tokens = a.partition_tokens;
  params.threshold_tokens = a.threshold_tokens;
  params.capacity = a.partition_capacity;
  params.max_partitions = a.max_partitions;
  params.partial_max = a.partial_max;
  params.partial_sum = a.partial_sum;
  params.partial_value = a.partial_value;
  params.partial_stride = 0;
  params.status = device_status_word();
  params.early_kv = (a.device_position == nullptr && a.early_kv_fetch) ? 1U : 0U;
  const bool split = a.partition_tokens != 0;
  const dim3 partition_grid(split ? a.partition_capacity : 1, kKvHeads, 1);
  const dim3 combine_grid(kQueryHeads, 4, 1);
  if (a.activations_f32) {
    launch_pair<true, false>(params, partition_grid, combine_grid, split, stream);
  } else {
    launch_pair<false, false>(params, partition_grid, combine_grid, split, stream);
  }
}

void launch_batched_decode_attention(const BatchedDecodeArgs &a, cudaStream_t stream) {
  DecodeParams params{};
  params.query = a.query;
  params.key = a.key;
  params.value = a.value;
  params.gate = a.gate;
  params.output = a.output;
  params.caches = a.kv_caches;
  params.max_ctx_array = a.max_context_tokens;
  if (a.block_tables != nullptr) {
    params.cache = static_cast<__nv_bfloat16 *>(a.page_pool);
    params.block_tables = a.block_tables;
    params.max_blocks = a.partition_capacity;
    params.pool_pages = a.pool_pages;
    params.max_ctx = a.partition_capacity * kPageTokens;
  }
  params.pos_array = a.positions;
  params.partition_tokens = 256;
  params.threshold_tokens = 256;
  params.capacity = a.partition_capacity;
  params.max_partitions = a.partition_capacity;
  const std::size_t partials = static_cast<std::size_t>(kQueryHeads) * a.partition_capacity;
  params.partial_stride = partials;
  params.partial_max = a.workspace;
  params.partial_sum = a.workspace + static_cast<std::size_t>(a.batch) * partials;
  params.partial_value = a.workspace + 2 * static_cast<std::size_t>(a.batch) * partials;
  params.status = device_status_word();
  const dim3 partition_grid(a.partition_capacity, kKvHeads, a.batch);
  const dim3 combine_grid(kQueryHeads, 4, a.batch);
  launch_pair<false, true>(params, partition_grid, combine_grid, true, stream);
}

} // namespace rib200

// ---- decode with library-owned scratch -------------------------------------------------------
//
// Split-k partials of the entry point below live in this array instead of a caller workspace.  It is sized for
// the largest cache the entry point accepts: 16 heads x (32768 / 256) partitions x (max + sum + 256 values)
// floats = 2 113 536 bytes.  Every GPU that loads the library keeps that much memory until the process exits.
constexpr std::uint32_t kStaticScratchMaxContext = 32768;
constexpr std::uint32_t kStaticScratchPartitions = kStaticScratchMaxContext / 256;
constexpr std::size_t kStaticScratchFloats = static_cast<std::size_t>(16) * kStaticScratchPartitions * (256 + 2);
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

// In host code `g_decode_scratch` is only a handle for the runtime, not a device address, so a kernel must
// never be given the name itself.  The real address is looked up once per device, with that device current.
static float *static_scratch_for_current_device() {
  using namespace rib200;
  static std::mutex lock;
  static float *address[64] = {};
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  std::lock_guard<std::mutex> guard(lock);
  if (address[device] == nullptr) {
    float *ptr = nullptr;
    cuda_ok(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_decode_scratch),
            "decode scratch: cudaGetSymbolAddress");
    require(ptr != nullptr, "decode scratch: the runtime returned a null address", RIB200_STATUS_INTERNAL);
    address[device] = ptr;
  }
  return address[device];
}

extern "C" Rib200Status rib200_online_attention_decode_static_scratch(
    const void *query, const void *key, const void *value, const void *gate, void *output, void *kv_cache,
    size_t kv_cache_bytes, const Rib200AttentionShape *shape, int32_t activation_dtype,
    const uint32_t *device_position, void *stream) {
  using namespace rib200;
  return guarded([&] {
    require(shape != nullptr, "static-scratch decode: shape pointer is null");
    require(query != nullptr && key != nullptr && value != nullptr && gate != nullptr && output != nullptr,
            "static-scratch decode: an activation pointer is null");
    require(kv_cache != nullptr, "static-scratch decode: KV cache pointer is null");
    require(stream != nullptr, "static-scratch decode: CUDA stream is null");
    require(shape->tokens == 1 && shape->query_heads == kQueryHeads && shape->kv_heads == kKvHeads &&
                shape->head_dim == kHeadDim,
            "static-scratch decode: needs one token, 16 query heads, 4 kv heads, head_dim 256");
    require(shape->max_context_tokens != 0 && shape->past_tokens < shape->max_context_tokens,
            "static-scratch decode: position outside the cache");
    require(shape->max_context_tokens <= kStaticScratchMaxContext,
            "static-scratch decode: max_context_tokens exceeds the 32768 tokens the built-in scratch is sized for; "
            "use rib200_online_attention_decode with a caller workspace");
    require(activation_dtype == RIB200_DTYPE_F32 || activation_dtype == RIB200_DTYPE_BF16,
            "static-scratch decode: activations must be F32 or BF16");
    require(kv_cache_bytes >= 2 * shape->max_context_tokens * kKvHeads * kHeadDim * sizeof(__nv_bfloat16),
            "static-scratch decode: KV cache is too small");
    for (const void *ptr : {query, key, value, gate, static_cast<const void *>(output),
                            static_cast<const void *>(kv_cache)}) {
      require(reinterpret_cast<std::uintptr_t>(ptr) % 16 == 0,
              "static-scratch decode: pointers must be 16-byte aligned");
    }
    const std::uint32_t max_ctx = static_cast<std::uint32_t>(shape->max_context_tokens);
    const std::uint32_t partitions = (max_ctx + 255) / 256;
    float *scratch = static_scratch_for_current_device();
    DecodeParams params{};
    params.query = query;
    params.key = key;
    params.value = value;
    params.gate = gate;
    params.output = output;
    params.cache = static_cast<__nv_bfloat16 *>(kv_cache);
    params.pos_array = device_position;
    params.max_ctx = max_ctx;
    params.host_pos = static_cast<std::uint32_t>(shape->past_tokens);
    params.partition_tokens = 256;
    params.threshold_tokens = 256;
    params.capacity = partitions;
    params.max_partitions = partitions;
    const std::size_t partials = static_cast<std::size_t>(kQueryHeads) * partitions;
    params.partial_max = scratch;
    params.partial_sum = scratch + partials;
    params.partial_value = scratch + 2 * partials;
    params.partial_stride = 0;
    params.status = device_status_word();
    const dim3 partition_grid(partitions, kKvHeads, 1);
    const dim3 combine_grid(kQueryHeads, 4, 1);
    auto *cuda_stream = static_cast<cudaStream_t>(stream);
    if (activation_dtype == RIB200_DTYPE_F32) {
      launch_pair<true, false>(params, partition_grid, combine_grid, true, cuda_stream);
    } else {
      launch_pair<false, false>(params, partition_grid, combine_grid, true, cuda_stream);
    }
  });
}
