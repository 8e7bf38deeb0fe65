// Recurrent gated delta-rule update (cpp/kernels/qwen35_delta.cu:482-576, CPU form
// cpp/reference/qwen35.cpp:459-518) for key_dim = value_dim = 128.
//
// Per value head the FP32 state S[128][128] is read once and written once per token:
//   a = S^T k, b = S^T q            (one pass, both products together)
//   delta = (v - decay * a) * beta
//   out   = decay * b + delta * (k . q)
//   S     = decay * S + k delta^T
// which is the reference's "decay, read, correct, write, read again" sequence folded into one pass.
//
// A CTA owns 64 state columns of one head; a warp owns 8 of them and a lane 4 state rows, so a lane's
// slice (4 x 8 floats) stays in registers across tokens, every load is a full 32-byte sector and the two
// reductions over the 128 rows are warp shuffles: the kernel has no block-level barrier at all.  For a
// batch of decoding sequences the grid is (2, value_heads, sequences) and the step is bound by HBM.

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

namespace rib200 {
namespace {

constexpr int kDim = 128;

struct RecurrentParams {
  const void *q, *k, *v;
  std::size_t q_stride, k_stride, v_stride;
  const float *beta;
  const float *log_decay;
  float *state;
  float *const *states;
  float *out;
  std::uint32_t tokens;
  std::uint32_t key_heads;
  std::uint32_t value_heads;
};

template <bool F32> __device__ __forceinline__ void load4(const void *base, std::size_t index, float (&o)[4]) {
  if constexpr (F32) {
    const float4 v = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + index);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  } else {
    const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + index);
    o[0] = __uint_as_float(raw.x << 16);
    o[1] = __uint_as_float(raw.x & 0xFFFF0000U);
    o[2] = __uint_as_float(raw.y << 16);
    o[3] = __uint_as_float(raw.y & 0xFFFF0000U);
  }
}

template <bool F32>
__global__ void __launch_bounds__(256, 4) gdn_recurrent_kernel(const RecurrentParams p) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::uint32_t head = blockIdx.y;
  const std::uint32_t seq = blockIdx.z;
  const std::uint32_t key_head = head % p.key_heads;
  const int col0 = blockIdx.x * 64 + warp * 8;
  const int row0 = lane * 4;
  // Launched with programmatic stream serialisation: the grid may be resident while the kernel in front of it (the
  // previous token's step, in a run of decode steps) is still finishing.  Nothing is read or written before that
  // kernel has completed, so the ordering is that of a plain launch, minus most of the launch latency; the kernel
  // behind this one is let in on the same terms.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  float *state = (p.states != nullptr ? p.states[seq] : p.state) + static_cast<std::size_t>(head) * kDim * kDim;

  float s[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 lo = *reinterpret_cast<const float4 *>(state + (row0 + i) * kDim + col0);
    const float4 hi = *reinterpret_cast<const float4 *>(state + (row0 + i) * kDim + col0 + 4);
    s[i][0] = lo.x; s[i][1] = lo.y; s[i][2] = lo.z; s[i][3] = lo.w;
    s[i][4] = hi.x; s[i][5] = hi.y; s[i][6] = hi.z; s[i][7] = hi.w;
  }

  for (std::uint32_t tok = 0; tok < p.tokens; ++tok) {
    const std::size_t item = static_cast<std::size_t>(seq) * p.tokens + tok;
    float kk[4];
    float qq[4];
    float vlo[4];
    float vhi[4];
    load4<F32>(p.k, item * p.k_stride + key_head * kDim + row0, kk);
    load4<F32>(p.q, item * p.q_stride + key_head * kDim + row0, qq);
    load4<F32>(p.v, item * p.v_stride + head * kDim + col0, vlo);
    load4<F32>(p.v, item * p.v_stride + head * kDim + col0 + 4, vhi);
    const float beta = p.beta[item * p.value_heads + head];
    const float decay = expf(p.log_decay[item * p.value_heads + head]);

    float red[17];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      red[c] = s[0][c] * kk[0] + s[1][c] * kk[1] + s[2][c] * kk[2] + s[3][c] * kk[3];
      red[8 + c] = s[0][c] * qq[0] + s[1][c] * qq[1] + s[2][c] * qq[2] + s[3][c] * qq[3];
    }
    red[16] = kk[0] * qq[0] + kk[1] * qq[1] + kk[2] * qq[2] + kk[3] * qq[3];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
#pragma unroll
      for (int c = 0; c < 17; ++c) {
        red[c] += __shfl_xor_sync(0xFFFFFFFFU, red[c], offset);
      }
    }
    float delta[8];
    float o[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float vc = c < 4 ? vlo[c] : vhi[c - 4];
      delta[c] = (vc - decay * red[c]) * beta;
      o[c] = decay * red[8 + c] + delta[c] * red[16];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        s[i][c] = decay * s[i][c] + kk[i] * delta[c];
      }
    }
    if (lane == 0) {
      float *dst = p.out + (item * p.value_heads + head) * kDim + col0;
      *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4 *>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    *reinterpret_cast<float4 *>(state + (row0 + i) * kDim + col0) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
    *reinterpret_cast<float4 *>(state + (row0 + i) * kDim + col0 + 4) =
        make_float4(s[i][4], s[i][5], s[i][6], s[i][7]);
  }
}

// Batched decode step: one token for each of many sequences.  One CTA per SM walks an equal share of the
// (sequence, value head) pairs.  A head's whole 64 KiB state - one contiguous block of memory - streams through a
// three-stage ring in shared memory without any thread touching global memory for it: one producer lane brings a
// unit's state in with a single bulk copy (completion counted on an mbarrier) two units ahead, together with the
// token's k, q and v vectors; sixteen compute warps update it in place; one store lane sends it back with a single
// bulk store and hands the stage to the producer once it has been read.  (Row-sized copies, 128 each way per unit,
// were measured: the copy engine's rate of operations then bounds the step, 75 us against 57.)  The state sits in the
// stage as it sits in memory, rows of 512 bytes, so a warp owns 8 rows and a lane 4 columns of every one of them
// (16-byte accesses, consecutive lanes consecutive addresses); the sums over the 128 rows are 8 rows in a thread,
// then 16 partial sums per column through shared memory.  (Splitting a head's columns over two CTAs, as the
// single-sequence kernel does, makes each of them touch only half of every DRAM page and costs about half of the
// bandwidth.)  Every mbarrier wait is bounded; when one runs out the warp records RIB200_DEVICE_WAIT_TIMED_OUT, the
// CTA stops waiting and copying and runs to its end.
constexpr int kStageState = kDim * kDim * 4;           // 65 536: the state of one head
constexpr int kStageVectors = 3 * 256;                 // then the token's k, q, v (BF16, 256 bytes each)
constexpr int kStageBytes = kStageState + kStageVectors;
constexpr int kStages = 3;
constexpr int kComputeWarps = 16;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kBatchedThreads = (kComputeWarps + 2) * 32; // + a warp whose lane 0 loads + a warp whose lane 0 stores
constexpr int kPartialFloats = 2 * kComputeWarps * kDim + kComputeWarps + kDim; // a and b partial sums, k.q, delta
constexpr int kBarrierBytes = 3 * kStages * 8;
constexpr int kBatchedSmemBytes = kStages * kStageBytes + kPartialFloats * 4 + kBarrierBytes + 16;
constexpr long long kBatchedWaitLimit = 1LL << 28;
static_assert(kStageBytes % 16 == 0 && kBatchedSmemBytes <= 232448, "stages on 16-byte boundaries, fits an SM");

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
__device__ __forceinline__ void bulk_g2s(std::uint32_t dst, const void *src, std::uint32_t bytes, std::uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, std::uint32_t src, std::uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes)
               : "memory");
}

__global__ void __launch_bounds__(kBatchedThreads, 1)
    gdn_batched_decode_kernel(const RecurrentParams p, std::uint32_t sequences, unsigned int *status) {
  extern __shared__ __align__(16) unsigned char ring[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Work units are (sequence, value head) pairs in that order; the CTAs split them into contiguous ranges whose
  // lengths differ by at most one, so that every SM streams the same number of states (64 sequences x 32 heads
  // over 148 CTAs: 13 or 14 each).
  const std::uint32_t units = sequences * p.value_heads;
  const std::uint32_t unit0 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(units) * blockIdx.x / gridDim.x);
  const std::uint32_t unit1 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(units) * (blockIdx.x + 1) / gridDim.x);
  const std::uint32_t count = unit1 - unit0;
  const std::uint32_t ring_base = static_cast<std::uint32_t>(__cvta_generic_to_shared(ring));
  float *partial = reinterpret_cast<float *>(ring + kStages * kStageBytes); // [2][16 warps][128 columns]
  float *partial_kq = partial + 2 * kComputeWarps * kDim;                   // [16 warps]
  float *shared_delta = partial_kq + kComputeWarps;                         // [128 columns]
  const std::uint32_t bars = ring_base + kStages * kStageBytes + kPartialFloats * 4;
  auto bar_full = [&](std::uint32_t s) { return bars + s * 8; };
  auto bar_computed = [&](std::uint32_t s) { return bars + (kStages + s) * 8; };
  auto bar_drained = [&](std::uint32_t s) { return bars + (2 * kStages + s) * 8; };
  volatile std::uint32_t *abort_flag =
      reinterpret_cast<volatile std::uint32_t *>(ring + kStages * kStageBytes + kPartialFloats * 4 + kBarrierBytes);

  // The state pointers of this CTA's first units are read once: a dependent pointer load in front of every copy
  // would sit on the critical path of each unit.
  constexpr std::uint32_t kKnownPointers = 64;
  __shared__ float *known[kKnownPointers];
  if (threadIdx.x < kKnownPointers && threadIdx.x < count) {
    known[threadIdx.x] = p.states[(unit0 + threadIdx.x) / p.value_heads];
  }
  if (threadIdx.x == 0) {
    for (std::uint32_t s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_computed(s), 1);
      mbar_init(bar_drained(s), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  auto state_of = [&](std::uint32_t n) {
    return (n < kKnownPointers ? known[n] : p.states[(unit0 + n) / p.value_heads]) +
           static_cast<std::size_t>((unit0 + n) % p.value_heads) * kDim * kDim;
  };
  // bounded wait: false when this warp (or another one before it) gave up
  auto wait = [&](std::uint32_t bar, std::uint32_t parity) {
    if (*abort_flag != 0) {
      return false;
    }
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
    const long long started = clock64();
    while (!mbar_try_wait(bar, parity)) {
      if (*abort_flag != 0) {
        return false;
      }
      if (clock64() - started > kBatchedWaitLimit) {
        *abort_flag = 1;
        atomicOr(status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
        return false;
      }
    }
    return true;
  };

  auto compute_barrier = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(kComputeThreads) : "memory"); };
  auto compute_barrier_any = [](bool mine) {
    std::uint32_t any;
    asm volatile("{\n"
                 ".reg .pred in, out;\n"
                 "setp.ne.u32 in, %1, 0;\n"
                 "bar.red.or.pred out, 1, %2, in;\n"
                 "selp.u32 %0, 1, 0, out;\n"
                 "}\n"
                 : "=r"(any)
                 : "r"(static_cast<std::uint32_t>(mine)), "n"(kComputeThreads)
                 : "memory");
    return any != 0;
  };

  if (warp == kComputeWarps) {
    // ---- producer lane: a unit's state as one copy, and the token's three vectors ----
    if (lane == 0) {
      std::uint32_t issued = 0;
      for (std::uint32_t n = 0; n < count; ++n) {
        const std::uint32_t s = n % kStages;
        if (n >= kStages && !wait(bar_drained(s), ((n / kStages) - 1) & 1U)) {
          break;
        }
        const std::size_t item = (unit0 + n) / p.value_heads;
        const std::uint32_t head = (unit0 + n) % p.value_heads;
        const std::uint32_t key_head = head % p.key_heads;
        const std::uint32_t dst = ring_base + s * kStageBytes;
        if ((reinterpret_cast<std::uintptr_t>(state_of(n)) & 15U) != 0) {
          // a bulk copy from an address off a 16-byte boundary would fault: record it and stop the CTA instead
          atomicOr(status, static_cast<unsigned int>(RIB200_DEVICE_POINTER_MISALIGNED));
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(bar_full(s), kStageBytes);
        bulk_g2s(dst, state_of(n), kStageState, bar_full(s));
        bulk_g2s(dst + kStageState, static_cast<const __nv_bfloat16 *>(p.k) + item * p.k_stride + key_head * kDim, 256,
                 bar_full(s));
        bulk_g2s(dst + kStageState + 256, static_cast<const __nv_bfloat16 *>(p.q) + item * p.q_stride + key_head * kDim,
                 256, bar_full(s));
        bulk_g2s(dst + kStageState + 512, static_cast<const __nv_bfloat16 *>(p.v) + item * p.v_stride + head * kDim, 256,
                 bar_full(s));
        issued = n + 1;
      }
      if (*abort_flag != 0) {
        // after giving up: let the copies already issued land before the CTA's shared memory goes away
        for (std::uint32_t n = issued > kStages ? issued - kStages : 0; n < issued; ++n) {
          const long long started = clock64();
          while (!mbar_try_wait(bar_full(n % kStages), (n / kStages) & 1U) && clock64() - started < kBatchedWaitLimit) {
          }
        }
      }
    }
  } else if (warp == kComputeWarps + 1) {
    // ---- store lane: the updated state back as one copy ----
    if (lane == 0) {
      for (std::uint32_t n = 0; n < count; ++n) {
        const std::uint32_t s = n % kStages;
        if (!wait(bar_computed(s), (n / kStages) & 1U)) {
          break;
        }
        bulk_s2g(state_of(n), ring_base + s * kStageBytes, kStageState);
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); // the state has left the stage
        mbar_arrive(bar_drained(s));
      }
      asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    }
  } else {
    // ---- compute warps: warp w owns rows 8 w .. 8 w + 7, lane l columns 4 l .. 4 l + 3 ----
    const int row0 = warp * 8;
    const int col0 = lane * 4;
    auto gates_of = [&](std::uint32_t n, float &beta, float &log_decay) {
      const std::size_t at =
          static_cast<std::size_t>((unit0 + n) / p.value_heads) * p.value_heads + (unit0 + n) % p.value_heads;
      beta = p.beta[at];
      log_decay = p.log_decay[at];
    };
    float beta = 0.0F;
    float log_decay = 0.0F;
    if (count > 0) {
      gates_of(0, beta, log_decay);
    }
    bool healthy = true;
    for (std::uint32_t n = 0; n < count; ++n) {
      const std::uint32_t s = n % kStages;
      const std::size_t item = (unit0 + n) / p.value_heads;
      const std::uint32_t head = (unit0 + n) % p.value_heads;
      float next_beta = 0.0F;
      float next_log_decay = 0.0F;
      if (n + 1 < count) {
        gates_of(n + 1, next_beta, next_log_decay); // in flight while this unit is worked on
      }
      healthy = wait(bar_full(s), (n / kStages) & 1U) && healthy;
      // Every compute thread takes the same way out: the barrier ORs what each of them saw, so a flag that one of
      // the copy lanes raises while the threads pass by cannot send some of them on to a barrier the others skip.
      if (compute_barrier_any(!healthy || *abort_flag != 0)) {
        break;
      }
      unsigned char *stage = ring + s * kStageBytes;
      float kk[8];
      float qq[8];
      {
        const uint4 kraw = *reinterpret_cast<const uint4 *>(stage + kStageState + row0 * 2);
        const uint4 qraw = *reinterpret_cast<const uint4 *>(stage + kStageState + 256 + row0 * 2);
        const std::uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
        const std::uint32_t qw[4] = {qraw.x, qraw.y, qraw.z, qraw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kk[2 * i] = __uint_as_float(kw[i] << 16);
          kk[2 * i + 1] = __uint_as_float(kw[i] & 0xFFFF0000U);
          qq[2 * i] = __uint_as_float(qw[i] << 16);
          qq[2 * i + 1] = __uint_as_float(qw[i] & 0xFFFF0000U);
        }
      }
      const float decay = expf(log_decay);
      float4 st[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        st[r] = *reinterpret_cast<const float4 *>(stage + (row0 + r) * 512 + col0 * 4);
      }
      float4 a = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
      float4 b = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
      float kq = 0.0F;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        a.x += st[r].x * kk[r]; a.y += st[r].y * kk[r]; a.z += st[r].z * kk[r]; a.w += st[r].w * kk[r];
        b.x += st[r].x * qq[r]; b.y += st[r].y * qq[r]; b.z += st[r].z * qq[r]; b.w += st[r].w * qq[r];
        kq += kk[r] * qq[r];
      }
      *reinterpret_cast<float4 *>(partial + warp * kDim + col0) = a;
      *reinterpret_cast<float4 *>(partial + (kComputeWarps + warp) * kDim + col0) = b;
      if (lane == 0) {
        partial_kq[warp] = kq;
      }
      compute_barrier();
      if (threadIdx.x < kDim) {
        // column c: the 16 partial sums, delta, the output
        const int c = threadIdx.x;
        float sum_a = 0.0F;
        float sum_b = 0.0F;
        float sum_kq = 0.0F;
#pragma unroll
        for (int w = 0; w < kComputeWarps; ++w) {
          sum_a += partial[w * kDim + c];
          sum_b += partial[(kComputeWarps + w) * kDim + c];
          sum_kq += partial_kq[w];
        }
        const float vc = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(stage + kStageState + 512)[c]);
        const float delta = (vc - decay * sum_a) * beta;
        shared_delta[c] = delta;
        p.out[(item * p.value_heads + head) * kDim + c] = decay * sum_b + delta * sum_kq;
      }
      compute_barrier();
      const float4 delta = *reinterpret_cast<const float4 *>(shared_delta + col0);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float4 v;
        v.x = decay * st[r].x + kk[r] * delta.x;
        v.y = decay * st[r].y + kk[r] * delta.y;
        v.z = decay * st[r].z + kk[r] * delta.z;
        v.w = decay * st[r].w + kk[r] * delta.w;
        *reinterpret_cast<float4 *>(stage + (row0 + r) * 512 + col0 * 4) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); // the bulk store reads what was just written
      compute_barrier();
      if (threadIdx.x == 0) {
        mbar_arrive(bar_computed(s));
      }
      beta = next_beta;
      log_decay = next_log_decay;
    }
  }
  __syncthreads(); // nobody leaves while copies into or out of the ring may still be under way
}

} // namespace

void launch_gdn_recurrent(const GdnCoreArgs &a, cudaStream_t stream) {
  RecurrentParams p{};
  p.q = a.q;
  p.k = a.k;
  p.v = a.v;
  p.q_stride = a.q_stride;
  p.k_stride = a.k_stride;
  p.v_stride = a.v_stride;
  p.beta = a.beta;
  p.log_decay = a.log_decay;
  p.state = a.state;
  p.states = a.states;
  p.out = a.out;
  p.tokens = a.tokens;
  p.key_heads = a.key_heads;
  p.value_heads = a.value_heads;
  if (a.states != nullptr && a.tokens == 1 && !a.qkv_f32 && a.sequences >= 8) {
    static std::once_flag flags[64];
    int device = 0;
    cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
    require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
    std::call_once(flags[device], [] {
      cuda_ok(cudaFuncSetAttribute(gdn_batched_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kBatchedSmemBytes),
              "gated-delta batched decode shared-memory opt-in");
    });
    // one CTA per SM, each walking its share of the (sequence, head) units
    int sm_count = 148;
    cuda_ok(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device), "SM count query");
    const std::uint32_t units = a.sequences * a.value_heads;
    const std::uint32_t ctas = std::max(1U, std::min(units / 2, static_cast<std::uint32_t>(sm_count)));
    gdn_batched_decode_kernel<<<ctas, kBatchedThreads, kBatchedSmemBytes, stream>>>(p, a.sequences, device_status_word());
    cuda_ok(cudaGetLastError(), "gated-delta batched decode launch");
    return;
  }
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(2, a.value_heads, a.sequences);
  config.blockDim = dim3(256, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  if (a.qkv_f32) {
    cuda_ok(cudaLaunchKernelEx(&config, gdn_recurrent_kernel<true>, p), "gated-delta recurrent launch");
  } else {
    cuda_ok(cudaLaunchKernelEx(&config, gdn_recurrent_kernel<false>, p), "gated-delta recurrent launch");
  }
}

} // namespace rib200
