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

// Batched decode step: one token for each of many sequences.  One CTA of sixteen warps per SM walks an equal share
// of the (sequence, value head) pairs.  A head's whole 64 KiB state - one contiguous block of memory - streams through
// a three-stage cp.async ring in shared memory, so the next sequences' states are in flight while the current one
// is updated; the update is written back into its stage and leaves as full 512-byte rows.  (Splitting a head's
// columns over two CTAs, as the single-sequence kernel does, makes each of them touch only half of every DRAM
// page and costs about half of the bandwidth.)  A warp owns 8 state columns, a lane the rows lane, lane+32,
// lane+64, lane+96; rows sit at a 528-byte pitch, which keeps the 16-byte shared-memory accesses conflict-free.
constexpr int kStagePitch = 528;                     // bytes per state row in shared memory (512 + 16)
constexpr int kStageBytes = kDim * kStagePitch;      // 67 584
constexpr int kStages = 3;
constexpr int kBatchedThreads = 512;
constexpr int kBatchedSmemBytes = kStages * kStageBytes;

__device__ __forceinline__ void cp_async_16(std::uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(std::uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kBatchedThreads, 1)
    gdn_batched_decode_kernel(const RecurrentParams p, std::uint32_t sequences) {
  extern __shared__ __align__(16) unsigned char ring[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int col0 = warp * 8;
  // Work units are (sequence, value head) pairs in that order; the CTAs split them into contiguous ranges whose
  // lengths differ by at most one, so that every SM streams the same number of states (64 sequences x 32 heads
  // over 148 CTAs: 13 or 14 each).
  const std::uint32_t units = sequences * p.value_heads;
  const std::uint32_t unit0 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(units) * blockIdx.x / gridDim.x);
  const std::uint32_t unit1 = static_cast<std::uint32_t>(static_cast<std::uint64_t>(units) * (blockIdx.x + 1) / gridDim.x);
  const std::uint32_t count = unit1 - unit0;
  const std::uint32_t ring_base = static_cast<std::uint32_t>(__cvta_generic_to_shared(ring));

  // The state pointers of this CTA's first units are read once: a dependent pointer load in front of every copy
  // and every write-back would sit on the critical path of each unit.
  constexpr std::uint32_t kKnownPointers = 64;
  __shared__ float *known[kKnownPointers];
  if (threadIdx.x < kKnownPointers && threadIdx.x < count) {
    known[threadIdx.x] = p.states[(unit0 + threadIdx.x) / p.value_heads];
  }
  __syncthreads();
  auto state_of = [&](std::uint32_t n) {
    return n < kKnownPointers ? known[n] : p.states[(unit0 + n) / p.value_heads];
  };

  // copy the head's 128 x 128 state of this CTA's n-th sequence into stage n % kStages
  auto issue = [&](std::uint32_t n) {
    const std::uint32_t seq = (unit0 + n) / p.value_heads;
    const std::uint32_t head = (unit0 + n) % p.value_heads;
    const std::uint32_t key_head = head % p.key_heads;
    const float *src = state_of(n) + static_cast<std::size_t>(head) * kDim * kDim;
    const std::uint32_t dst = ring_base + (n % kStages) * kStageBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + i * kBatchedThreads; // 4096 chunks of 16 bytes
      const int row = idx >> 5;
      const int chunk = idx & 31;
      cp_async_16(dst + row * kStagePitch + chunk * 16, src + row * kDim + chunk * 4);
    }
    // The token's own vectors ride in the 16 spare bytes at the end of the rows (k: rows 0-15, q: 16-31,
    // this head's v: 32-47, beta and the log decay: row 48), so that they arrive with the state, two sequences
    // ahead of their use, instead of as loads queued behind the stream when they are needed.
    const std::size_t item = seq;
    if (threadIdx.x < 48) {
      const int which = threadIdx.x >> 4;
      const int chunk = threadIdx.x & 15;
      const __nv_bfloat16 *vec =
          which == 0   ? static_cast<const __nv_bfloat16 *>(p.k) + item * p.k_stride + key_head * kDim
          : which == 1 ? static_cast<const __nv_bfloat16 *>(p.q) + item * p.q_stride + key_head * kDim
                       : static_cast<const __nv_bfloat16 *>(p.v) + item * p.v_stride + head * kDim;
      cp_async_16(dst + threadIdx.x * kStagePitch + 512, vec + chunk * 8);
    } else if (threadIdx.x == 48) {
      cp_async_4(dst + 48 * kStagePitch + 512, p.beta + item * p.value_heads + head);
    } else if (threadIdx.x == 49) {
      cp_async_4(dst + 48 * kStagePitch + 516, p.log_decay + item * p.value_heads + head);
    }
  };

#pragma unroll
  for (int n = 0; n < kStages - 1; ++n) {
    if (static_cast<std::uint32_t>(n) < count) {
      issue(n);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  }

  for (std::uint32_t n = 0; n < count; ++n) {
    const std::size_t item = (unit0 + n) / p.value_heads;
    const std::uint32_t head = (unit0 + n) % p.value_heads;

    // Stage (n-1) % kStages is refilled next: its write-back was issued by all threads before they arrived here.
    __syncthreads();
    if (n + kStages - 1 < count) {
      issue(n + kStages - 1);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    asm volatile("cp.async.wait_group %0;\n" ::"n"(kStages - 1) : "memory");
    __syncthreads(); // the stage was filled by all threads

    unsigned char *stage = ring + (n % kStages) * kStageBytes;
    // the token's vectors, from the spare bytes of the stage
    float kk[4];
    float qq[4];
    float vlo[4];
    float vhi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      kk[i] = __bfloat162float(
          *reinterpret_cast<const __nv_bfloat16 *>(stage + (e >> 3) * kStagePitch + 512 + (e & 7) * 2));
      qq[i] = __bfloat162float(
          *reinterpret_cast<const __nv_bfloat16 *>(stage + (16 + (e >> 3)) * kStagePitch + 512 + (e & 7) * 2));
    }
    {
      const uint4 raw = *reinterpret_cast<const uint4 *>(stage + (32 + warp) * kStagePitch + 512);
      vlo[0] = __uint_as_float(raw.x << 16);
      vlo[1] = __uint_as_float(raw.x & 0xFFFF0000U);
      vlo[2] = __uint_as_float(raw.y << 16);
      vlo[3] = __uint_as_float(raw.y & 0xFFFF0000U);
      vhi[0] = __uint_as_float(raw.z << 16);
      vhi[1] = __uint_as_float(raw.z & 0xFFFF0000U);
      vhi[2] = __uint_as_float(raw.w << 16);
      vhi[3] = __uint_as_float(raw.w & 0xFFFF0000U);
    }
    const float beta = *reinterpret_cast<const float *>(stage + 48 * kStagePitch + 512);
    const float decay = expf(*reinterpret_cast<const float *>(stage + 48 * kStagePitch + 516));
    float s[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float *row = reinterpret_cast<const float *>(stage + (lane + 32 * i) * kStagePitch) + col0;
      const float4 lo = *reinterpret_cast<const float4 *>(row);
      const float4 hi = *reinterpret_cast<const float4 *>(row + 4);
      s[i][0] = lo.x; s[i][1] = lo.y; s[i][2] = lo.z; s[i][3] = lo.w;
      s[i][4] = hi.x; s[i][5] = hi.y; s[i][6] = hi.z; s[i][7] = hi.w;
    }
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
    // new state back into the stage, then out as whole rows
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float *row = reinterpret_cast<float *>(stage + (lane + 32 * i) * kStagePitch) + col0;
      float4 lo;
      float4 hi;
      lo.x = decay * s[i][0] + kk[i] * delta[0];
      lo.y = decay * s[i][1] + kk[i] * delta[1];
      lo.z = decay * s[i][2] + kk[i] * delta[2];
      lo.w = decay * s[i][3] + kk[i] * delta[3];
      hi.x = decay * s[i][4] + kk[i] * delta[4];
      hi.y = decay * s[i][5] + kk[i] * delta[5];
      hi.z = decay * s[i][6] + kk[i] * delta[6];
      hi.w = decay * s[i][7] + kk[i] * delta[7];
      *reinterpret_cast<float4 *>(row) = lo;
      *reinterpret_cast<float4 *>(row + 4) = hi;
    }
    if (lane == 0) {
      float *dst = p.out + (item * p.value_heads + head) * kDim + col0;
      *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<float4 *>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
    __syncthreads(); // the whole updated state is in the stage
    float *state = state_of(n) + static_cast<std::size_t>(head) * kDim * kDim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = threadIdx.x + i * kBatchedThreads;
      const int row = idx >> 5;
      const int chunk = idx & 31;
      *reinterpret_cast<float4 *>(state + row * kDim + chunk * 4) =
          *reinterpret_cast<const float4 *>(stage + row * kStagePitch + chunk * 16);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
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
    gdn_batched_decode_kernel<<<ctas, kBatchedThreads, kBatchedSmemBytes, stream>>>(p, a.sequences);
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
