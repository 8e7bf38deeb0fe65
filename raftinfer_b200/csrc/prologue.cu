// The step in front of both attention kernels: de-interleave the query/gate projection, per-head RMSNorm with
// weight, partial NeoX-style RoPE on q and k, and the casts of gate and v.  The reference runs it as three launches
// with their intermediates in global memory (cpp/execution/qwen35_executor.cu:1989-2015 calling
// cpp/kernels/qwen35_primitives.cu:159-209 qk_norm_rope_kernel and :367-385 split_full_query_gate_kernel; CPU form
// cpp/reference/qwen35.cpp:125-186,298-313).  Here one launch reads the projections once and writes q, gate, k, v in
// the dtype the attention kernels take.  The two reference entry points are also served, by the same kernel.
//
// HBM-bound: every element is read once and written once.  Bytes per token: (2 Hq + 2 Hkv) D input elements plus
// the same number of output elements.  One CTA per token: its first warp computes the token's rotary_dim / 2
// (cos, sin) pairs once (angle formed and reduced in double, as the CPU reference forms it) and every head of the
// token reuses them; a
// warp then owns one head vector at a time, a lane 8 (or 4) consecutive dims, so loads and stores are whole
// 16/32-byte pieces and the sum of squares is five shuffles.  The rotation partner of dim i is dim i +- rotary/2,
// which sits at the same place in a lane rotary / 2 / dims-per-lane further on: one shuffle per element.

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

namespace rib200 {
namespace {

constexpr int kMaxPairs = 128;
constexpr int kPrologueThreads = 256;

struct PrologueParams {
  // q: vectors of `q_heads` heads per token, `q_head_stride` elements apart (2 D when the gate is interleaved)
  const void *q_in;
  const void *k_in;
  const void *v_in; // null: no cast of v
  const void *q_weight;
  const void *k_weight;
  void *q_out;
  void *gate_out; // null: the input holds no gate
  void *k_out;
  void *v_out;
  std::uint32_t tokens;
  std::uint32_t q_heads;
  std::uint32_t kv_heads; // 0: only q vectors
  std::uint32_t q_head_stride;
  std::uint32_t rotary_dim;
  std::uint64_t position_offset;
  const std::uint32_t *device_position;
  float epsilon;
  double inv_freq[kMaxPairs]; // base^(-2 p / rotary_dim)
};

template <class T> struct Elements;
template <> struct Elements<float> {
  template <int N> static __device__ __forceinline__ void load(const void *base, std::size_t index, float (&x)[N]) {
    const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + index);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const float4 v = src[i];
      x[4 * i] = v.x;
      x[4 * i + 1] = v.y;
      x[4 * i + 2] = v.z;
      x[4 * i + 3] = v.w;
    }
  }
  template <int N> static __device__ __forceinline__ void store(void *base, std::size_t index, const float (&x)[N]) {
    float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(base) + index);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      dst[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    }
  }
};
template <> struct Elements<__nv_bfloat16> {
  template <int N> static __device__ __forceinline__ void load(const void *base, std::size_t index, float (&x)[N]) {
    if constexpr (N % 8 == 0) { // eight elements per 16-byte access
      const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(base) + index);
#pragma unroll
      for (int i = 0; i < N / 8; ++i) {
        const uint4 v = src[i];
        const std::uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          x[8 * i + 2 * h] = __uint_as_float(w[h] << 16);
          x[8 * i + 2 * h + 1] = __uint_as_float(w[h] & 0xFFFF0000U);
        }
      }
      return;
    }
    const uint2 *src = reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + index);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const uint2 v = src[i];
      x[4 * i] = __uint_as_float(v.x << 16);
      x[4 * i + 1] = __uint_as_float(v.x & 0xFFFF0000U);
      x[4 * i + 2] = __uint_as_float(v.y << 16);
      x[4 * i + 3] = __uint_as_float(v.y & 0xFFFF0000U);
    }
  }
  template <int N> static __device__ __forceinline__ void store(void *base, std::size_t index, const float (&x)[N]) {
    if constexpr (N % 8 == 0) {
      uint4 *wide = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(base) + index);
#pragma unroll
      for (int i = 0; i < N / 8; ++i) {
        std::uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const __nv_bfloat162 pair = __floats2bfloat162_rn(x[8 * i + 2 * h], x[8 * i + 2 * h + 1]);
          w[h] = *reinterpret_cast<const std::uint32_t *>(&pair);
        }
        wide[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      return;
    }
    uint2 *dst = reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(base) + index);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(x[4 * i], x[4 * i + 1]);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(x[4 * i + 2], x[4 * i + 3]);
      dst[i] = make_uint2(*reinterpret_cast<const std::uint32_t *>(&lo), *reinterpret_cast<const std::uint32_t *>(&hi));
    }
  }
};

// In: projection dtype, W: norm-weight dtype, Out: output dtype, PerLane: head_dim / 32
template <class In, class W, class Out, int PerLane>
__global__ void __launch_bounds__(kPrologueThreads) attention_prologue_kernel(const PrologueParams p) {
  __shared__ float rope_cos[kMaxPairs];
  __shared__ float rope_sin[kMaxPairs];
  constexpr int kHeadDimT = 32 * PerLane;
  const std::uint32_t token = blockIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const std::uint32_t pairs = p.rotary_dim / 2;

  const std::uint32_t vectors = p.q_heads + 2 * p.kv_heads; // q heads, then k heads, then v heads
  const std::uint32_t lane_dim = lane * PerLane;
  const std::uint32_t partner_lanes = pairs / PerLane; // lanes between a dim and its rotation partner

  // A warp's vectors are fetched one ahead of their use: the loads of the first are in flight while the angles
  // are computed, those of the next while the current one is normalised and rotated.
  struct Fetched {
    float x[PerLane];
    float gate[PerLane];
  };
  float q_w[PerLane];
  float k_w[PerLane];
  Elements<W>::template load<PerLane>(p.q_weight, lane_dim, q_w);
  if (p.kv_heads != 0) {
    Elements<W>::template load<PerLane>(p.k_weight, lane_dim, k_w);
  }
  auto fetch = [&](std::uint32_t vec, Fetched &f) {
    if (vec >= p.q_heads + p.kv_heads) {
      if (p.v_in != nullptr) {
        const std::uint32_t head = vec - p.q_heads - p.kv_heads;
        const std::size_t at = (static_cast<std::size_t>(token) * p.kv_heads + head) * kHeadDimT + lane_dim;
        Elements<In>::template load<PerLane>(p.v_in, at, f.x);
      }
      return;
    }
    const bool is_q = vec < p.q_heads;
    const std::uint32_t head = is_q ? vec : vec - p.q_heads;
    const std::size_t in_at = is_q ? (static_cast<std::size_t>(token) * p.q_heads + head) * p.q_head_stride + lane_dim
                                   : (static_cast<std::size_t>(token) * p.kv_heads + head) * kHeadDimT + lane_dim;
    Elements<In>::template load<PerLane>(is_q ? p.q_in : p.k_in, in_at, f.x);
    if (is_q && p.gate_out != nullptr) {
      Elements<In>::template load<PerLane>(p.q_in, in_at + kHeadDimT, f.gate);
    }
  };
  auto finish = [&](std::uint32_t vec, Fetched &f) {
    if (vec >= p.q_heads + p.kv_heads) {
      if (p.v_in != nullptr) { // v: a cast
        const std::uint32_t head = vec - p.q_heads - p.kv_heads;
        const std::size_t at = (static_cast<std::size_t>(token) * p.kv_heads + head) * kHeadDimT + lane_dim;
        Elements<Out>::template store<PerLane>(p.v_out, at, f.x);
      }
      return;
    }
    const bool is_q = vec < p.q_heads;
    const std::uint32_t head = is_q ? vec : vec - p.q_heads;
    const std::size_t out_at =
        (static_cast<std::size_t>(token) * (is_q ? p.q_heads : p.kv_heads) + head) * kHeadDimT + lane_dim;
    if (is_q && p.gate_out != nullptr) {
      Elements<Out>::template store<PerLane>(p.gate_out, out_at, f.gate);
    }
    // RMSNorm: mean square (FP32 tree; the CPU reference sums in double, the difference is a few 1e-8 relative),
    // scale 1 / sqrt(mean + epsilon) in float as the reference
    float sum = 0.0F;
#pragma unroll
    for (int i = 0; i < PerLane; ++i) {
      sum += f.x[i] * f.x[i];
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      sum += __shfl_xor_sync(0xFFFFFFFFU, sum, offset);
    }
    const float scale = 1.0F / sqrtf(sum * (1.0F / static_cast<float>(kHeadDimT)) + p.epsilon);
#pragma unroll
    for (int i = 0; i < PerLane; ++i) {
      f.x[i] = f.x[i] * scale * (is_q ? q_w[i] : k_w[i]);
    }
    // partial RoPE, pairs (i, i + rotary / 2): every lane takes part in the shuffles, the rotary lanes use them
    const bool first_half = lane_dim < pairs;
    const bool rotates = lane_dim < p.rotary_dim;
    const int source = first_half ? lane + static_cast<int>(partner_lanes) : lane - static_cast<int>(partner_lanes);
#pragma unroll
    for (int i = 0; i < PerLane; ++i) {
      const float partner = __shfl_sync(0xFFFFFFFFU, f.x[i], source & 31);
      if (rotates) {
        const std::uint32_t pair = (first_half ? lane_dim : lane_dim - pairs) + i;
        const float c = rope_cos[pair];
        const float s = rope_sin[pair];
        f.x[i] = first_half ? f.x[i] * c - partner * s : partner * s + f.x[i] * c;
      }
    }
    Elements<Out>::template store<PerLane>(is_q ? p.q_out : p.k_out, out_at, f.x);
  };

  Fetched current;
  if (static_cast<std::uint32_t>(warp) < vectors) {
    fetch(warp, current);
  }
  // the token's angles, once: theta = position * base^(-2 pair / rotary), cos and sin taken in double
  {
    const std::uint64_t position =
        (p.device_position != nullptr ? static_cast<std::uint64_t>(*p.device_position) : p.position_offset) + token;
    for (std::uint32_t pair = threadIdx.x; pair < pairs; pair += kPrologueThreads) {
      // the angle in double, brought into [-pi, pi] in double, then the float sine and cosine of that
      const double theta = static_cast<double>(position) * p.inv_freq[pair];
      const double turns = rint(theta * 0.15915494309189535);
      const float reduced = static_cast<float>(fma(turns, -6.283185307179586, theta));
      float s;
      float c;
      sincosf(reduced, &s, &c);
      rope_cos[pair] = c;
      rope_sin[pair] = s;
    }
  }
  __syncthreads();
  constexpr std::uint32_t kWarps = kPrologueThreads / 32;
  for (std::uint32_t vec = warp; vec < vectors; vec += kWarps) {
    Fetched next;
    if (vec + kWarps < vectors) {
      fetch(vec + kWarps, next);
    }
    finish(vec, current);
    current = next;
  }
}

template <class T>
__global__ void split_query_gate_kernel(const T *query_gate, T *query, T *gate, std::size_t total_vec,
                                        std::uint32_t vec_per_head) {
  // one thread per 16-byte piece of the output
  const std::size_t index = static_cast<std::size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total_vec) {
    return;
  }
  const std::size_t head = index / vec_per_head;
  const std::size_t piece = index - head * vec_per_head;
  const uint4 *src = reinterpret_cast<const uint4 *>(query_gate) + head * 2 * vec_per_head + piece;
  reinterpret_cast<uint4 *>(query)[index] = src[0];
  reinterpret_cast<uint4 *>(gate)[index] = src[vec_per_head];
}

template <class In, class W, class Out> void launch_typed(const PrologueParams &p, int per_lane, cudaStream_t stream) {
  if (per_lane == 8) {
    attention_prologue_kernel<In, W, Out, 8><<<p.tokens, kPrologueThreads, 0, stream>>>(p);
  } else {
    attention_prologue_kernel<In, W, Out, 4><<<p.tokens, kPrologueThreads, 0, stream>>>(p);
  }
  cuda_ok(cudaGetLastError(), "attention prologue launch");
}

void launch_prologue(const PrologueParams &p, std::size_t head_dim, int32_t in_dtype, int32_t weight_dtype,
                     int32_t out_dtype, cudaStream_t stream) {
  const int per_lane = static_cast<int>(head_dim / 32);
  const bool in32 = in_dtype == RIB200_DTYPE_F32;
  const bool w32 = weight_dtype == RIB200_DTYPE_F32;
  const bool out32 = out_dtype == RIB200_DTYPE_F32;
  if (in32 && w32 && out32) {
    launch_typed<float, float, float>(p, per_lane, stream);
  } else if (in32 && w32) {
    launch_typed<float, float, __nv_bfloat16>(p, per_lane, stream);
  } else if (in32 && !w32 && out32) {
    launch_typed<float, __nv_bfloat16, float>(p, per_lane, stream);
  } else if (in32) {
    launch_typed<float, __nv_bfloat16, __nv_bfloat16>(p, per_lane, stream);
  } else if (w32) {
    launch_typed<__nv_bfloat16, float, __nv_bfloat16>(p, per_lane, stream);
  } else {
    launch_typed<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(p, per_lane, stream);
  }
}

void check_rope(std::size_t head_dim, std::size_t rotary_dim, float rope_base, float epsilon, const char *who) {
  (void)who;
  require(head_dim > 0, "qk_norm_rope head_dim must be positive");
  require(rotary_dim > 0, "qk_norm_rope rotary_dim must be positive");
  require(rotary_dim <= head_dim, "qk_norm_rope rotary_dim exceeds head_dim");
  require(rotary_dim % 2 == 0, "qk_norm_rope rotary_dim must be even");
  require(std::isfinite(rope_base) && rope_base > 0.0F, "qk_norm_rope rope_base must be finite and positive");
  require(std::isfinite(epsilon) && epsilon >= 0.0F, "qk_norm_rope epsilon must be finite and non-negative");
  unsupported(head_dim == 256 || head_dim == 128, "qk_norm_rope: built for head_dim 128 and 256");
  unsupported((rotary_dim / 2) % (head_dim / 32) == 0 && rotary_dim / 2 <= kMaxPairs,
              "qk_norm_rope: rotary_dim / 2 must be a multiple of head_dim / 32");
}

void fill_frequencies(PrologueParams &p, std::size_t rotary_dim, float rope_base) {
  for (std::size_t pair = 0; pair < rotary_dim / 2; ++pair) {
    const double exponent = static_cast<double>(2 * pair) / static_cast<double>(rotary_dim);
    p.inv_freq[pair] = 1.0 / std::pow(static_cast<double>(rope_base), exponent);
  }
}

void check_dtypes(int32_t dtype, int32_t weight_dtype) {
  require(dtype == RIB200_DTYPE_F32 || dtype == RIB200_DTYPE_BF16, "unsupported activation dtype");
  require(weight_dtype == RIB200_DTYPE_F32 || weight_dtype == RIB200_DTYPE_BF16 || weight_dtype == RIB200_DTYPE_F16,
          "unsupported weight dtype");
  unsupported(weight_dtype != RIB200_DTYPE_F16, "qk_norm_rope: FP16 norm weights are not built");
}

void aligned(const void *ptr, const char *message) {
  require(reinterpret_cast<std::uintptr_t>(ptr) % 16 == 0, message);
}

} // namespace
} // namespace rib200

using namespace rib200;

extern "C" Rib200Status rib200_qk_norm_rope(const void *input, const void *weight, void *output,
                                            const Rib200QkNormRopeShape *shape, float epsilon, int32_t dtype,
                                            int32_t weight_dtype, void *stream, const uint32_t *device_position) {
  return guarded([&] {
    require(input != nullptr, "qk_norm_rope input pointer is null");
    require(weight != nullptr, "qk_norm_rope weight pointer is null");
    require(output != nullptr, "qk_norm_rope output pointer is null");
    require(shape != nullptr, "qk_norm_rope shape pointer is null");
    const Rib200QkNormRopeShape &s = *shape;
    require(s.tokens > 0, "qk_norm_rope tokens must be positive");
    require(s.heads > 0, "qk_norm_rope heads must be positive");
    check_rope(s.head_dim, s.rotary_dim, s.rope_base, epsilon, "qk_norm_rope");
    require(s.position_offset <= std::numeric_limits<std::size_t>::max() - (s.tokens - 1),
            "qk_norm_rope position range overflow");
    require(stream != nullptr, "CUDA stream is null");
    check_dtypes(dtype, weight_dtype);
    (void)mul(mul(s.tokens, s.heads, "qk_norm_rope vector overflow"), s.head_dim, "qk_norm_rope shape overflow");
    require(s.tokens <= 0x7FFFFFFFU && s.heads <= 0xFFFFU, "qk_norm_rope grid dimension overflow");
    aligned(input, "qk_norm_rope input is not 16-byte aligned");
    aligned(weight, "qk_norm_rope weight is not 16-byte aligned");
    aligned(output, "qk_norm_rope output is not 16-byte aligned");
    PrologueParams p{};
    p.q_in = input;
    p.q_weight = weight;
    p.q_out = output;
    p.tokens = static_cast<std::uint32_t>(s.tokens);
    p.q_heads = static_cast<std::uint32_t>(s.heads);
    p.kv_heads = 0;
    p.q_head_stride = static_cast<std::uint32_t>(s.head_dim);
    p.rotary_dim = static_cast<std::uint32_t>(s.rotary_dim);
    p.position_offset = s.position_offset;
    p.device_position = device_position;
    p.epsilon = epsilon;
    fill_frequencies(p, s.rotary_dim, s.rope_base);
    launch_prologue(p, s.head_dim, dtype, weight_dtype, dtype, static_cast<cudaStream_t>(stream));
  });
}

extern "C" Rib200Status rib200_split_full_query_gate(const void *query_gate, void *query, void *gate, size_t tokens,
                                                     size_t heads, size_t head_dim, int32_t dtype, void *stream) {
  return guarded([&] {
    require(query_gate != nullptr, "split_full_query_gate input pointer is null");
    require(query != nullptr, "split_full_query_gate query pointer is null");
    require(gate != nullptr, "split_full_query_gate gate pointer is null");
    require(tokens > 0, "split_full_query_gate tokens must be positive");
    require(heads > 0, "split_full_query_gate heads must be positive");
    require(head_dim > 0, "split_full_query_gate head_dim must be positive");
    require(stream != nullptr, "CUDA stream is null");
    require(dtype == RIB200_DTYPE_F32 || dtype == RIB200_DTYPE_BF16, "unsupported activation dtype");
    const std::size_t hidden = mul(heads, head_dim, "split_full_query_gate hidden overflow");
    const std::size_t total = mul(tokens, hidden, "split_full_query_gate shape overflow");
    const std::size_t element = dtype == RIB200_DTYPE_F32 ? 4 : 2;
    unsupported(head_dim * element % 16 == 0, "split_full_query_gate: a head must be a whole number of 16-byte pieces");
    aligned(query_gate, "split_full_query_gate input is not 16-byte aligned");
    aligned(query, "split_full_query_gate query is not 16-byte aligned");
    aligned(gate, "split_full_query_gate gate is not 16-byte aligned");
    const std::size_t total_vec = total * element / 16;
    const std::uint32_t vec_per_head = static_cast<std::uint32_t>(head_dim * element / 16);
    const std::size_t blocks = (total_vec + 255) / 256;
    require(blocks <= 0x7FFFFFFFU, "split_full_query_gate grid dimension overflow");
    split_query_gate_kernel<uint4><<<static_cast<unsigned int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(query_gate), static_cast<uint4 *>(query), static_cast<uint4 *>(gate), total_vec,
        vec_per_head);
    cuda_ok(cudaGetLastError(), "split_full_query_gate launch");
  });
}

extern "C" Rib200Status rib200_attention_prologue(const void *query_gate, const void *key, const void *value,
                                                  const void *query_norm_weight, const void *key_norm_weight,
                                                  void *query, void *gate, void *key_out, void *value_out,
                                                  const Rib200AttentionShape *shape, size_t rotary_dim,
                                                  float rope_base, float epsilon, int32_t dtype, int32_t weight_dtype,
                                                  int32_t output_dtype, const uint32_t *device_position,
                                                  void *stream) {
  return guarded([&] {
    require(shape != nullptr, "attention prologue: shape pointer is null");
    const Rib200AttentionShape &s = *shape;
    for (const void *ptr : {query_gate, key, value, query_norm_weight, key_norm_weight,
                            static_cast<const void *>(query), static_cast<const void *>(gate),
                            static_cast<const void *>(key_out), static_cast<const void *>(value_out)}) {
      require(ptr != nullptr, "attention prologue: a tensor pointer is null");
      aligned(ptr, "attention prologue: a tensor is not 16-byte aligned");
    }
    require(s.tokens > 0 && s.query_heads > 0 && s.kv_heads > 0, "attention prologue: sizes must be positive");
    check_rope(s.head_dim, rotary_dim, rope_base, epsilon, "attention prologue");
    require(stream != nullptr, "CUDA stream is null");
    check_dtypes(dtype, weight_dtype);
    require(output_dtype == RIB200_DTYPE_BF16 || output_dtype == dtype,
            "attention prologue: outputs are BF16 or the input dtype");
    require(s.tokens <= 0x7FFFFFFFU && s.query_heads <= 0xFFFFU && s.kv_heads <= 0xFFFFU,
            "attention prologue: grid dimension overflow");
    PrologueParams p{};
    p.q_in = query_gate;
    p.k_in = key;
    p.v_in = value;
    p.q_weight = query_norm_weight;
    p.k_weight = key_norm_weight;
    p.q_out = query;
    p.gate_out = gate;
    p.k_out = key_out;
    p.v_out = value_out;
    p.tokens = static_cast<std::uint32_t>(s.tokens);
    p.q_heads = static_cast<std::uint32_t>(s.query_heads);
    p.kv_heads = static_cast<std::uint32_t>(s.kv_heads);
    p.q_head_stride = static_cast<std::uint32_t>(2 * s.head_dim);
    p.rotary_dim = static_cast<std::uint32_t>(rotary_dim);
    p.position_offset = s.past_tokens;
    p.device_position = device_position;
    p.epsilon = epsilon;
    fill_frequencies(p, rotary_dim, rope_base);
    launch_prologue(p, s.head_dim, dtype, weight_dtype, output_dtype, static_cast<cudaStream_t>(stream));
  });
}
