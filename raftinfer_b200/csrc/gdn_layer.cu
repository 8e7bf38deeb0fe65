// The steps of qwen35_gated_delta on either side of the recurrence, for key_dim = value_dim = 128:
//   prologue  depthwise causal convolution + SiLU over the q|k|v channels, L2 normalisation of every q
//             and k head (q also scaled by 1/sqrt(128)), beta = sigmoid(b), log decay = A * softplus(a + dt)
//             (cpp/kernels/qwen35_delta.cu:236-276,375-411,522-529; CPU cpp/reference/qwen35.cpp:417-469);
//   state     shift of the convolution history [channel][W-1] (cpp/kernels/qwen35_delta.cu:267-275);
//   epilogue  per-head RMSNorm(128) * weight * SiLU(z) (cpp/kernels/qwen35_delta.cu:579-621).
// Unlike the reference's convolution kernel, which walks the tokens serially per channel, every
// (token, head vector) pair is independent: a tap is read from the token stream or, for the first W-1
// tokens, from the carried history.  conv_width 4 on aligned tensors takes the warp-per-vector kernels
// (16-byte accesses); other widths and odd alignments take the one-CTA-per-vector kernels.

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace rib200 {
namespace {

constexpr int kDim = 128;
constexpr float kQkEpsilon = 1.0e-6F;

__device__ __forceinline__ float load_any(const void *base, std::size_t index, int32_t dtype) {
  if (dtype == RIB200_DTYPE_F32) {
    return static_cast<const float *>(base)[index];
  }
  if (dtype == RIB200_DTYPE_F16) {
    return __half2float(static_cast<const __half *>(base)[index]);
  }
  return __bfloat162float(static_cast<const __nv_bfloat16 *>(base)[index]);
}

__device__ __forceinline__ void store_any(void *base, std::size_t index, int32_t dtype, float value) {
  if (dtype == RIB200_DTYPE_F32) {
    static_cast<float *>(base)[index] = value;
  } else if (dtype == RIB200_DTYPE_F16) {
    static_cast<__half *>(base)[index] = __float2half_rn(value);
  } else {
    static_cast<__nv_bfloat16 *>(base)[index] = __float2bfloat16_rn(value);
  }
}

__device__ __forceinline__ float silu(float x) { return x / (1.0F + expf(-x)); }

__device__ __forceinline__ float softplus(float x) {
  if (x > 20.0F) {
    return x;
  }
  if (x < -20.0F) {
    return expf(x);
  }
  return log1pf(expf(x));
}

// sum over the 128 threads of the block, returned to all of them
__device__ __forceinline__ float block_sum_128(float value, float *scratch) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    value += __shfl_xor_sync(0xFFFFFFFFU, value, offset);
  }
  if ((threadIdx.x & 31) == 0) {
    scratch[threadIdx.x >> 5] = value;
  }
  __syncthreads();
  return (scratch[0] + scratch[1]) + (scratch[2] + scratch[3]);
}

struct LayerParams {
  const void *input;
  const void *conv_weight, *recurrent_a, *dt_bias, *output_norm_weight;
  void *output;
  float *convolution_state;
  float *convolved;
  float *beta;
  float *log_decay;
  const float *raw;
  std::uint32_t tokens, key_heads, value_heads, conv_width;
  std::uint32_t conv_dim, token_stride;
  float epsilon;
  int32_t dtype, weight_dtype;
};

// grid (2*Hk + Hv head vectors, tokens), 128 threads = the 128 channels of the vector
__global__ void __launch_bounds__(kDim) gdn_prologue_kernel(const LayerParams p) {
  __shared__ float scratch[4];
  const std::uint32_t vec = blockIdx.x;
  const std::uint32_t tok = blockIdx.y;
  const std::uint32_t channel = vec * kDim + threadIdx.x;
  const std::uint32_t history = p.conv_width - 1;
  const std::size_t weight_base = static_cast<std::size_t>(channel) * p.conv_width;
  float sum = load_any(p.input, static_cast<std::size_t>(tok) * p.token_stride + channel, p.dtype) *
              load_any(p.conv_weight, weight_base + history, p.weight_dtype);
  for (std::uint32_t h = 0; h < history; ++h) {
    const std::uint32_t source = tok + h; // position in [history | tokens]
    const float previous =
        source < history
            ? p.convolution_state[static_cast<std::size_t>(channel) * history + source]
            : load_any(p.input, static_cast<std::size_t>(source - history) * p.token_stride + channel, p.dtype);
    sum += previous * load_any(p.conv_weight, weight_base + h, p.weight_dtype);
  }
  float value = silu(sum);
  if (vec < 2 * p.key_heads) {
    const float squares = block_sum_128(value * value, scratch);
    value *= rsqrtf(squares + kQkEpsilon);
    if (vec < p.key_heads) {
      value *= rsqrtf(static_cast<float>(kDim));
    }
  } else if (threadIdx.x == 0) {
    const std::uint32_t head = vec - 2 * p.key_heads;
    const std::size_t gates = static_cast<std::size_t>(tok) * p.token_stride + p.conv_dim;
    const float b = load_any(p.input, gates + head, p.dtype);
    const float a = load_any(p.input, gates + p.value_heads + head, p.dtype);
    p.beta[static_cast<std::size_t>(tok) * p.value_heads + head] = 1.0F / (1.0F + expf(-b));
    p.log_decay[static_cast<std::size_t>(tok) * p.value_heads + head] =
        load_any(p.recurrent_a, head, p.weight_dtype) * softplus(a + load_any(p.dt_bias, head, p.weight_dtype));
  }
  p.convolved[static_cast<std::size_t>(tok) * p.conv_dim + channel] = value;
}

// ---- fast forms for conv_width == 4 (the model's width) ---------------------------------------------
// A warp owns one head vector (128 channels, four per lane) over four consecutive tokens: the seven input rows
// it needs are fetched once, 8 or 16 bytes per lane and row, whole 256/512-byte segments per warp, and slide
// through registers; the sum of squares of a q or k vector is five shuffles.  Dtype is a template parameter.
template <int Dtype> struct Io;
template <> struct Io<RIB200_DTYPE_F32> {
  static __device__ __forceinline__ float4 load4(const void *base, std::size_t index) {
    return *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + index);
  }
  static __device__ __forceinline__ void store4(void *base, std::size_t index, float4 v) {
    *reinterpret_cast<float4 *>(static_cast<float *>(base) + index) = v;
  }
};
template <> struct Io<RIB200_DTYPE_BF16> {
  static __device__ __forceinline__ float4 load4(const void *base, std::size_t index) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + index);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000U),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000U));
  }
  static __device__ __forceinline__ void store4(void *base, std::size_t index, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(base) + index) =
        make_uint2(*reinterpret_cast<const std::uint32_t *>(&lo), *reinterpret_cast<const std::uint32_t *>(&hi));
  }
};
template <> struct Io<RIB200_DTYPE_F16> {
  static __device__ __forceinline__ float4 load4(const void *base, std::size_t index) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(static_cast<const __half *>(base) + index);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
  static __device__ __forceinline__ void store4(void *base, std::size_t index, float4 v) {
    const __half2 lo = __floats2half2_rn(v.x, v.y);
    const __half2 hi = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(static_cast<__half *>(base) + index) =
        make_uint2(*reinterpret_cast<const std::uint32_t *>(&lo), *reinterpret_cast<const std::uint32_t *>(&hi));
  }
};

// SiLU on the special-function unit (ex2 + rcp instead of a full-precision exponential and division): the vector
// kernels are bound by instruction issue otherwise.  Relative error about 1e-6.
__device__ __forceinline__ float silu_fast(float x) {
  float e;
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(x * -1.4426950408889634F));
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(1.0F + e));
  return x * r;
}

constexpr int kTokensPerWarp = 4;  // tokens of one step of a warp
constexpr int kStepsPerWarp = 4;   // steps a warp walks: its window of input rows slides, nothing is read twice
constexpr int kFastWidth = 4;

// grid (ceil(tokens / 16), ceil((2 Hk + Hv + 1) / 8)), 256 threads: warp w of the CTA takes head vector
// 8 blockIdx.y + w over 16 consecutive tokens, four at a time; the rows of the next four are in flight while the
// current four are convolved, and the last three rows of a step are the history of the next.  The vector after the
// last one stands for the gates (lane = value head, any head count).
template <int Dtype> __global__ void __launch_bounds__(256, 3) gdn_prologue_w4_kernel(const LayerParams p) {
  grid_dependents_may_launch(); // the kernels behind this one set themselves up early and wait for it to end
  const int lane = threadIdx.x & 31;
  const std::uint32_t vec = blockIdx.y * 8 + (threadIdx.x >> 5);
  const std::uint32_t vectors = 2 * p.key_heads + p.value_heads;
  const std::uint32_t first = blockIdx.x * (kTokensPerWarp * kStepsPerWarp);
  if (vec > vectors) {
    return;
  }
  if (vec == vectors) {
    for (std::uint32_t head = lane; head < p.value_heads; head += 32) {
      const float a_coeff = load_any(p.recurrent_a, head, p.weight_dtype);
      const float dt = load_any(p.dt_bias, head, p.weight_dtype);
      for (std::uint32_t tok = first; tok < min(p.tokens, first + kTokensPerWarp * kStepsPerWarp); ++tok) {
        const std::size_t gates = static_cast<std::size_t>(tok) * p.token_stride + p.conv_dim;
        const float b = load_any(p.input, gates + head, p.dtype);
        const float a = load_any(p.input, gates + p.value_heads + head, p.dtype);
        p.beta[static_cast<std::size_t>(tok) * p.value_heads + head] = 1.0F / (1.0F + expf(-b));
        p.log_decay[static_cast<std::size_t>(tok) * p.value_heads + head] = a_coeff * softplus(a + dt);
      }
    }
    return;
  }
  const std::uint32_t channel = vec * kDim + 4 * lane;
  // taps of this lane's four channels: weight[channel][4], oldest first
  float w[4][kFastWidth];
  if (p.weight_dtype == RIB200_DTYPE_F32) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float4 taps = *reinterpret_cast<const float4 *>(static_cast<const float *>(p.conv_weight) +
                                                            static_cast<std::size_t>(channel + c) * kFastWidth);
      w[c][0] = taps.x;
      w[c][1] = taps.y;
      w[c][2] = taps.z;
      w[c][3] = taps.w;
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int h = 0; h < kFastWidth; ++h) {
        w[c][h] = load_any(p.conv_weight, static_cast<std::size_t>(channel + c) * kFastWidth + h, p.weight_dtype);
      }
    }
  }
  auto load_row = [&](long long tok) {
    if (tok >= 0 && tok < static_cast<long long>(p.tokens)) {
      return Io<Dtype>::load4(p.input, static_cast<std::size_t>(tok) * p.token_stride + channel);
    }
    return make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  };
  // window: x[0..2] the three rows before the step, x[3..6] the step's own rows
  float4 x[kTokensPerWarp + kFastWidth - 1];
#pragma unroll
  for (int r = 0; r < kTokensPerWarp + kFastWidth - 1; ++r) {
    x[r] = load_row(static_cast<long long>(first) + r - (kFastWidth - 1));
  }
  if (first == 0) {
    // history [channel][3]: element h is the token 3 - h steps before this call's first one
    const float *hist = p.convolution_state + static_cast<std::size_t>(channel) * (kFastWidth - 1);
#pragma unroll
    for (int h = 0; h < kFastWidth - 1; ++h) {
      x[h] = make_float4(hist[h], hist[(kFastWidth - 1) + h], hist[2 * (kFastWidth - 1) + h],
                         hist[3 * (kFastWidth - 1) + h]);
    }
  }
  const bool is_qk = vec < 2 * p.key_heads;
  const float q_scale = vec < p.key_heads ? rsqrtf(static_cast<float>(kDim)) : 1.0F;
#pragma unroll
  for (int step = 0; step < kStepsPerWarp; ++step) {
    const std::uint32_t tok0 = first + step * kTokensPerWarp;
    if (tok0 >= p.tokens) {
      break;
    }
    float4 next[kTokensPerWarp];
    if (step + 1 < kStepsPerWarp) {
#pragma unroll
      for (int r = 0; r < kTokensPerWarp; ++r) {
        next[r] = load_row(static_cast<long long>(tok0) + kTokensPerWarp + r);
      }
    }
#pragma unroll
    for (int i = 0; i < kTokensPerWarp; ++i) {
      const std::uint32_t tok = tok0 + i;
      float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
      // the reference adds the current token's tap first, then the history taps oldest first
      sum.x = x[i + 3].x * w[0][3];
      sum.y = x[i + 3].y * w[1][3];
      sum.z = x[i + 3].z * w[2][3];
      sum.w = x[i + 3].w * w[3][3];
#pragma unroll
      for (int h = 0; h < kFastWidth - 1; ++h) {
        sum.x += x[i + h].x * w[0][h];
        sum.y += x[i + h].y * w[1][h];
        sum.z += x[i + h].z * w[2][h];
        sum.w += x[i + h].w * w[3][h];
      }
      float4 value = make_float4(silu_fast(sum.x), silu_fast(sum.y), silu_fast(sum.z), silu_fast(sum.w));
      if (is_qk) {
        float squares = (value.x * value.x + value.y * value.y) + (value.z * value.z + value.w * value.w);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
          squares += __shfl_xor_sync(0xFFFFFFFFU, squares, offset);
        }
        const float scale = rsqrtf(squares + kQkEpsilon) * q_scale;
        value.x *= scale;
        value.y *= scale;
        value.z *= scale;
        value.w *= scale;
      }
      if (tok < p.tokens) {
        *reinterpret_cast<float4 *>(p.convolved + static_cast<std::size_t>(tok) * p.conv_dim + channel) = value;
      }
    }
    if (step + 1 < kStepsPerWarp) {
#pragma unroll
      for (int h = 0; h < kFastWidth - 1; ++h) {
        x[h] = x[kTokensPerWarp + h];
      }
#pragma unroll
      for (int r = 0; r < kTokensPerWarp; ++r) {
        x[kFastWidth - 1 + r] = next[r];
      }
    }
  }
}

// grid (ceil(tokens * value_heads / 8)), 256 threads: a warp per (token, value head), four channels per lane
template <int Dtype> __global__ void __launch_bounds__(256) gdn_epilogue_warp_kernel(const LayerParams p) {
  grid_dependency_wait(); // launched with programmatic serialisation behind the recurrence, whose output it reads
  const int lane = threadIdx.x & 31;
  const std::size_t item = static_cast<std::size_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= static_cast<std::size_t>(p.tokens) * p.value_heads) {
    return;
  }
  const std::size_t tok = item / p.value_heads;
  const std::uint32_t head = static_cast<std::uint32_t>(item % p.value_heads);
  const std::size_t index = item * kDim + 4 * lane; // [token][head][128]
  const float4 value = *reinterpret_cast<const float4 *>(p.raw + index);
  const float4 z = Io<Dtype>::load4(p.input, tok * p.token_stride + p.conv_dim + 2 * p.value_heads + head * kDim +
                                                 4 * lane);
  float squares = (value.x * value.x + value.y * value.y) + (value.z * value.z + value.w * value.w);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    squares += __shfl_xor_sync(0xFFFFFFFFU, squares, offset);
  }
  const float scale = rsqrtf(squares / static_cast<float>(kDim) + p.epsilon);
  float4 out;
  out.x = value.x * scale * load_any(p.output_norm_weight, 4 * lane, p.weight_dtype) * silu_fast(z.x);
  out.y = value.y * scale * load_any(p.output_norm_weight, 4 * lane + 1, p.weight_dtype) * silu_fast(z.y);
  out.z = value.z * scale * load_any(p.output_norm_weight, 4 * lane + 2, p.weight_dtype) * silu_fast(z.z);
  out.w = value.w * scale * load_any(p.output_norm_weight, 4 * lane + 3, p.weight_dtype) * silu_fast(z.w);
  Io<Dtype>::store4(p.output, index, out);
}

// Whether the vector forms apply: every row segment a lane touches must start on the boundary of its access.
bool vector_forms_apply(const LayerParams &p) {
  const std::size_t element = p.dtype == RIB200_DTYPE_F32 ? 4 : 2;
  const std::size_t access = 4 * element;
  if (p.weight_dtype == RIB200_DTYPE_F32 && reinterpret_cast<std::uintptr_t>(p.conv_weight) % 16 != 0) {
    return false; // the four taps of a channel are fetched as one 16-byte word
  }
  return reinterpret_cast<std::uintptr_t>(p.input) % access == 0 &&
         reinterpret_cast<std::uintptr_t>(p.output) % access == 0 && (p.token_stride * element) % access == 0 &&
         ((p.conv_dim + 2 * p.value_heads) * element) % access == 0;
}

// one thread per channel: new history[h] = element tokens + h of [old history | token stream]
__global__ void gdn_conv_state_kernel(const LayerParams p) {
  grid_dependents_may_launch();
  const std::uint32_t channel = blockIdx.x * blockDim.x + threadIdx.x;
  const std::uint32_t history = p.conv_width - 1;
  if (channel >= p.conv_dim || history == 0) {
    return;
  }
  float next[8];
  for (std::uint32_t h = 0; h < history; ++h) {
    const std::size_t source = static_cast<std::size_t>(p.tokens) + h;
    next[h] = source < history
                  ? p.convolution_state[static_cast<std::size_t>(channel) * history + source]
                  : load_any(p.input, (source - history) * p.token_stride + channel, p.dtype);
  }
  // launched with programmatic serialisation behind the prologue, which reads the old history: write after it ended
  grid_dependency_wait();
  for (std::uint32_t h = 0; h < history; ++h) {
    p.convolution_state[static_cast<std::size_t>(channel) * history + h] = next[h];
  }
}

// grid (value_heads, tokens), 128 threads
__global__ void __launch_bounds__(kDim) gdn_epilogue_kernel(const LayerParams p) {
  grid_dependency_wait();
  __shared__ float scratch[4];
  const std::uint32_t head = blockIdx.x;
  const std::uint32_t tok = blockIdx.y;
  const std::size_t hidden = static_cast<std::size_t>(p.value_heads) * kDim;
  const std::size_t index = static_cast<std::size_t>(tok) * hidden + head * kDim + threadIdx.x;
  const float value = p.raw[index];
  const float squares = block_sum_128(value * value, scratch);
  const float scale = rsqrtf(squares / static_cast<float>(kDim) + p.epsilon);
  const float z = load_any(p.input,
                           static_cast<std::size_t>(tok) * p.token_stride + p.conv_dim + 2 * p.value_heads +
                               head * kDim + threadIdx.x,
                           p.dtype);
  const float normalised = value * scale * load_any(p.output_norm_weight, threadIdx.x, p.weight_dtype);
  store_any(p.output, index, p.dtype, normalised * silu(z));
}

LayerParams make_params(const GdnLayerArgs &a) {
  LayerParams p{};
  p.input = a.input;
  p.conv_weight = a.conv_weight;
  p.recurrent_a = a.recurrent_a;
  p.dt_bias = a.dt_bias;
  p.output_norm_weight = a.output_norm_weight;
  p.output = a.output;
  p.convolution_state = a.convolution_state;
  p.convolved = a.convolved;
  p.beta = a.beta;
  p.log_decay = a.log_decay;
  p.raw = a.raw;
  p.tokens = a.tokens;
  p.key_heads = a.key_heads;
  p.value_heads = a.value_heads;
  p.conv_width = a.conv_width;
  p.conv_dim = (2 * a.key_heads + a.value_heads) * kDim;
  p.token_stride = p.conv_dim + 2 * a.value_heads + a.value_heads * kDim;
  p.epsilon = a.epsilon;
  p.dtype = a.dtype;
  p.weight_dtype = a.weight_dtype;
  return p;
}

} // namespace

void launch_gdn_prologue(const GdnLayerArgs &a, cudaStream_t stream) {
  const LayerParams p = make_params(a);
  // a call of a few tokens is latency, not bandwidth: the one-CTA-per-vector kernel spreads it wider
  if (a.conv_width == kFastWidth && a.tokens >= 2 * kTokensPerWarp && vector_forms_apply(p)) {
    constexpr std::uint32_t kTokensPerCta = kTokensPerWarp * kStepsPerWarp;
    const dim3 grid((a.tokens + kTokensPerCta - 1) / kTokensPerCta, (2 * a.key_heads + a.value_heads + 1 + 7) / 8);
    if (a.dtype == RIB200_DTYPE_F32) {
      gdn_prologue_w4_kernel<RIB200_DTYPE_F32><<<grid, 256, 0, stream>>>(p);
    } else if (a.dtype == RIB200_DTYPE_F16) {
      gdn_prologue_w4_kernel<RIB200_DTYPE_F16><<<grid, 256, 0, stream>>>(p);
    } else {
      gdn_prologue_w4_kernel<RIB200_DTYPE_BF16><<<grid, 256, 0, stream>>>(p);
    }
  } else {
    gdn_prologue_kernel<<<dim3(2 * a.key_heads + a.value_heads, a.tokens), kDim, 0, stream>>>(p);
  }
  cuda_ok(cudaGetLastError(), "gated-delta prologue launch");
  if (a.conv_width > 1) {
    launch_programmatic(gdn_conv_state_kernel, dim3((p.conv_dim + 255) / 256), dim3(256), 0, stream,
                        "gated-delta convolution-state launch", p);
  }
}

void launch_gdn_epilogue(const GdnLayerArgs &a, cudaStream_t stream) {
  const LayerParams p = make_params(a);
  if (vector_forms_apply(p)) {
    const std::size_t items = static_cast<std::size_t>(a.tokens) * a.value_heads;
    const unsigned int grid = static_cast<unsigned int>((items + 7) / 8);
    const char *what = "gated-delta epilogue launch";
    if (a.dtype == RIB200_DTYPE_F32) {
      launch_programmatic(gdn_epilogue_warp_kernel<RIB200_DTYPE_F32>, dim3(grid), dim3(256), 0, stream, what, p);
    } else if (a.dtype == RIB200_DTYPE_F16) {
      launch_programmatic(gdn_epilogue_warp_kernel<RIB200_DTYPE_F16>, dim3(grid), dim3(256), 0, stream, what, p);
    } else {
      launch_programmatic(gdn_epilogue_warp_kernel<RIB200_DTYPE_BF16>, dim3(grid), dim3(256), 0, stream, what, p);
    }
    return;
  }
  launch_programmatic(gdn_epilogue_kernel, dim3(a.value_heads, a.tokens), dim3(kDim), 0, stream,
                      "gated-delta epilogue launch", p);
}

} // namespace rib200
