// The steps of qwen35_gated_delta on either side of the recurrence, for key_dim = value_dim = 128:
//   prologue  depthwise causal convolution + SiLU over the q|k|v channels, L2 normalisation of every q
//             and k head (q also scaled by 1/sqrt(128)), beta = sigmoid(b), log decay = A * softplus(a + dt)
//             (cpp/kernels/qwen35_delta.cu:236-276,375-411,522-529; CPU cpp/reference/qwen35.cpp:417-469);
//   state     shift of the convolution history [channel][W-1] (cpp/kernels/qwen35_delta.cu:267-275);
//   epilogue  per-head RMSNorm(128) * weight * SiLU(z) (cpp/kernels/qwen35_delta.cu:579-621).
// Unlike the reference's convolution kernel, which walks the tokens serially per channel, every
// (token, head vector) pair is its own CTA: a tap is read from the token stream or, for the first W-1
// tokens, from the carried history.

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

// one thread per channel: new history[h] = element tokens + h of [old history | token stream]
__global__ void gdn_conv_state_kernel(const LayerParams p) {
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
  for (std::uint32_t h = 0; h < history; ++h) {
    p.convolution_state[static_cast<std::size_t>(channel) * history + h] = next[h];
  }
}

// grid (value_heads, tokens), 128 threads
__global__ void __launch_bounds__(kDim) gdn_epilogue_kernel(const LayerParams p) {
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
  gdn_prologue_kernel<<<dim3(2 * a.key_heads + a.value_heads, a.tokens), kDim, 0, stream>>>(p);
  cuda_ok(cudaGetLastError(), "gated-delta prologue launch");
  if (a.conv_width > 1) {
    gdn_conv_state_kernel<<<(p.conv_dim + 255) / 256, 256, 0, stream>>>(p);
    cuda_ok(cudaGetLastError(), "gated-delta convolution-state launch");
  }
}

void launch_gdn_epilogue(const GdnLayerArgs &a, cudaStream_t stream) {
  const LayerParams p = make_params(a);
  gdn_epilogue_kernel<<<dim3(a.value_heads, a.tokens), kDim, 0, stream>>>(p);
  cuda_ok(cudaGetLastError(), "gated-delta epilogue launch");
}

} // namespace rib200
