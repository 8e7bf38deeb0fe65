// Host side of the gated-delta entry points: validation and dispatch.  Argument meaning and refusal
// behaviour follow cpp/kernels/qwen35_delta.cu:49-131 (shape), :199-226 (policy), :811-868 (pointers,
// dtypes, alignment).  Narrowing: key_dim == value_dim == 128 (other head sizes return UNSUPPORTED).
//
// Workspace.  The reference sizes its scratch as tokens * (conv_dim + hidden) floats
// (cpp/kernels/qwen35_delta.cu:107-114).  This library asks for a little more through the same query:
// the per-token gates (2 * value_heads floats) and, for runs of 64 tokens or more, the scratch of the
// chunked prefill.  Callers size the buffer through the query, as the reference's executor does.

#include "common.hpp"

#include <cmath>
#include <cstring>

namespace rib200 {
namespace {

constexpr std::size_t kDim = 128;
constexpr std::size_t kChunkThreshold = 64;

struct Checked {
  std::size_t key_size, value_size, conv_dim, token_stride, convolution_elements, recurrent_elements;
  std::size_t convolved_floats, gate_floats, raw_floats, chunk_bytes, workspace_bytes;
};

const Rib200GatedDeltaShape &deref(const Rib200GatedDeltaShape *shape) {
  require(shape != nullptr, "gated-delta shape pointer is null");
  return *shape;
}

Checked validate_shape(const Rib200GatedDeltaShape &s) {
  require(s.tokens > 0, "gated-delta tokens must be positive");
  require(s.hidden_size > 0, "gated-delta hidden_size must be positive");
  require(s.key_heads > 0, "gated-delta key_heads must be positive");
  require(s.value_heads > 0, "gated-delta value_heads must be positive");
  require(s.key_dim > 0, "gated-delta key_dim must be positive");
  require(s.value_dim > 0, "gated-delta value_dim must be positive");
  require(s.conv_width > 0, "gated-delta conv_width must be positive");
  require(std::isfinite(s.epsilon) && s.epsilon >= 0.0F, "gated-delta epsilon must be finite and non-negative");
  require(s.value_heads % s.key_heads == 0, "gated-delta value_heads must be a multiple of key_heads");
  Checked c{};
  c.key_size = mul(s.key_heads, s.key_dim, "gated-delta key size overflows");
  c.value_size = mul(s.value_heads, s.value_dim, "gated-delta value size overflows");
  require(c.value_size == s.hidden_size, "gated-delta value_heads * value_dim must equal hidden_size");
  c.conv_dim = add(mul(c.key_size, 2, "gated-delta conv size overflows"), c.value_size,
                   "gated-delta conv size overflows");
  c.token_stride = add(add(c.conv_dim, mul(s.value_heads, 2, "gated-delta input size overflows"),
                           "gated-delta input size overflows"),
                       s.hidden_size, "gated-delta input size overflows");
  (void)mul(s.tokens, c.token_stride, "gated-delta input size overflows");
  (void)mul(c.conv_dim, s.conv_width, "gated-delta convolution weight size overflows");
  c.convolution_elements = mul(c.conv_dim, s.conv_width - 1, "gated-delta convolution state size overflows");
  c.recurrent_elements = mul(c.value_size, s.key_dim, "gated-delta recurrent state size overflows");
  c.convolved_floats = mul(s.tokens, c.conv_dim, "gated-delta workspace size overflows");
  c.raw_floats = mul(s.tokens, s.hidden_size, "gated-delta workspace size overflows");
  c.gate_floats = mul(s.tokens, mul(s.value_heads, 2, "gated-delta workspace size overflows"),
                      "gated-delta workspace size overflows");
  c.chunk_bytes = s.tokens >= kChunkThreshold && s.key_dim == kDim && s.value_dim == kDim
                      ? gdn_chunk_workspace_bytes(s.tokens, s.key_heads, s.value_heads)
                      : 0;
  c.workspace_bytes =
      add(mul(add(add(c.convolved_floats, c.raw_floats, "gated-delta workspace size overflows"), c.gate_floats,
                  "gated-delta workspace size overflows"),
              sizeof(float), "gated-delta workspace size overflows"),
          c.chunk_bytes, "gated-delta workspace size overflows");
  require(s.tokens <= 0x7FFFFFFFU && c.conv_dim <= 0x7FFFFFFFU, "gated-delta shape exceeds the launch limits");
  return c;
}

// cpp/kernels/qwen35_delta.cu:199-226
void validate_policy(Rib200GatedDeltaLaunchPolicy policy, const Rib200GatedDeltaShape &s) {
  require(policy.warps_per_block == 4, "gated-delta schedule needs four warps per block");
  require(policy.transposed_boundary_state == 0, "gated-delta transposed boundary state is not initialised");
  switch (policy.schedule) {
  case RIB200_DELTA_SCHEDULE_CURRENT:
    break;
  case RIB200_DELTA_SCHEDULE_PREFILL_SM120:
  case RIB200_DELTA_SCHEDULE_DECODE_SM120:
    require(s.key_dim == 64 || s.key_dim == 128, "gated-delta candidate schedule needs key_dim 64 or 128");
    require(s.value_dim == s.key_dim, "gated-delta candidate schedule needs value_dim == key_dim");
    if (policy.schedule == RIB200_DELTA_SCHEDULE_DECODE_SM120) {
      require(s.tokens == 1, "gated-delta decode schedule takes exactly one token");
    }
    break;
  default:
    require(false, "unknown gated-delta schedule");
  }
}

std::size_t dtype_alignment(int32_t dtype) { return dtype == RIB200_DTYPE_F32 ? 4 : 2; }

void require_aligned(const void *ptr, std::size_t alignment, const char *message) {
  require(reinterpret_cast<std::uintptr_t>(ptr) % alignment == 0, message);
}

void run_core(const GdnCoreArgs &core, void *chunk_scratch, cudaStream_t stream) {
  if (core.tokens >= kChunkThreshold && core.sequences == 1) {
    launch_gdn_chunked(core, chunk_scratch, stream);
  } else {
    launch_gdn_recurrent(core, stream);
  }
}

} // namespace
} // namespace rib200

using namespace rib200;

extern "C" {

Rib200Status rib200_gated_delta_workspace_bytes(const Rib200GatedDeltaShape *shape, size_t *bytes) {
  return guarded([&] {
    require(bytes != nullptr, "output pointer is null");
    *bytes = validate_shape(deref(shape)).workspace_bytes;
  });
}

// The reference keeps its "current" schedule until a tuner promotes a candidate
// (cpp/kernels/qwen35_delta.cu:759-769); the schedules name sm_120 register layouts that do not exist
// here, so the policy is carried for interface compatibility and every accepted policy runs the same
// sm_100a kernels.
Rib200Status rib200_gated_delta_select_policy(const Rib200GatedDeltaShape *shape, size_t bucket_tokens,
                                              Rib200GatedDeltaLaunchPolicy *policy) {
  return guarded([&] {
    (void)shape;
    (void)bucket_tokens;
    require(policy != nullptr, "output pointer is null");
    policy->schedule = RIB200_DELTA_SCHEDULE_CURRENT;
    policy->warps_per_block = 4;
    policy->transposed_boundary_state = 0;
  });
}

Rib200Status rib200_gated_delta_schedule_diagnostic(const Rib200GatedDeltaShape *shape, size_t bucket_tokens,
                                                    Rib200GatedDeltaScheduleDiagnostic *diagnostic) {
  return guarded([&] {
    require(diagnostic != nullptr, "output pointer is null");
    const Rib200GatedDeltaShape &s = deref(shape);
    std::memset(diagnostic, 0, sizeof(*diagnostic));
    diagnostic->bucket_tokens = bucket_tokens;
    diagnostic->key_dim = s.key_dim;
    diagnostic->value_dim = s.value_dim;
    diagnostic->candidate_schedule =
        bucket_tokens == 1 ? RIB200_DELTA_SCHEDULE_DECODE_SM120 : RIB200_DELTA_SCHEDULE_PREFILL_SM120;
    diagnostic->schedule = RIB200_DELTA_SCHEDULE_CURRENT;
    diagnostic->warps_per_block = 4;
    std::strncpy(diagnostic->rejection_reason, "not_tuned", sizeof(diagnostic->rejection_reason) - 1);
  });
}

Rib200Status rib200_gated_delta(const void *input, const void *conv_weight, const void *recurrent_a,
                                const void *dt_bias, const void *output_norm_weight, void *output,
                                float *convolution_state, float *recurrent_state, void *workspace,
                                size_t workspace_bytes, const Rib200GatedDeltaShape *shape,
                                Rib200GatedDeltaLaunchPolicy policy, int32_t dtype, int32_t weight_dtype,
                                void *stream) {
  return guarded([&] {
    const Rib200GatedDeltaShape &s = deref(shape);
    const Checked c = validate_shape(s);
    validate_policy(policy, s);
    require(dtype == RIB200_DTYPE_F32 || dtype == RIB200_DTYPE_F16 || dtype == RIB200_DTYPE_BF16,
            "gated-delta: unknown activation dtype");
    require(weight_dtype == RIB200_DTYPE_F32 || weight_dtype == dtype ||
                (dtype == RIB200_DTYPE_F32 &&
                 (weight_dtype == RIB200_DTYPE_F16 || weight_dtype == RIB200_DTYPE_BF16)),
            "gated-delta: weight dtype does not go with the activation dtype");
    require(input != nullptr, "gated-delta: input pointer is null");
    require(conv_weight != nullptr, "gated-delta: convolution weight pointer is null");
    require(recurrent_a != nullptr, "gated-delta: recurrent coefficient pointer is null");
    require(dt_bias != nullptr, "gated-delta: dt-bias pointer is null");
    require(output_norm_weight != nullptr, "gated-delta: output norm weight pointer is null");
    require(output != nullptr, "gated-delta: output pointer is null");
    require(c.convolution_elements == 0 || convolution_state != nullptr,
            "gated-delta: convolution state pointer is null");
    require(c.recurrent_elements == 0 || recurrent_state != nullptr, "gated-delta: recurrent state pointer is null");
    require(workspace != nullptr, "gated-delta: workspace pointer is null");
    require(workspace_bytes >= c.workspace_bytes, "gated-delta: workspace is too small");
    require_aligned(input, dtype_alignment(dtype), "gated-delta: input is not dtype-aligned");
    require_aligned(conv_weight, dtype_alignment(weight_dtype), "gated-delta: convolution weight is not dtype-aligned");
    require_aligned(recurrent_a, dtype_alignment(weight_dtype),
                    "gated-delta: recurrent coefficient is not dtype-aligned");
    require_aligned(dt_bias, dtype_alignment(weight_dtype), "gated-delta: dt-bias is not dtype-aligned");
    require_aligned(output_norm_weight, dtype_alignment(weight_dtype),
                    "gated-delta: output norm weight is not dtype-aligned");
    require_aligned(output, dtype_alignment(dtype), "gated-delta: output is not dtype-aligned");
    require_aligned(workspace, 4, "gated-delta: workspace is not float-aligned");
    require_aligned(recurrent_state, 4, "gated-delta: recurrent state is not float-aligned");
    if (c.convolution_elements != 0) {
      require_aligned(convolution_state, 4, "gated-delta: convolution state is not float-aligned");
    }
    require(stream != nullptr, "gated-delta: CUDA stream is null");
    unsupported(s.key_dim == kDim && s.value_dim == kDim, "gated-delta: built for key_dim == value_dim == 128");
    unsupported(s.conv_width <= 9, "gated-delta: conv_width above 9 is not built");
    unsupported(s.tokens <= 65535, "gated-delta: at most 65535 tokens per call");
    require_aligned(workspace, 16, "gated-delta: workspace is not 16-byte aligned");
    require_aligned(recurrent_state, 16, "gated-delta: recurrent state is not 16-byte aligned");

    auto *cuda_stream = static_cast<cudaStream_t>(stream);
    auto *floats = static_cast<float *>(workspace);
    GdnLayerArgs layer{};
    layer.input = input;
    layer.conv_weight = conv_weight;
    layer.recurrent_a = recurrent_a;
    layer.dt_bias = dt_bias;
    layer.output_norm_weight = output_norm_weight;
    layer.output = output;
    layer.convolution_state = convolution_state;
    layer.convolved = floats;
    float *raw = floats + c.convolved_floats;
    layer.raw = raw;
    layer.beta = raw + c.raw_floats;
    layer.log_decay = layer.beta + c.gate_floats / 2;
    layer.tokens = static_cast<std::uint32_t>(s.tokens);
    layer.key_heads = static_cast<std::uint32_t>(s.key_heads);
    layer.value_heads = static_cast<std::uint32_t>(s.value_heads);
    layer.conv_width = static_cast<std::uint32_t>(s.conv_width);
    layer.epsilon = s.epsilon;
    layer.dtype = dtype;
    layer.weight_dtype = weight_dtype;
    launch_gdn_prologue(layer, cuda_stream);

    GdnCoreArgs core{};
    core.q = floats;
    core.k = floats + c.key_size;
    core.v = floats + 2 * c.key_size;
    core.q_stride = core.k_stride = core.v_stride = c.conv_dim;
    core.qkv_f32 = true;
    core.beta = layer.beta;
    core.log_decay = layer.log_decay;
    core.state = recurrent_state;
    core.out = raw;
    core.tokens = layer.tokens;
    core.sequences = 1;
    core.key_heads = layer.key_heads;
    core.value_heads = layer.value_heads;
    void *chunk_scratch = layer.log_decay + c.gate_floats / 2;
    run_core(core, chunk_scratch, cuda_stream);
    launch_gdn_epilogue(layer, cuda_stream);
  });
}

Rib200Status rib200_gdn_core_workspace_bytes(size_t tokens, size_t key_heads, size_t value_heads, size_t key_dim,
                                             size_t value_dim, size_t *bytes) {
  return guarded([&] {
    require(bytes != nullptr, "output pointer is null");
    require(tokens > 0 && key_heads > 0 && value_heads > 0, "gdn core: sizes must be positive");
    unsupported(key_dim == kDim && value_dim == kDim, "gdn core: built for key_dim == value_dim == 128");
    *bytes = tokens >= kChunkThreshold ? gdn_chunk_workspace_bytes(tokens, key_heads, value_heads) : 0;
  });
}

Rib200Status rib200_gdn_core(const void *q, const void *k, const void *v, const float *beta,
                             const float *log_decay, float *state, float *out, void *workspace,
                             size_t workspace_bytes, size_t tokens, size_t key_heads, size_t value_heads,
                             size_t key_dim, size_t value_dim, int32_t qkv_dtype, void *stream) {
  return guarded([&] {
    require(q != nullptr && k != nullptr && v != nullptr, "gdn core: an operand pointer is null");
    require(beta != nullptr && log_decay != nullptr, "gdn core: a gate pointer is null");
    require(state != nullptr && out != nullptr, "gdn core: state or output pointer is null");
    require(stream != nullptr, "gdn core: CUDA stream is null");
    require(tokens > 0 && tokens <= 0x7FFFFFFFU, "gdn core: tokens out of range");
    require(key_heads > 0 && value_heads > 0 && value_heads % key_heads == 0 && value_heads <= 65535,
            "gdn core: value_heads must be a positive multiple of key_heads");
    unsupported(key_dim == kDim && value_dim == kDim, "gdn core: built for key_dim == value_dim == 128");
    require(qkv_dtype == RIB200_DTYPE_F32 || qkv_dtype == RIB200_DTYPE_BF16, "gdn core: q/k/v must be F32 or BF16");
    const std::size_t need = tokens >= kChunkThreshold ? gdn_chunk_workspace_bytes(tokens, key_heads, value_heads) : 0;
    require(need == 0 || workspace != nullptr, "gdn core: workspace is null");
    require(workspace_bytes >= need, "gdn core: workspace is too small");
    for (const void *ptr : {q, k, v, static_cast<const void *>(state), static_cast<const void *>(out),
                            static_cast<const void *>(workspace)}) {
      require_aligned(ptr, 16, "gdn core: pointers must be 16-byte aligned");
    }
    GdnCoreArgs core{};
    core.q = q;
    core.k = k;
    core.v = v;
    core.q_stride = core.k_stride = key_heads * kDim;
    core.v_stride = value_heads * kDim;
    core.qkv_f32 = qkv_dtype == RIB200_DTYPE_F32;
    core.beta = beta;
    core.log_decay = log_decay;
    core.state = state;
    core.out = out;
    core.tokens = static_cast<std::uint32_t>(tokens);
    core.sequences = 1;
    core.key_heads = static_cast<std::uint32_t>(key_heads);
    core.value_heads = static_cast<std::uint32_t>(value_heads);
    run_core(core, workspace, static_cast<cudaStream_t>(stream));
  });
}

Rib200Status rib200_batched_gdn_decode(const void *q, const void *k, const void *v, const float *beta,
                                       const float *log_decay, float *const *states, float *out, size_t batch,
                                       size_t key_heads, size_t value_heads, void *stream) {
  return guarded([&] {
    require(q != nullptr && k != nullptr && v != nullptr, "batched gdn decode: an operand pointer is null");
    require(beta != nullptr && log_decay != nullptr, "batched gdn decode: a gate pointer is null");
    require(states != nullptr && out != nullptr, "batched gdn decode: states or output pointer is null");
    require(stream != nullptr, "batched gdn decode: CUDA stream is null");
    require(batch > 0 && batch <= 65535, "batched gdn decode: batch must be in 1..65535");
    require(key_heads > 0 && value_heads > 0 && value_heads % key_heads == 0 && value_heads <= 65535,
            "batched gdn decode: value_heads must be a positive multiple of key_heads");
    for (const void *ptr : {q, k, v, static_cast<const void *>(out)}) {
      require_aligned(ptr, 16, "batched gdn decode: pointers must be 16-byte aligned");
    }
    GdnCoreArgs core{};
    core.q = q;
    core.k = k;
    core.v = v;
    core.q_stride = core.k_stride = key_heads * kDim;
    core.v_stride = value_heads * kDim;
    core.qkv_f32 = false;
    core.beta = beta;
    core.log_decay = log_decay;
    core.states = states;
    core.out = out;
    core.tokens = 1;
    core.sequences = static_cast<std::uint32_t>(batch);
    core.key_heads = static_cast<std::uint32_t>(key_heads);
    core.value_heads = static_cast<std::uint32_t>(value_heads);
    launch_gdn_recurrent(core, static_cast<cudaStream_t>(stream));
  });
}

} // extern "C"
