// Drop-in C++ face of librib200 for RAFTInfer's executor: the types and free functions of
// cpp/kernels/qwen35_attention.cuh, cpp/kernels/qwen35_online_attention.cuh and cpp/kernels/qwen35_delta.cuh,
// with the same names, argument order and exception types, implemented as inline wrappers over the C ABI in
// rib200.h.  A non-OK status becomes the exception the reference would have thrown, carrying the status message.
//
// The enums below repeat cpp/include/raftinfer/tensor.h:10-15 and cpp/execution/qwen35_execution_policy.hpp:7-27;
// define RIB200_USE_RAFTINFER_TYPES before including this header inside the RAFTInfer tree to take them from
// <raftinfer/tensor.h> and "execution/qwen35_execution_policy.hpp" instead.
#pragma once

#include "../rib200.h"

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#ifdef RIB200_USE_RAFTINFER_TYPES
#include "execution/qwen35_execution_policy.hpp"
#include <raftinfer/tensor.h>
#else
extern "C" {
typedef enum RaftInferDataType {
  RAFTINFER_DTYPE_F32 = 1,
  RAFTINFER_DTYPE_F16 = 2,
  RAFTINFER_DTYPE_BF16 = 3,
  RAFTINFER_DTYPE_Q4_K = 100
} RaftInferDataType;
}
namespace raftinfer {
enum class Qwen35AttentionImplementation : std::uint8_t { materialized_reference, online_tiled };
enum class Qwen35DecodeAttentionMode : std::uint8_t { auto_select, single_block, split_k_256, split_k_512 };
enum class Qwen35KvCacheDType : std::uint8_t { f32, bf16 };
enum class Qwen35KvCacheLayout : std::uint8_t { token_major, head_major };
} // namespace raftinfer
#endif

namespace raftinfer::kernels {

// cpp/kernels/qwen35_primitives.cuh:15-19
class Qwen35PrimitiveError : public std::runtime_error {
public:
  explicit Qwen35PrimitiveError(const std::string &message) : std::runtime_error(message) {}
};

// cpp/kernels/qwen35_delta.cuh:14-18
class Qwen35DeltaError : public std::runtime_error {
public:
  explicit Qwen35DeltaError(const std::string &message) : std::runtime_error(message) {}
};

struct Qwen35AttentionShape {
  std::size_t tokens;
  std::size_t query_heads;
  std::size_t kv_heads;
  std::size_t head_dim;
  std::size_t max_context_tokens;
  std::size_t past_tokens;
};

struct Qwen35AttentionLaunchPolicy {
  raftinfer::Qwen35AttentionImplementation implementation;
  raftinfer::Qwen35KvCacheDType kv_cache_dtype;
  raftinfer::Qwen35KvCacheLayout kv_cache_layout;
};

struct Qwen35OnlineDecodePlan {
  Qwen35DecodeAttentionMode resolved_mode{Qwen35DecodeAttentionMode::single_block};
  std::size_t partition_tokens{};
  std::size_t split_k_threshold_tokens{};
  std::size_t context_bucket_tokens{};
  std::size_t active_partition_capacity{1};
  bool operator==(const Qwen35OnlineDecodePlan &o) const {
    return resolved_mode == o.resolved_mode && partition_tokens == o.partition_tokens &&
           split_k_threshold_tokens == o.split_k_threshold_tokens &&
           context_bucket_tokens == o.context_bucket_tokens &&
           active_partition_capacity == o.active_partition_capacity;
  }
};

struct Qwen35OnlineDecodeWorkspaceLayout {
  std::size_t partial_count{};
  std::size_t max_offset_bytes{};
  std::size_t sum_offset_bytes{};
  std::size_t value_offset_bytes{};
  std::size_t bytes{};
  bool operator==(const Qwen35OnlineDecodeWorkspaceLayout &o) const {
    return partial_count == o.partial_count && max_offset_bytes == o.max_offset_bytes &&
           sum_offset_bytes == o.sum_offset_bytes && value_offset_bytes == o.value_offset_bytes && bytes == o.bytes;
  }
};

struct GatedDeltaShape {
  std::size_t tokens;
  std::size_t hidden_size;
  std::size_t key_heads;
  std::size_t value_heads;
  std::size_t key_dim;
  std::size_t value_dim;
  std::size_t conv_width;
  float epsilon;
};

enum class GatedDeltaSchedule : std::uint8_t {
  register_resident_current,
  register_resident_prefill_sm120,
  register_resident_decode_sm120,
};

struct GatedDeltaLaunchPolicy {
  GatedDeltaSchedule schedule{GatedDeltaSchedule::register_resident_current};
  std::uint32_t warps_per_block{4};
  bool transposed_boundary_state{false};
};

struct GatedDeltaScheduleDiagnostic {
  std::size_t bucket_tokens{};
  std::size_t key_dim{};
  std::size_t value_dim{};
  GatedDeltaSchedule candidate_schedule{GatedDeltaSchedule::register_resident_current};
  GatedDeltaSchedule schedule{GatedDeltaSchedule::register_resident_current};
  std::uint32_t warps_per_block{};
  bool transposed_boundary_state{};
  bool candidate_accepted{};
  bool correctness_passed{};
  float current_median_ms{};
  float candidate_median_ms{};
  std::string rejection_reason;
};

namespace detail {

inline void check(Rib200Status status) {
  if (status.code != RIB200_STATUS_OK) {
    throw Qwen35PrimitiveError(status.message != nullptr ? status.message : "rib200 failure");
  }
}

inline void check_delta(Rib200Status status) {
  if (status.code != RIB200_STATUS_OK) {
    throw Qwen35DeltaError(status.message != nullptr ? status.message : "rib200 failure");
  }
}

inline Rib200AttentionShape to_c(const Qwen35AttentionShape &s) {
  return Rib200AttentionShape{s.tokens, s.query_heads, s.kv_heads, s.head_dim, s.max_context_tokens, s.past_tokens};
}

inline Rib200AttentionLaunchPolicy to_c(const Qwen35AttentionLaunchPolicy &p) {
  return Rib200AttentionLaunchPolicy{static_cast<std::uint8_t>(p.implementation),
                                     static_cast<std::uint8_t>(p.kv_cache_dtype),
                                     static_cast<std::uint8_t>(p.kv_cache_layout)};
}

inline Rib200OnlineDecodePlan to_c(const Qwen35OnlineDecodePlan &p) {
  return Rib200OnlineDecodePlan{static_cast<std::uint8_t>(p.resolved_mode), p.partition_tokens,
                                p.split_k_threshold_tokens, p.context_bucket_tokens, p.active_partition_capacity};
}

inline Rib200GatedDeltaShape to_c(const GatedDeltaShape &s) {
  return Rib200GatedDeltaShape{s.tokens,  s.hidden_size, s.key_heads,  s.value_heads,
                               s.key_dim, s.value_dim,   s.conv_width, s.epsilon};
}

inline Rib200GatedDeltaLaunchPolicy to_c(const GatedDeltaLaunchPolicy &p) {
  return Rib200GatedDeltaLaunchPolicy{static_cast<std::uint8_t>(p.schedule), p.warps_per_block,
                                      static_cast<std::uint8_t>(p.transposed_boundary_state ? 1 : 0)};
}

} // namespace detail

inline std::size_t qwen35_attention_workspace_floats(Qwen35AttentionShape shape) {
  const Rib200AttentionShape s = detail::to_c(shape);
  std::size_t out = 0;
  detail::check(rib200_attention_workspace_floats(&s, &out));
  return out;
}

inline std::size_t qwen35_attention_workspace_bytes(Qwen35AttentionShape shape) {
  return qwen35_attention_workspace_floats(shape) * sizeof(float);
}

inline std::size_t qwen35_attention_cache_bytes(Qwen35AttentionShape shape, Qwen35AttentionLaunchPolicy policy) {
  const Rib200AttentionShape s = detail::to_c(shape);
  std::size_t out = 0;
  detail::check(rib200_attention_cache_bytes(&s, detail::to_c(policy), &out));
  return out;
}

inline std::size_t qwen35_attention_workspace_bytes(Qwen35AttentionShape shape, Qwen35AttentionLaunchPolicy policy) {
  const Rib200AttentionShape s = detail::to_c(shape);
  std::size_t out = 0;
  detail::check(rib200_attention_workspace_bytes(&s, detail::to_c(policy), &out));
  return out;
}

inline void qwen35_causal_attention(const void *query, const void *key, const void *value, const void *gate,
                                    void *output, void *kv_cache, std::size_t kv_cache_bytes, void *workspace,
                                    std::size_t workspace_bytes, Qwen35AttentionShape shape,
                                    RaftInferDataType activation_dtype, Qwen35AttentionLaunchPolicy policy,
                                    cudaStream_t stream) {
  const Rib200AttentionShape s = detail::to_c(shape);
  detail::check(rib200_causal_attention(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace,
                                        workspace_bytes, &s, static_cast<int32_t>(activation_dtype),
                                        detail::to_c(policy), stream));
}

// The reference's second overload drives its materialized logits path over an FP32 token-major cache
// (cpp/kernels/qwen35_attention.cuh:46-51).  That path is the reference's GPU-side test oracle and is not built;
// the call reports it.
inline void qwen35_causal_attention(const void *query, const void *key, const void *value, const void *gate,
                                    void *output, float *kv_cache, float *logits_workspace,
                                    std::size_t logits_workspace_floats, Qwen35AttentionShape shape,
                                    RaftInferDataType dtype, cudaStream_t stream) {
  const Qwen35AttentionLaunchPolicy policy{raftinfer::Qwen35AttentionImplementation::materialized_reference,
                                           raftinfer::Qwen35KvCacheDType::f32,
                                           raftinfer::Qwen35KvCacheLayout::token_major};
  qwen35_causal_attention(query, key, value, gate, output, kv_cache, qwen35_attention_cache_bytes(shape, policy),
                          logits_workspace, logits_workspace_floats * sizeof(float), shape, dtype, policy, stream);
}

inline Qwen35OnlineDecodePlan qwen35_online_decode_plan(Qwen35AttentionShape shape,
                                                        Qwen35DecodeAttentionMode requested,
                                                        std::size_t context_tokens) {
  const Rib200AttentionShape s = detail::to_c(shape);
  Rib200OnlineDecodePlan p{};
  detail::check(rib200_online_decode_plan(&s, static_cast<std::uint8_t>(requested), context_tokens, &p));
  Qwen35OnlineDecodePlan plan;
  plan.resolved_mode = static_cast<Qwen35DecodeAttentionMode>(p.resolved_mode);
  plan.partition_tokens = p.partition_tokens;
  plan.split_k_threshold_tokens = p.split_k_threshold_tokens;
  plan.context_bucket_tokens = p.context_bucket_tokens;
  plan.active_partition_capacity = p.active_partition_capacity;
  return plan;
}

inline Qwen35OnlineDecodeWorkspaceLayout
qwen35_online_decode_workspace_layout(Qwen35AttentionShape shape, Qwen35DecodeAttentionMode resolved_mode) {
  const Rib200AttentionShape s = detail::to_c(shape);
  Rib200OnlineDecodeWorkspaceLayout l{};
  detail::check(rib200_online_decode_workspace_layout(&s, static_cast<std::uint8_t>(resolved_mode), &l));
  return Qwen35OnlineDecodeWorkspaceLayout{l.partial_count, l.max_offset_bytes, l.sum_offset_bytes,
                                           l.value_offset_bytes, l.bytes};
}

inline bool qwen35_online_attention_prefill_supported(Qwen35AttentionShape shape, RaftInferDataType activation_dtype,
                                                      Qwen35AttentionLaunchPolicy policy) noexcept {
  const Rib200AttentionShape s = detail::to_c(shape);
  int32_t supported = 0;
  const Rib200Status status = rib200_online_attention_prefill_supported(
      &s, static_cast<int32_t>(activation_dtype), detail::to_c(policy), &supported);
  return status.code == RIB200_STATUS_OK && supported != 0;
}

inline std::size_t qwen35_online_attention_workspace_bytes(Qwen35AttentionShape shape) noexcept {
  (void)shape;
  return 0;
}

inline void qwen35_online_attention_prefill(const void *query, const void *key, const void *value, const void *gate,
                                            void *output, void *kv_cache, std::size_t kv_cache_bytes,
                                            Qwen35AttentionShape shape, RaftInferDataType activation_dtype,
                                            Qwen35KvCacheDType cache_dtype, Qwen35KvCacheLayout cache_layout,
                                            cudaStream_t stream) {
  const Rib200AttentionShape s = detail::to_c(shape);
  detail::check(rib200_online_attention_prefill(query, key, value, gate, output, kv_cache, kv_cache_bytes, &s,
                                                static_cast<int32_t>(activation_dtype),
                                                static_cast<std::uint8_t>(cache_dtype),
                                                static_cast<std::uint8_t>(cache_layout), stream));
}

inline void qwen35_online_attention_decode(const void *query, const void *key, const void *value, const void *gate,
                                           void *output, void *kv_cache, std::size_t kv_cache_bytes, void *workspace,
                                           std::size_t workspace_bytes, Qwen35AttentionShape shape,
                                           RaftInferDataType activation_dtype, Qwen35KvCacheDType cache_dtype,
                                           Qwen35KvCacheLayout cache_layout, Qwen35OnlineDecodePlan plan,
                                           const std::uint32_t *device_position, cudaStream_t stream) {
  const Rib200AttentionShape s = detail::to_c(shape);
  const Rib200OnlineDecodePlan p = detail::to_c(plan);
  detail::check(rib200_online_attention_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace,
                                               workspace_bytes, &s, static_cast<int32_t>(activation_dtype),
                                               static_cast<std::uint8_t>(cache_dtype),
                                               static_cast<std::uint8_t>(cache_layout), &p, device_position, stream));
}

inline void qwen35_online_attention_decode(const void *query, const void *key, const void *value, const void *gate,
                                           void *output, void *kv_cache, std::size_t kv_cache_bytes,
                                           Qwen35AttentionShape shape, RaftInferDataType activation_dtype,
                                           Qwen35KvCacheDType cache_dtype, Qwen35KvCacheLayout cache_layout,
                                           const std::uint32_t *device_position, cudaStream_t stream) {
  const Qwen35OnlineDecodePlan plan =
      qwen35_online_decode_plan(shape, Qwen35DecodeAttentionMode::single_block, shape.past_tokens + 1);
  qwen35_online_attention_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, nullptr, 0, shape,
                                 activation_dtype, cache_dtype, cache_layout, plan, device_position, stream);
}

inline std::size_t qwen35_gated_delta_workspace_bytes(const GatedDeltaShape &shape) {
  const Rib200GatedDeltaShape s = detail::to_c(shape);
  std::size_t out = 0;
  detail::check_delta(rib200_gated_delta_workspace_bytes(&s, &out));
  return out;
}

inline GatedDeltaLaunchPolicy qwen35_gated_delta_select_policy(const GatedDeltaShape &shape,
                                                               std::size_t bucket_tokens) noexcept {
  (void)shape;
  (void)bucket_tokens;
  return GatedDeltaLaunchPolicy{};
}

inline GatedDeltaScheduleDiagnostic qwen35_gated_delta_schedule_diagnostic(const GatedDeltaShape &shape,
                                                                           std::size_t bucket_tokens) noexcept {
  GatedDeltaScheduleDiagnostic d;
  d.bucket_tokens = bucket_tokens;
  d.key_dim = shape.key_dim;
  d.value_dim = shape.value_dim;
  d.candidate_schedule = bucket_tokens == 1 ? GatedDeltaSchedule::register_resident_decode_sm120
                                            : GatedDeltaSchedule::register_resident_prefill_sm120;
  d.warps_per_block = 4;
  d.rejection_reason = "not_tuned";
  return d;
}

inline void qwen35_gated_delta(const void *input, const void *conv_weight, const void *recurrent_a,
                               const void *dt_bias, const void *output_norm_weight, void *output,
                               float *convolution_state, float *recurrent_state, void *workspace,
                               std::size_t workspace_bytes, GatedDeltaShape shape, GatedDeltaLaunchPolicy policy,
                               RaftInferDataType dtype, RaftInferDataType weight_dtype, cudaStream_t stream) {
  const Rib200GatedDeltaShape s = detail::to_c(shape);
  detail::check_delta(rib200_gated_delta(input, conv_weight, recurrent_a, dt_bias, output_norm_weight, output,
                                         convolution_state, recurrent_state, workspace, workspace_bytes, &s,
                                         detail::to_c(policy), static_cast<int32_t>(dtype),
                                         static_cast<int32_t>(weight_dtype), stream));
}

inline void qwen35_gated_delta(const void *input, const void *conv_weight, const void *recurrent_a,
                               const void *dt_bias, const void *output_norm_weight, void *output,
                               float *convolution_state, float *recurrent_state, void *workspace,
                               std::size_t workspace_bytes, GatedDeltaShape shape, RaftInferDataType dtype,
                               RaftInferDataType weight_dtype, cudaStream_t stream) {
  qwen35_gated_delta(input, conv_weight, recurrent_a, dt_bias, output_norm_weight, output, convolution_state,
                     recurrent_state, workspace, workspace_bytes, shape,
                     qwen35_gated_delta_select_policy(shape, shape.tokens), dtype, weight_dtype, stream);
}

} // namespace raftinfer::kernels
