// Drop-in C++ face of the two pre-attention primitives of cpp/kernels/qwen35_primitives.cuh that librib200 serves:
// qwen35_qk_norm_rope (:61-66) and qwen35_split_full_query_gate (:90-93), with the reference's names, argument
// order and exception type, plus the fused call that replaces the executor's three
// (cpp/execution/qwen35_executor.cu:1989-2015).  The rest of that reference header (embedding, rms_norm, swiglu,
// argmax, ...) is not part of the path this library replaces: include this header for the translation units that
// call only these entry points, or call the C ABI of rib200.h next to the reference's own header.
#pragma once

#include "kernels.hpp"

namespace raftinfer::kernels {

// cpp/kernels/qwen35_primitives.cuh:32-39
struct QkNormRopeShape {
  std::size_t tokens;
  std::size_t heads;
  std::size_t head_dim;
  std::size_t rotary_dim;
  std::size_t position_offset;
  float rope_base;
};

inline void qwen35_qk_norm_rope(const void *input, const void *weight, void *output, QkNormRopeShape shape,
                                float epsilon, RaftInferDataType dtype, RaftInferDataType weight_dtype,
                                cudaStream_t stream, const std::uint32_t *device_position = nullptr) {
  const Rib200QkNormRopeShape s{shape.tokens,     shape.heads,           shape.head_dim,
                                shape.rotary_dim, shape.position_offset, shape.rope_base};
  detail::check(rib200_qk_norm_rope(input, weight, output, &s, epsilon, static_cast<int32_t>(dtype),
                                    static_cast<int32_t>(weight_dtype), stream, device_position));
}

inline void qwen35_split_full_query_gate(const void *query_gate, void *query, void *gate, std::size_t tokens,
                                         std::size_t heads, std::size_t head_dim, RaftInferDataType dtype,
                                         cudaStream_t stream) {
  detail::check(rib200_split_full_query_gate(query_gate, query, gate, tokens, heads, head_dim,
                                             static_cast<int32_t>(dtype), stream));
}

// No counterpart in the reference as one call: split + norm/rope of q + norm/rope of k + casts, outputs in
// output_dtype (BF16 for the attention kernels' fastest path).
inline void qwen35_attention_prologue(const void *query_gate, const void *key, const void *value,
                                      const void *query_norm_weight, const void *key_norm_weight, void *query,
                                      void *gate, void *key_out, void *value_out, Qwen35AttentionShape shape,
                                      std::size_t rotary_dim, float rope_base, float epsilon, RaftInferDataType dtype,
                                      RaftInferDataType weight_dtype, RaftInferDataType output_dtype,
                                      cudaStream_t stream, const std::uint32_t *device_position = nullptr) {
  const Rib200AttentionShape s = detail::to_c(shape);
  detail::check(rib200_attention_prologue(query_gate, key, value, query_norm_weight, key_norm_weight, query, gate,
                                          key_out, value_out, &s, rotary_dim, rope_base, epsilon,
                                          static_cast<int32_t>(dtype), static_cast<int32_t>(weight_dtype),
                                          static_cast<int32_t>(output_dtype), device_position, stream));
}

} // namespace raftinfer::kernels
