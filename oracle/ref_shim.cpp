// TEST INFRASTRUCTURE ONLY.  extern "C" doorway onto the RAFTInfer CPU
// reference library (cpp/reference/qwen35.cpp, correctness.cpp), compiled
// unmodified from the reference checkout by oracle/Makefile into
// oracle/_ref/libraftinfer_ref.so.  This file holds no arithmetic of its own:
// it only adapts pointers to the std::span signatures of
// cpp/reference/qwen35.hpp:64-88 and cpp/reference/correctness.hpp:30-34.

#include "reference/correctness.hpp"
#include "reference/qwen35.hpp"

#include <cstddef>
#include <cstring>
#include <exception>
#include <span>

namespace ref = raftinfer::reference;

extern "C" {

// qwen35_gated_full_attention, cpp/reference/qwen35.hpp:70-73.
int ref_full_attention(const float *input, float *output, const float *q_norm,
                       const float *k_norm, const float *out_w,
                       std::size_t tokens, std::size_t hidden,
                       std::size_t q_heads, std::size_t kv_heads,
                       std::size_t head_dim, std::size_t rotary,
                       std::size_t pos_offset, float rope_base, float eps) {
  try {
    const ref::FullAttentionReferenceArgs args{
        .tokens = tokens,
        .hidden_size = hidden,
        .query_heads = q_heads,
        .kv_heads = kv_heads,
        .head_dim = head_dim,
        .rotary_dim = rotary,
        .position_offset = pos_offset,
        .rope_base = rope_base,
        .epsilon = eps};
    const std::size_t stride = q_heads * head_dim + 2 * kv_heads * head_dim + hidden;
    ref::qwen35_gated_full_attention(
        std::span<const float>(input, tokens * stride),
        std::span<float>(output, tokens * hidden),
        ref::FullAttentionReferenceWeights{
            .query_norm_weight = std::span<const float>(q_norm, head_dim),
            .key_norm_weight = std::span<const float>(k_norm, head_dim),
            .output_weight = std::span<const float>(out_w, hidden * hidden)},
        args);
    return 0;
  } catch (const std::exception &) {
    return 1;
  }
}

// qwen35_gated_delta_prefill / _step, cpp/reference/qwen35.hpp:78-88.
// conv_state [conv_dim][W-1] and rec_state [Hv][dk][dv] are read and written
// back.  per_step != 0 drives qwen35_gated_delta_step token by token.
int ref_gated_delta(const float *input, float *output, const float *conv_w,
                    const float *rec_a, const float *dt_bias,
                    const float *out_norm_w, float *conv_state,
                    float *rec_state, std::size_t tokens, std::size_t hidden,
                    std::size_t key_heads, std::size_t value_heads,
                    std::size_t key_dim, std::size_t value_dim,
                    std::size_t conv_width, float eps, int per_step) {
  try {
    ref::GatedDeltaReferenceArgs args{.tokens = tokens,
                                      .hidden_size = hidden,
                                      .key_heads = key_heads,
                                      .value_heads = value_heads,
                                      .key_dim = key_dim,
                                      .value_dim = value_dim,
                                      .conv_width = conv_width,
                                      .epsilon = eps};
    const std::size_t conv_dim = 2 * key_heads * key_dim + value_heads * value_dim;
    const std::size_t stride = conv_dim + 2 * value_heads + hidden;
    ref::GatedDeltaReferenceState state(args);
    std::memcpy(state.convolution.data(), conv_state,
                state.convolution.size() * sizeof(float));
    std::memcpy(state.recurrent.data(), rec_state,
                state.recurrent.size() * sizeof(float));
    const ref::GatedDeltaReferenceWeights weights{
        .conv_weight = std::span<const float>(conv_w, conv_dim * conv_width),
        .recurrent_a = std::span<const float>(rec_a, value_heads),
        .dt_bias = std::span<const float>(dt_bias, value_heads),
        .output_norm_weight = std::span<const float>(out_norm_w, value_dim)};
    if (per_step != 0) {
      for (std::size_t t = 0; t < tokens; ++t) {
        ref::qwen35_gated_delta_step(
            std::span<const float>(input + t * stride, stride),
            std::span<float>(output + t * hidden, hidden), weights, args,
            state);
      }
    } else {
      ref::qwen35_gated_delta_prefill(
          std::span<const float>(input, tokens * stride),
          std::span<float>(output, tokens * hidden), weights, args, state);
    }
    std::memcpy(conv_state, state.convolution.data(),
                state.convolution.size() * sizeof(float));
    std::memcpy(rec_state, state.recurrent.data(),
                state.recurrent.size() * sizeof(float));
    return 0;
  } catch (const std::exception &) {
    return 1;
  }
}

// compare, cpp/reference/correctness.hpp:30-34.
int ref_compare(const float *cand, const float *reference, std::size_t n,
                double rel_floor, double *out4) {
  try {
    const auto m = ref::compare(std::span<const float>(cand, n),
                                std::span<const float>(reference, n), rel_floor);
    out4[0] = m.max_absolute_error;
    out4[1] = m.max_relative_error;
    out4[2] = m.cosine_similarity;
    out4[3] = static_cast<double>(m.nonfinite_mismatches);
    return 0;
  } catch (const std::exception &) {
    return 1;
  }
}

} // extern "C"
