// Host-only check of the C++ drop-in header: it must compile with the call patterns RAFTInfer's executor uses
// (cpp/execution/qwen35_executor.cu:2027-2055,2118-2126), and the planner / refusal behaviour must match the
// reference's contract tests (cpp/tests/qwen35_cuda_attention_test.cu:263-440).  No GPU is touched: every call
// below either is pure host arithmetic or is refused before a launch.
#include <raftinfer_b200/kernels.hpp>
#include <raftinfer_b200/primitives.hpp>

#include <cstdio>
#include <cstdlib>

namespace rk = raftinfer::kernels;
using Mode = raftinfer::Qwen35DecodeAttentionMode;

#define EXPECT(cond)                                                                                         \
  do {                                                                                                       \
    if (!(cond)) {                                                                                           \
      std::fprintf(stderr, "%s:%d: expectation failed: %s\n", __FILE__, __LINE__, #cond);                    \
      std::exit(1);                                                                                          \
    }                                                                                                        \
  } while (0)

template <class Error, class Fn> bool throws(Fn &&fn) {
  try {
    fn();
  } catch (const Error &) {
    return true;
  }
  return false;
}

int main() {
  const rk::Qwen35AttentionShape model{1, 16, 4, 256, 4096, 0};
  const auto single = rk::qwen35_online_decode_plan(model, Mode::single_block, 128);
  EXPECT(single.resolved_mode == Mode::single_block && single.context_bucket_tokens == 512 &&
         single.active_partition_capacity == 1);
  const auto automatic = rk::qwen35_online_decode_plan(model, Mode::auto_select, 513);
  EXPECT((automatic == rk::Qwen35OnlineDecodePlan{Mode::split_k_256, 256, 256, 1024, 4}));
  const auto layout = rk::qwen35_online_decode_workspace_layout(model, Mode::split_k_256);
  EXPECT(layout.partial_count == 256 && layout.bytes == 264192 && layout.value_offset_bytes == 2048);
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] { (void)rk::qwen35_online_decode_plan(model, Mode::single_block, 0); }));

  const rk::Qwen35AttentionLaunchPolicy policy{raftinfer::Qwen35AttentionImplementation::online_tiled,
                                               raftinfer::Qwen35KvCacheDType::bf16,
                                               raftinfer::Qwen35KvCacheLayout::head_major};
  EXPECT(rk::qwen35_attention_cache_bytes(model, policy) == 4096u * 4096u);
  EXPECT(rk::qwen35_attention_workspace_bytes(model, policy) == 0);
  EXPECT(rk::qwen35_online_attention_workspace_bytes(model) == 0);
  EXPECT(rk::qwen35_online_attention_prefill_supported({4, 16, 4, 256, 8, 0}, RAFTINFER_DTYPE_BF16, policy));
  EXPECT(!rk::qwen35_online_attention_prefill_supported({4, 16, 4, 256, 8, 0}, RAFTINFER_DTYPE_F16, policy));

  // executor call patterns, refused on the null stream before anything is launched
  void *fake = reinterpret_cast<void *>(0x1000);
  const auto plan = rk::qwen35_online_decode_plan(model, Mode::split_k_256, 1);
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_online_attention_decode(fake, fake, fake, fake, fake, fake, 1u << 26, fake, layout.bytes, model,
                                       RAFTINFER_DTYPE_F32, raftinfer::Qwen35KvCacheDType::bf16,
                                       raftinfer::Qwen35KvCacheLayout::head_major, plan, nullptr, nullptr);
  }));
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_causal_attention(fake, fake, fake, fake, fake, fake, 1u << 26, nullptr, 0, {4, 16, 4, 256, 8, 0},
                                RAFTINFER_DTYPE_F32, policy, nullptr);
  }));
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_online_attention_decode(fake, fake, fake, fake, fake, fake, 1u << 26, model, RAFTINFER_DTYPE_F32,
                                       raftinfer::Qwen35KvCacheDType::bf16,
                                       raftinfer::Qwen35KvCacheLayout::head_major, nullptr, nullptr);
  }));

  const rk::GatedDeltaShape delta{3, 4096, 16, 32, 128, 128, 4, 1.0e-6F};
  EXPECT(rk::qwen35_gated_delta_workspace_bytes(delta) >= 3 * (8192 + 4096) * sizeof(float));
  EXPECT(rk::qwen35_gated_delta_select_policy(delta, 3).warps_per_block == 4);
  EXPECT(rk::qwen35_gated_delta_schedule_diagnostic(delta, 1).rejection_reason == "not_tuned");
  EXPECT(throws<rk::Qwen35DeltaError>([&] {
    rk::qwen35_gated_delta(fake, fake, fake, fake, fake, fake, static_cast<float *>(fake),
                           static_cast<float *>(fake), fake, 1u << 30, delta, RAFTINFER_DTYPE_BF16,
                           RAFTINFER_DTYPE_F32, nullptr);
  }));
  auto bad = delta;
  bad.value_heads = 33;
  EXPECT(throws<rk::Qwen35DeltaError>([&] { (void)rk::qwen35_gated_delta_workspace_bytes(bad); }));
  // the two pre-attention primitives, called the way cpp/execution/qwen35_executor.cu:1989-2015 calls them
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_split_full_query_gate(fake, fake, fake, 4, 16, 256, RAFTINFER_DTYPE_F32, nullptr);
  }));
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_qk_norm_rope(fake, fake, fake,
                            rk::QkNormRopeShape{.tokens = 4, .heads = 16, .head_dim = 256, .rotary_dim = 258,
                                                .position_offset = 0, .rope_base = 1.0e7F},
                            1.0e-6F, RAFTINFER_DTYPE_F32, RAFTINFER_DTYPE_F32, reinterpret_cast<cudaStream_t>(fake));
  }));
  EXPECT(throws<rk::Qwen35PrimitiveError>([&] {
    rk::qwen35_attention_prologue(fake, fake, fake, fake, fake, fake, fake, fake, fake, {4, 16, 4, 256, 8, 0}, 64,
                                  1.0e7F, 1.0e-6F, RAFTINFER_DTYPE_F32, RAFTINFER_DTYPE_F32, RAFTINFER_DTYPE_BF16,
                                  nullptr);
  }));
  std::puts("dropin ok");
  return 0;
}
