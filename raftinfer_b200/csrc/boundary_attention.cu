// Host side of the attention entry points: shape and plan arithmetic, argument validation and
// dispatch.  Argument meaning and refusal behaviour follow cpp/kernels/qwen35_attention.cu:109-129,
// 417-443,565-613 and cpp/kernels/qwen35_online_attention.cu:33-140,185-196,1071-1314.
//
// What this library narrows: activations FP32 or BF16; KV cache BF16 head-major only (other cache
// types return RIB200_STATUS_UNSUPPORTED instead of taking a second code path); every tensor pointer
// 16-byte aligned (the kernels move 16-byte vectors).

#include "common.hpp"

#include <cstdint>
#include <limits>

namespace rib200 {
namespace {

constexpr std::size_t kModelQueryHeads = 16;
constexpr std::size_t kModelKvHeads = 4;
constexpr std::size_t kModelHeadDim = 256;
constexpr std::size_t kMinimumBucketTokens = 512;

const Rib200AttentionShape &deref(const Rib200AttentionShape *shape) {
  require(shape != nullptr, "attention shape pointer is null");
  return *shape;
}

std::size_t context_now(const Rib200AttentionShape &s) {
  return add(s.past_tokens, s.tokens, "attention context length overflows");
}

std::size_t kv_row_elements(const Rib200AttentionShape &s) {
  return mul(s.kv_heads, s.head_dim, "attention KV row size overflows");
}

// cpp/kernels/qwen35_attention.cu:109-129
void validate_shape(const Rib200AttentionShape &s) {
  require(s.tokens > 0, "attention tokens must be positive");
  require(s.query_heads > 0, "attention query_heads must be positive");
  require(s.kv_heads > 0, "attention kv_heads must be positive");
  require(s.head_dim > 0, "attention head_dim must be positive");
  require(s.max_context_tokens > 0, "attention max_context_tokens must be positive");
  require(s.query_heads % s.kv_heads == 0, "attention query_heads must be a multiple of kv_heads");
  require(context_now(s) <= s.max_context_tokens, "attention context exceeds the cache capacity");
  (void)mul(s.tokens, mul(s.query_heads, s.head_dim, "attention row size overflows"),
            "attention output size overflows");
  (void)mul(2, mul(s.max_context_tokens, kv_row_elements(s), "attention cache size overflows"),
            "attention cache size overflows");
}

void validate_policy(Rib200AttentionLaunchPolicy policy) {
  require(policy.implementation <= RIB200_ATTENTION_ONLINE_TILED, "unknown attention implementation");
  require(policy.kv_cache_dtype <= RIB200_KV_CACHE_BF16, "unknown KV cache dtype");
  require(policy.kv_cache_layout <= RIB200_KV_LAYOUT_HEAD_MAJOR, "unknown KV cache layout");
}

std::size_t cache_element_bytes(std::uint8_t dtype) {
  require(dtype <= RIB200_KV_CACHE_BF16, "unknown KV cache dtype");
  return dtype == RIB200_KV_CACHE_F32 ? 4 : 2;
}

std::size_t cache_bytes(const Rib200AttentionShape &s, std::uint8_t dtype, const char *what) {
  return mul(mul(2, mul(s.max_context_tokens, kv_row_elements(s), what), what), cache_element_bytes(dtype), what);
}

std::size_t materialized_workspace_floats(const Rib200AttentionShape &s) {
  validate_shape(s);
  return mul(mul(s.tokens, s.query_heads, "attention workspace size overflows"), context_now(s),
             "attention workspace size overflows");
}

bool fits(std::size_t a, std::size_t b) { return a == 0 || b <= std::numeric_limits<std::size_t>::max() / a; }

// cpp/kernels/qwen35_online_attention.cu:33-94
bool prefill_signature_ok(const Rib200AttentionShape &s, int32_t activation_dtype, std::uint8_t cache_dtype,
                          std::uint8_t cache_layout) {
  if (s.tokens <= 1 || s.query_heads == 0 || s.kv_heads == 0 || s.head_dim == 0 || s.head_dim > kModelHeadDim ||
      s.max_context_tokens == 0 || s.query_heads % s.kv_heads != 0 || s.past_tokens > s.max_context_tokens ||
      s.tokens > s.max_context_tokens - s.past_tokens) {
    return false;
  }
  if (activation_dtype != RIB200_DTYPE_F32 && activation_dtype != RIB200_DTYPE_BF16) {
    return false;
  }
  if (cache_dtype > RIB200_KV_CACHE_BF16 || cache_layout > RIB200_KV_LAYOUT_HEAD_MAJOR) {
    return false;
  }
  if (!fits(s.kv_heads, s.head_dim) || !fits(s.query_heads, s.head_dim)) {
    return false;
  }
  const std::size_t kv_row = s.kv_heads * s.head_dim;
  if (!fits(s.tokens, kv_row) || !fits(s.max_context_tokens, kv_row) ||
      !fits(s.tokens, s.query_heads * s.head_dim)) {
    return false;
  }
  const std::size_t plane = s.max_context_tokens * kv_row;
  return fits(2, plane) && fits(2 * plane, cache_dtype == RIB200_KV_CACHE_F32 ? 4 : 2) &&
         s.max_context_tokens <= 0x7FFFFFFFU && s.tokens <= 0x7FFFFFFFU;
}

// cpp/kernels/qwen35_online_attention.cu:96-140
bool decode_signature_ok(const Rib200AttentionShape &s, int32_t activation_dtype, std::uint8_t cache_dtype,
                         std::uint8_t cache_layout) {
  if (s.tokens != 1 || s.query_heads != kModelQueryHeads || s.kv_heads != kModelKvHeads ||
      s.head_dim != kModelHeadDim || s.max_context_tokens == 0 || s.past_tokens >= s.max_context_tokens) {
    return false;
  }
  if (activation_dtype != RIB200_DTYPE_F32 && activation_dtype != RIB200_DTYPE_BF16) {
    return false;
  }
  if (cache_dtype > RIB200_KV_CACHE_BF16 || cache_layout > RIB200_KV_LAYOUT_HEAD_MAJOR) {
    return false;
  }
  const std::size_t kv_row = s.kv_heads * s.head_dim;
  if (!fits(s.max_context_tokens, kv_row)) {
    return false;
  }
  const std::size_t plane = s.max_context_tokens * kv_row;
  return fits(2, plane) && fits(2 * plane, 4);
}

bool model_decode_shape(const Rib200AttentionShape &s) {
  return s.tokens == 1 && s.query_heads == kModelQueryHeads && s.kv_heads == kModelKvHeads &&
         s.head_dim == kModelHeadDim && s.max_context_tokens != 0;
}

std::size_t partition_tokens_of(std::uint8_t mode) {
  switch (mode) {
  case RIB200_DECODE_SPLIT_K_256:
    return 256;
  case RIB200_DECODE_SPLIT_K_512:
    return 512;
  case RIB200_DECODE_SINGLE_BLOCK:
  case RIB200_DECODE_AUTO_SELECT:
    return 0;
  default:
    break;
  }
  require(false, "unknown online decode attention mode");
  return 0;
}

// cpp/kernels/qwen35_online_attention.cu:185-196: smallest power of two >= context starting at 512,
// capped at the cache capacity.
std::size_t bucket_tokens(const Rib200AttentionShape &s, std::size_t context) {
  std::size_t bucket = kMinimumBucketTokens;
  while (bucket < context && bucket < s.max_context_tokens) {
    if (bucket > std::numeric_limits<std::size_t>::max() / 2) {
      bucket = s.max_context_tokens;
      break;
    }
    bucket *= 2;
  }
  return bucket < s.max_context_tokens ? bucket : s.max_context_tokens;
}

Rib200OnlineDecodePlan make_plan(const Rib200AttentionShape &s, std::uint8_t requested, std::size_t context) {
  require(s.max_context_tokens != 0, "online decode plan: max_context_tokens is zero");
  require(context != 0, "online decode plan: context_tokens is zero");
  require(context <= s.max_context_tokens, "online decode plan: context_tokens exceed max_context_tokens");
  const std::uint8_t mode =
      requested == RIB200_DECODE_AUTO_SELECT ? static_cast<std::uint8_t>(RIB200_DECODE_SPLIT_K_256) : requested;
  const std::size_t part = partition_tokens_of(mode);
  if (part != 0) {
    require(model_decode_shape(s), "split-k online decode needs 16 query heads, 4 kv heads, head_dim 256");
  }
  Rib200OnlineDecodePlan plan{};
  plan.resolved_mode = mode;
  plan.context_bucket_tokens = bucket_tokens(s, context);
  if (part == 0) {
    plan.partition_tokens = 0;
    plan.split_k_threshold_tokens = 0;
    plan.active_partition_capacity = 1;
    return plan;
  }
  plan.partition_tokens = part;
  plan.split_k_threshold_tokens = part;
  plan.active_partition_capacity = ceil_div(plan.context_bucket_tokens, part, "online decode plan overflow");
  return plan;
}

Rib200OnlineDecodeWorkspaceLayout make_layout(const Rib200AttentionShape &s, std::uint8_t mode) {
  require(mode != RIB200_DECODE_AUTO_SELECT, "online decode workspace: the mode must be resolved first");
  const std::size_t part = partition_tokens_of(mode);
  Rib200OnlineDecodeWorkspaceLayout layout{};
  if (part == 0) {
    return layout;
  }
  require(model_decode_shape(s), "split-k online decode needs 16 query heads, 4 kv heads, head_dim 256");
  const std::size_t max_parts = ceil_div(s.max_context_tokens, part, "online decode workspace overflow");
  layout.partial_count = mul(s.query_heads, max_parts, "online decode workspace overflow");
  const std::size_t scalar_bytes = mul(layout.partial_count, sizeof(float), "online decode workspace overflow");
  layout.max_offset_bytes = 0;
  layout.sum_offset_bytes = scalar_bytes;
  layout.value_offset_bytes = mul(2, scalar_bytes, "online decode workspace overflow");
  layout.bytes = add(layout.value_offset_bytes,
                     mul(mul(layout.partial_count, s.head_dim, "online decode workspace overflow"), sizeof(float),
                         "online decode workspace overflow"),
                     "online decode workspace overflow");
  return layout;
}

void require_aligned16(const void *ptr, const char *message) {
  require(reinterpret_cast<std::uintptr_t>(ptr) % 16 == 0, message);
}

// `outputs` non-null: the head-sharded form, tiles go to `world` full-width buffers at `head_offset`.
void online_prefill(const void *query, const void *key, const void *value, const void *gate, void *output,
                    void *kv_cache, std::size_t kv_cache_bytes, const Rib200AttentionShape &s,
                    int32_t activation_dtype, std::uint8_t cache_dtype, std::uint8_t cache_layout,
                    cudaStream_t stream, void *const *outputs = nullptr, std::size_t world = 0, std::size_t rank = 0,
                    std::size_t total_query_heads = 0, std::size_t head_offset = 0) {
  require(query != nullptr, "online attention: query pointer is null");
  require(key != nullptr, "online attention: key pointer is null");
  require(value != nullptr, "online attention: value pointer is null");
  require(gate != nullptr, "online attention: gate pointer is null");
  require(output != nullptr || outputs != nullptr, "online attention: output pointer is null");
  require(kv_cache != nullptr, "online attention: KV cache pointer is null");
  require(stream != nullptr, "online attention: CUDA stream is null");
  require(prefill_signature_ok(s, activation_dtype, cache_dtype, cache_layout),
          "online attention: unsupported prefill signature");
  require(kv_cache_bytes >= cache_bytes(s, cache_dtype, "online attention cache size overflows"),
          "online attention: KV cache is too small");
  unsupported(cache_dtype == RIB200_KV_CACHE_BF16 && cache_layout == RIB200_KV_LAYOUT_HEAD_MAJOR,
              "online attention: this library serves the BF16 head-major KV cache only");
  unsupported(s.head_dim == kModelHeadDim && s.query_heads <= 1024,
              "online attention: prefill is built for head_dim 256");
  require_aligned16(query, "online attention: query is not 16-byte aligned");
  require_aligned16(key, "online attention: key is not 16-byte aligned");
  require_aligned16(value, "online attention: value is not 16-byte aligned");
  require_aligned16(gate, "online attention: gate is not 16-byte aligned");
  if (outputs == nullptr) {
    require_aligned16(output, "online attention: output is not 16-byte aligned");
  }
  require_aligned16(kv_cache, "online attention: KV cache is not 16-byte aligned");
  PrefillArgs args{};
  if (outputs != nullptr) {
    require(world >= 1 && world <= 8, "head-sharded prefill: world must be between 1 and 8");
    require(rank < world, "head-sharded prefill: rank is out of range");
    require(head_offset + s.query_heads <= total_query_heads,
            "head-sharded prefill: this rank's heads do not fit in the output row");
    for (std::size_t r = 0; r < world; ++r) {
      require(outputs[r] != nullptr, "head-sharded prefill: an output pointer is null");
      require_aligned16(outputs[r], "head-sharded prefill: an output is not 16-byte aligned");
      args.outputs[r] = outputs[r];
    }
    args.output_count = static_cast<std::uint32_t>(world);
    args.output_self = static_cast<std::uint32_t>(rank);
    args.output_heads = static_cast<std::uint32_t>(total_query_heads);
    args.output_head_offset = static_cast<std::uint32_t>(head_offset);
  }
  args.query = query;
  args.key = key;
  args.value = value;
  args.gate = gate;
  args.output = output;
  args.kv_cache = kv_cache;
  args.tokens = static_cast<std::uint32_t>(s.tokens);
  args.past_tokens = static_cast<std::uint32_t>(s.past_tokens);
  args.max_context_tokens = static_cast<std::uint32_t>(s.max_context_tokens);
  args.query_heads = static_cast<std::uint32_t>(s.query_heads);
  args.kv_heads = static_cast<std::uint32_t>(s.kv_heads);
  args.activations_f32 = activation_dtype == RIB200_DTYPE_F32;
  launch_prefill_attention(args, stream);
}

void online_decode(const void *query, const void *key, const void *value, const void *gate, void *output,
                   void *kv_cache, std::size_t kv_cache_bytes, void *workspace, std::size_t workspace_bytes,
                   const Rib200AttentionShape &s, int32_t activation_dtype, std::uint8_t cache_dtype,
                   std::uint8_t cache_layout, const Rib200OnlineDecodePlan &plan,
                   const std::uint32_t *device_position, cudaStream_t stream, bool early_kv_fetch = false) {
  require(query != nullptr, "online decode: query pointer is null");
  require(key != nullptr, "online decode: key pointer is null");
  require(value != nullptr, "online decode: value pointer is null");
  require(gate != nullptr, "online decode: gate pointer is null");
  require(output != nullptr, "online decode: output pointer is null");
  require(kv_cache != nullptr, "online decode: KV cache pointer is null");
  require(stream != nullptr, "online decode: CUDA stream is null");
  require(decode_signature_ok(s, activation_dtype, cache_dtype, cache_layout),
          "online decode: unsupported decode signature");
  require(plan.resolved_mode != RIB200_DECODE_AUTO_SELECT, "online decode: the plan mode must be resolved");
  const std::size_t part = partition_tokens_of(plan.resolved_mode);
  require(plan.partition_tokens == part, "online decode: plan partition size is inconsistent");
  if (part == 0) {
    require(plan.split_k_threshold_tokens == 0 && plan.active_partition_capacity == 1,
            "online decode: single-block plan is inconsistent");
    require(workspace_bytes == 0, "online decode: single-block decode takes no split-k workspace");
  } else {
    require(plan.split_k_threshold_tokens == part, "online decode: split-k threshold is inconsistent");
    require(plan.context_bucket_tokens != 0 && plan.context_bucket_tokens <= s.max_context_tokens,
            "online decode: split-k context bucket is invalid");
    require(plan.active_partition_capacity == ceil_div(plan.context_bucket_tokens, part, "online decode overflow"),
            "online decode: split-k partition capacity is inconsistent");
    require(device_position != nullptr || s.past_tokens + 1 <= plan.context_bucket_tokens,
            "online decode: context exceeds the planned bucket");
  }
  const Rib200OnlineDecodeWorkspaceLayout layout = make_layout(s, plan.resolved_mode);
  if (layout.bytes != 0) {
    require(workspace != nullptr, "online decode: split-k workspace is null");
    require(workspace_bytes >= layout.bytes, "online decode: split-k workspace is too small");
    require_aligned16(workspace, "online decode: workspace is not 16-byte aligned");
  }
  require(kv_cache_bytes >= cache_bytes(s, cache_dtype, "online decode cache size overflows"),
          "online decode: KV cache is too small");
  unsupported(cache_dtype == RIB200_KV_CACHE_BF16 && cache_layout == RIB200_KV_LAYOUT_HEAD_MAJOR,
              "online decode: this library serves the BF16 head-major KV cache only");
  require(s.max_context_tokens <= 0x7FFFFFFFU, "online decode: max_context_tokens exceeds 2^31");
  require_aligned16(query, "online decode: query is not 16-byte aligned");
  require_aligned16(key, "online decode: key is not 16-byte aligned");
  require_aligned16(value, "online decode: value is not 16-byte aligned");
  require_aligned16(gate, "online decode: gate is not 16-byte aligned");
  require_aligned16(output, "online decode: output is not 16-byte aligned");
  require_aligned16(kv_cache, "online decode: KV cache is not 16-byte aligned");

  DecodeArgs args{};
  args.query = query;
  args.key = key;
  args.value = value;
  args.gate = gate;
  args.output = output;
  args.kv_cache = kv_cache;
  args.max_context_tokens = static_cast<std::uint32_t>(s.max_context_tokens);
  args.host_position = static_cast<std::uint32_t>(s.past_tokens);
  args.device_position = device_position;
  args.partition_tokens = static_cast<std::uint32_t>(part);
  args.threshold_tokens = static_cast<std::uint32_t>(plan.split_k_threshold_tokens);
  args.partition_capacity = static_cast<std::uint32_t>(plan.active_partition_capacity);
  args.activations_f32 = activation_dtype == RIB200_DTYPE_F32;
  args.early_kv_fetch = early_kv_fetch;
  if (layout.bytes != 0) {
    auto *base = static_cast<unsigned char *>(workspace);
    args.partial_max = reinterpret_cast<float *>(base + layout.max_offset_bytes);
    args.partial_sum = reinterpret_cast<float *>(base + layout.sum_offset_bytes);
    args.partial_value = reinterpret_cast<float *>(base + layout.value_offset_bytes);
    args.max_partitions = static_cast<std::uint32_t>(layout.partial_count / s.query_heads);
  }
  launch_decode_attention(args, stream);
}

} // namespace
} // namespace rib200

using namespace rib200;

extern "C" {

Rib200Status rib200_attention_workspace_floats(const Rib200AttentionShape *shape, size_t *floats) {
  return guarded([&] {
    require(floats != nullptr, "output pointer is null");
    *floats = materialized_workspace_floats(deref(shape));
  });
}

Rib200Status rib200_attention_cache_bytes(const Rib200AttentionShape *shape, Rib200AttentionLaunchPolicy policy,
                                          size_t *bytes) {
  return guarded([&] {
    require(bytes != nullptr, "output pointer is null");
    validate_shape(deref(shape));
    validate_policy(policy);
    *bytes = cache_bytes(*shape, policy.kv_cache_dtype, "attention cache size overflows");
  });
}

Rib200Status rib200_attention_workspace_bytes(const Rib200AttentionShape *shape, Rib200AttentionLaunchPolicy policy,
                                              size_t *bytes) {
  return guarded([&] {
    require(bytes != nullptr, "output pointer is null");
    validate_policy(policy);
    if (policy.implementation == RIB200_ATTENTION_MATERIALIZED_REFERENCE) {
      *bytes = mul(materialized_workspace_floats(deref(shape)), sizeof(float), "attention workspace size overflows");
      return;
    }
    validate_shape(deref(shape));
    *bytes = 0;
  });
}

Rib200Status rib200_online_decode_plan(const Rib200AttentionShape *shape, uint8_t requested_mode,
                                       size_t context_tokens, Rib200OnlineDecodePlan *plan) {
  return guarded([&] {
    require(plan != nullptr, "output pointer is null");
    *plan = make_plan(deref(shape), requested_mode, context_tokens);
  });
}

Rib200Status rib200_online_decode_workspace_layout(const Rib200AttentionShape *shape, uint8_t resolved_mode,
                                                   Rib200OnlineDecodeWorkspaceLayout *layout) {
  return guarded([&] {
    require(layout != nullptr, "output pointer is null");
    *layout = make_layout(deref(shape), resolved_mode);
  });
}

Rib200Status rib200_online_attention_prefill_supported(const Rib200AttentionShape *shape, int32_t activation_dtype,
                                                       Rib200AttentionLaunchPolicy policy, int32_t *supported) {
  return guarded([&] {
    require(supported != nullptr, "output pointer is null");
    const Rib200AttentionShape &s = deref(shape);
    *supported = policy.implementation == RIB200_ATTENTION_ONLINE_TILED &&
                         prefill_signature_ok(s, activation_dtype, policy.kv_cache_dtype, policy.kv_cache_layout) &&
                         policy.kv_cache_dtype == RIB200_KV_CACHE_BF16 &&
                         policy.kv_cache_layout == RIB200_KV_LAYOUT_HEAD_MAJOR && s.head_dim == kModelHeadDim &&
                         s.query_heads <= 1024
                     ? 1
                     : 0;
  });
}

Rib200Status rib200_online_attention_workspace_bytes(const Rib200AttentionShape *shape, size_t *bytes) {
  return guarded([&] {
    (void)shape;
    require(bytes != nullptr, "output pointer is null");
    *bytes = 0;
  });
}

Rib200Status rib200_online_attention_prefill(const void *query, const void *key, const void *value,
                                             const void *gate, void *output, void *kv_cache, size_t kv_cache_bytes,
                                             const Rib200AttentionShape *shape, int32_t activation_dtype,
                                             uint8_t cache_dtype, uint8_t cache_layout, void *stream) {
  return guarded([&] {
    online_prefill(query, key, value, gate, output, kv_cache, kv_cache_bytes, deref(shape), activation_dtype,
                   cache_dtype, cache_layout, static_cast<cudaStream_t>(stream));
  });
}

Rib200Status rib200_online_attention_prefill_scatter(const void *query, const void *key, const void *value,
                                                     const void *gate, void *const *outputs, size_t world,
                                                     size_t rank, size_t total_query_heads, size_t head_offset,
                                                     void *kv_cache,
                                                     size_t kv_cache_bytes, const Rib200AttentionShape *shape,
                                                     int32_t activation_dtype, uint8_t cache_dtype,
                                                     uint8_t cache_layout, void *stream) {
  return guarded([&] {
    require(outputs != nullptr, "head-sharded prefill: output list is null");
    online_prefill(query, key, value, gate, nullptr, kv_cache, kv_cache_bytes, deref(shape), activation_dtype,
                   cache_dtype, cache_layout, static_cast<cudaStream_t>(stream), outputs, world, rank,
                   total_query_heads, head_offset);
  });
}

Rib200Status rib200_online_attention_decode(const void *query, const void *key, const void *value,
                                            const void *gate, void *output, void *kv_cache, size_t kv_cache_bytes,
                                            void *workspace, size_t workspace_bytes,
                                            const Rib200AttentionShape *shape, int32_t activation_dtype,
                                            uint8_t cache_dtype, uint8_t cache_layout,
                                            const Rib200OnlineDecodePlan *plan, const uint32_t *device_position,
                                            void *stream) {
  return guarded([&] {
    require(plan != nullptr, "online decode: plan pointer is null");
    online_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace, workspace_bytes,
                  deref(shape), activation_dtype, cache_dtype, cache_layout, *plan, device_position,
                  static_cast<cudaStream_t>(stream));
  });
}

Rib200Status rib200_online_attention_decode_early_kv_fetch(const void *query, const void *key, const void *value,
                                                           const void *gate, void *output, void *kv_cache,
                                                           size_t kv_cache_bytes, void *workspace,
                                                           size_t workspace_bytes, const Rib200AttentionShape *shape,
                                                           int32_t activation_dtype, uint8_t cache_dtype,
                                                           uint8_t cache_layout, const Rib200OnlineDecodePlan *plan,
                                                           void *stream) {
  return guarded([&] {
    require(plan != nullptr, "online decode: plan pointer is null");
    online_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, workspace, workspace_bytes,
                  deref(shape), activation_dtype, cache_dtype, cache_layout, *plan, nullptr,
                  static_cast<cudaStream_t>(stream), true);
  });
}

// One decode step driven from host memory: the token's rows go up, the step runs, the output comes back, and
// the call returns when it is there.
Rib200Status rib200_online_attention_decode_from_host(const void *host_token, void *host_output, void *device_token,
                                                      void *device_output, void *kv_cache, size_t kv_cache_bytes,
                                                      void *workspace, size_t workspace_bytes,
                                                      const Rib200AttentionShape *shape, int32_t activation_dtype,
                                                      uint8_t cache_dtype, uint8_t cache_layout,
                                                      const Rib200OnlineDecodePlan *plan,
                                                      const uint32_t *device_position, void *stream) {
  return guarded([&] {
    require(plan != nullptr, "online decode: plan pointer is null");
    require(host_token != nullptr && host_output != nullptr, "online decode from host: a host pointer is null");
    require(device_token != nullptr && device_output != nullptr, "online decode from host: a staging pointer is null");
    require(stream != nullptr, "online decode: CUDA stream is null");
    const Rib200AttentionShape &s = deref(shape);
    require(decode_signature_ok(s, activation_dtype, cache_dtype, cache_layout),
            "online decode: unsupported decode signature");
    const std::size_t element = activation_dtype == RIB200_DTYPE_F32 ? 4 : 2;
    const std::size_t q_bytes = s.query_heads * s.head_dim * element;
    const std::size_t kv_bytes = s.kv_heads * s.head_dim * element;
    require_aligned16(device_token, "online decode from host: staging is not 16-byte aligned");
    auto *staged = static_cast<unsigned char *>(device_token);
    cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
    // rows in the order q | k | v | gate
    cuda_ok(cudaMemcpyAsync(staged, host_token, 2 * q_bytes + 2 * kv_bytes, cudaMemcpyHostToDevice, cuda_stream),
            "online decode from host: copy in");
    // Page-locked host memory that the device can address takes the result straight from the kernel (16 heads x 256
    // values, written once); anything else gets it through device_output and a copy.
    void *direct = nullptr;
    cudaPointerAttributes attributes{};
    if (cudaPointerGetAttributes(&attributes, host_output) == cudaSuccess) {
      if (attributes.type == cudaMemoryTypeHost && attributes.devicePointer != nullptr &&
          reinterpret_cast<std::uintptr_t>(attributes.devicePointer) % 16 == 0) {
        direct = attributes.devicePointer;
      }
    } else {
      (void)cudaGetLastError(); // an unregistered pointer is not an error here
    }
    online_decode(staged, staged + q_bytes, staged + q_bytes + kv_bytes, staged + q_bytes + 2 * kv_bytes,
                  direct != nullptr ? direct : device_output, kv_cache, kv_cache_bytes, workspace, workspace_bytes, s,
                  activation_dtype, cache_dtype, cache_layout, *plan, device_position, cuda_stream);
    if (direct == nullptr) {
      cuda_ok(cudaMemcpyAsync(host_output, device_output, q_bytes, cudaMemcpyDeviceToHost, cuda_stream),
              "online decode from host: copy out");
    }
    cuda_ok(cudaStreamSynchronize(cuda_stream), "online decode from host: synchronise");
  });
}

// Dispatcher, cpp/kernels/qwen35_attention.cu:565-613.
Rib200Status rib200_causal_attention(const void *query, const void *key, const void *value, const void *gate,
                                     void *output, void *kv_cache, size_t kv_cache_bytes, void *workspace,
                                     size_t workspace_bytes, const Rib200AttentionShape *shape,
                                     int32_t activation_dtype, Rib200AttentionLaunchPolicy policy, void *stream) {
  return guarded([&] {
    const Rib200AttentionShape &s = deref(shape);
    validate_policy(policy);
    std::size_t need = 0;
    if (policy.implementation == RIB200_ATTENTION_MATERIALIZED_REFERENCE) {
      need = mul(materialized_workspace_floats(s), sizeof(float), "attention workspace size overflows");
    } else {
      validate_shape(s);
    }
    require(query != nullptr, "attention: query pointer is null");
    require(key != nullptr, "attention: key pointer is null");
    require(value != nullptr, "attention: value pointer is null");
    require(gate != nullptr, "attention: gate pointer is null");
    require(output != nullptr, "attention: output pointer is null");
    require(kv_cache != nullptr, "attention: kv_cache pointer is null");
    require(need == 0 || workspace != nullptr, "attention: workspace pointer is null");
    require(stream != nullptr, "attention: CUDA stream is null");
    require(kv_cache_bytes >= cache_bytes(s, policy.kv_cache_dtype, "attention cache size overflows"),
            "attention: KV cache is too small");
    require(workspace_bytes >= need, "attention: workspace is too small");
    require(activation_dtype == RIB200_DTYPE_F32 || activation_dtype == RIB200_DTYPE_F16 ||
                activation_dtype == RIB200_DTYPE_BF16,
            "attention: unknown activation dtype");
    unsupported(policy.implementation == RIB200_ATTENTION_ONLINE_TILED,
                "attention: the materialized logits path is the reference's test oracle and is not built here");
    require(workspace == nullptr && workspace_bytes == 0, "attention: the online path takes no logits workspace");
    auto *cuda_stream = static_cast<cudaStream_t>(stream);
    if (s.tokens == 1) {
      const Rib200OnlineDecodePlan plan = make_plan(s, RIB200_DECODE_SINGLE_BLOCK, s.past_tokens + 1);
      online_decode(query, key, value, gate, output, kv_cache, kv_cache_bytes, nullptr, 0, s, activation_dtype,
                    policy.kv_cache_dtype, policy.kv_cache_layout, plan, nullptr, cuda_stream);
      return;
    }
    online_prefill(query, key, value, gate, output, kv_cache, kv_cache_bytes, s, activation_dtype,
                   policy.kv_cache_dtype, policy.kv_cache_layout, cuda_stream);
  });
}

Rib200Status rib200_batched_decode_workspace_bytes(size_t batch, size_t max_context_tokens, size_t *bytes) {
  return guarded([&] {
    require(bytes != nullptr, "output pointer is null");
    require(batch > 0 && max_context_tokens > 0, "batched decode: batch and max_context_tokens must be positive");
    const std::size_t capacity = ceil_div(max_context_tokens, 256, "batched decode workspace overflow");
    const std::size_t partials = mul(mul(batch, kModelQueryHeads, "batched decode workspace overflow"), capacity,
                                     "batched decode workspace overflow");
    *bytes = mul(mul(partials, kModelHeadDim + 2, "batched decode workspace overflow"), sizeof(float),
                 "batched decode workspace overflow");
  });
}

Rib200Status rib200_batched_decode_attention(const void *query, const void *key, const void *value,
                                             const void *gate, void *output, void *const *kv_caches,
                                             const uint32_t *max_context_tokens, const uint32_t *positions,
                                             size_t batch, size_t largest_max_context_tokens, void *workspace,
                                             size_t workspace_bytes, void *stream) {
  return guarded([&] {
    require(query != nullptr && key != nullptr && value != nullptr && gate != nullptr && output != nullptr,
            "batched decode: an activation pointer is null");
    require(kv_caches != nullptr && max_context_tokens != nullptr && positions != nullptr,
            "batched decode: a per-sequence array pointer is null");
    require(workspace != nullptr, "batched decode: workspace is null");
    require(stream != nullptr, "batched decode: CUDA stream is null");
    require(batch > 0 && batch <= 65535, "batched decode: batch must be in 1..65535");
    require(largest_max_context_tokens > 0 && largest_max_context_tokens <= 0x7FFFFFFFU,
            "batched decode: largest_max_context_tokens out of range");
    const std::size_t capacity = ceil_div(largest_max_context_tokens, 256, "batched decode overflow");
    const std::size_t partials =
        mul(mul(batch, kModelQueryHeads, "batched decode overflow"), capacity, "batched decode overflow");
    const std::size_t need =
        mul(mul(partials, kModelHeadDim + 2, "batched decode overflow"), sizeof(float), "batched decode overflow");
    require(workspace_bytes >= need, "batched decode: workspace is too small");
    require_aligned16(query, "batched decode: query is not 16-byte aligned");
    require_aligned16(key, "batched decode: key is not 16-byte aligned");
    require_aligned16(value, "batched decode: value is not 16-byte aligned");
    require_aligned16(gate, "batched decode: gate is not 16-byte aligned");
    require_aligned16(output, "batched decode: output is not 16-byte aligned");
    require_aligned16(workspace, "batched decode: workspace is not 16-byte aligned");
    BatchedDecodeArgs args{};
    args.query = query;
    args.key = key;
    args.value = value;
    args.gate = gate;
    args.output = output;
    args.kv_caches = kv_caches;
    args.max_context_tokens = max_context_tokens;
    args.positions = positions;
    args.batch = static_cast<std::uint32_t>(batch);
    args.partition_capacity = static_cast<std::uint32_t>(capacity);
    args.workspace = static_cast<float *>(workspace);
    launch_batched_decode_attention(args, static_cast<cudaStream_t>(stream));
  });
}

Rib200Status rib200_paged_decode_attention(const void *query, const void *key, const void *value, const void *gate,
                                           void *output, void *page_pool, size_t pool_pages,
                                           const uint32_t *block_tables, size_t max_blocks_per_sequence,
                                           const uint32_t *positions, size_t batch, void *workspace,
                                           size_t workspace_bytes, void *stream) {
  return guarded([&] {
    require(query != nullptr && key != nullptr && value != nullptr && gate != nullptr && output != nullptr,
            "paged decode: an activation pointer is null");
    require(page_pool != nullptr && block_tables != nullptr && positions != nullptr,
            "paged decode: the page pool, the block tables or the positions pointer is null");
    require(workspace != nullptr, "paged decode: workspace is null");
    require(stream != nullptr, "paged decode: CUDA stream is null");
    require(batch > 0 && batch <= 65535, "paged decode: batch must be in 1..65535");
    require(pool_pages > 0 && pool_pages <= 0x7FFFFFFFU, "paged decode: pool_pages out of range");
    require(max_blocks_per_sequence > 0 && max_blocks_per_sequence <= (0x7FFFFFFFU / 256),
            "paged decode: max_blocks_per_sequence out of range");
    const std::size_t partials = mul(mul(batch, kModelQueryHeads, "paged decode overflow"), max_blocks_per_sequence,
                                     "paged decode overflow");
    const std::size_t need =
        mul(mul(partials, kModelHeadDim + 2, "paged decode overflow"), sizeof(float), "paged decode overflow");
    require(workspace_bytes >= need, "paged decode: workspace is too small");
    require_aligned16(query, "paged decode: query is not 16-byte aligned");
    require_aligned16(key, "paged decode: key is not 16-byte aligned");
    require_aligned16(value, "paged decode: value is not 16-byte aligned");
    require_aligned16(gate, "paged decode: gate is not 16-byte aligned");
    require_aligned16(output, "paged decode: output is not 16-byte aligned");
    require_aligned16(page_pool, "paged decode: page pool is not 16-byte aligned");
    require_aligned16(workspace, "paged decode: workspace is not 16-byte aligned");
    BatchedDecodeArgs args{};
    args.query = query;
    args.key = key;
    args.value = value;
    args.gate = gate;
    args.output = output;
    args.positions = positions;
    args.batch = static_cast<std::uint32_t>(batch);
    args.partition_capacity = static_cast<std::uint32_t>(max_blocks_per_sequence);
    args.workspace = static_cast<float *>(workspace);
    args.page_pool = page_pool;
    args.block_tables = block_tables;
    args.pool_pages = static_cast<std::uint32_t>(pool_pages);
    launch_batched_decode_attention(args, static_cast<cudaStream_t>(stream));
  });
}

} // extern "C"
