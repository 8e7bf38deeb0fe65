// Shared host-side plumbing of librib200: status conversion, checked size arithmetic and the
// internal launcher declarations that the boundary files call.
#pragma once

#include "../../include/rib200.h"

#include <cuda_runtime.h>
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <limits>
#include <string>

namespace rib200 {

// Thrown by validation code; converted to a Rib200Status at the C boundary.
struct Failure {
  int32_t code;
  std::string message;
};

inline void require(bool ok, const char *message, int32_t code = RIB200_STATUS_INVALID_ARGUMENT) {
  if (!ok) {
    throw Failure{code, message};
  }
}

inline void unsupported(bool ok, const char *message) { require(ok, message, RIB200_STATUS_UNSUPPORTED); }

inline std::size_t mul(std::size_t a, std::size_t b, const char *what) {
  require(a == 0 || b <= std::numeric_limits<std::size_t>::max() / a, what);
  return a * b;
}

inline std::size_t add(std::size_t a, std::size_t b, const char *what) {
  require(b <= std::numeric_limits<std::size_t>::max() - a, what);
  return a + b;
}

inline std::size_t ceil_div(std::size_t n, std::size_t d, const char *what) {
  require(d != 0, what);
  return n / d + (n % d == 0 ? 0 : 1);
}

inline void cuda_ok(cudaError_t err, const char *what) {
  if (err != cudaSuccess) {
    throw Failure{RIB200_STATUS_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(err)};
  }
}

Rib200Status ok_status();
Rib200Status fail_status(int32_t code, const std::string &message);

template <class Fn> Rib200Status guarded(Fn &&fn) {
  try {
    fn();
    return ok_status();
  } catch (const Failure &f) {
    return fail_status(f.code, f.message);
  } catch (const std::exception &e) {
    return fail_status(RIB200_STATUS_INTERNAL, e.what());
  } catch (...) {
    return fail_status(RIB200_STATUS_INTERNAL, "unknown failure");
  }
}

// Address of the per-device status word (file-scope __device__ variable), resolved once per device.
unsigned int *device_status_word();

// ---- decode attention (decode_attention.cu) -------------------------------------------------
struct DecodeArgs {
  const void *query;  // [16][256] activation dtype
  const void *key;    // [4][256]
  const void *value;  // [4][256]
  const void *gate;   // [16][256]
  void *output;       // [16][256]
  void *kv_cache;     // bf16 [2][4][max_ctx][256]
  float *partial_max; // split-k only
  float *partial_sum;
  float *partial_value;
  std::uint32_t max_context_tokens;
  std::uint32_t host_position;
  const std::uint32_t *device_position;
  std::uint32_t partition_tokens;   // 0 = single block
  std::uint32_t threshold_tokens;   // contexts below this are served directly by partition 0
  std::uint32_t partition_capacity; // grid.x
  std::uint32_t max_partitions;     // stride of the partial arrays
  bool activations_f32;
  bool early_kv_fetch; // host position only: the cache rows are fetched before the dependent-launch wait
};
// 128-byte opaque image of a driver tensor map (TMA descriptor); 64-byte aligned as the driver's type is.
struct alignas(64) TensorMapBytes {
  unsigned char bytes[128];
};
// Tiled map over a row-major FP32 matrix [rows][row_floats], box [box_rows][box_floats], 128-byte swizzle
// (box_floats * 4 must be 128).  Defined next to the other tensor-map code in prefill_attention.cu.
void encode_f32_rows_map(void *map_out, void *base, std::uint64_t row_floats, std::uint64_t rows,
                         std::uint32_t box_floats, std::uint32_t box_rows);

// Tiled map without swizzle over rows of FP32 or BF16 elements: `rows` rows of `row_elements` elements that lie
// `row_stride_elements` apart (a head range inside wider token rows); box [box_rows][box_elements]; rows past the
// last one arrive as zeros.  Base and row stride must be multiples of 16 bytes.
void encode_plain_rows_map(void *map_out, const void *base, bool f32, std::uint64_t row_elements,
                           std::uint64_t row_stride_elements, std::uint64_t rows, std::uint32_t box_elements,
                           std::uint32_t box_rows);

// Launch with programmatic stream serialisation: the grid may become resident while the kernel in front of it on the
// stream is still running (once that one has executed griddepcontrol.launch_dependents in every CTA, or ended), and
// must execute griddepcontrol.wait before it touches anything an earlier kernel of the stream writes or reads.
#ifdef __CUDACC__
template <typename... Params, typename... Args>
inline void launch_programmatic(void (*kernel)(Params...), dim3 grid, dim3 block, std::size_t shared_bytes,
                                cudaStream_t stream, const char *what, Args &&...args) {
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  cuda_ok(cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...), what);
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
#endif

void launch_decode_attention(const DecodeArgs &args, cudaStream_t stream);

// One decode step for a batch of ragged sequences (BF16 activations).
struct BatchedDecodeArgs {
  const void *query, *key, *value, *gate;
  void *output;
  void *const *kv_caches;
  const std::uint32_t *max_context_tokens;
  const std::uint32_t *positions;
  std::uint32_t batch;
  std::uint32_t partition_capacity; // partitions of the largest cache
  float *workspace;                 // max[batch][16*cap], then sum[batch][16*cap], then value[batch][16*cap][256]
  // paged form: kv_caches and max_context_tokens are null, partition_capacity is the width of a table row
  void *page_pool;                    // [pool_pages][2][4][256][256] BF16
  const std::uint32_t *block_tables;  // [batch][partition_capacity] page indices
  std::uint32_t pool_pages;
};
void launch_batched_decode_attention(const BatchedDecodeArgs &args, cudaStream_t stream);

// ---- prefill attention (prefill_attention.cu) -----------------------------------------------
struct PrefillArgs {
  const void *query;  // [tokens][query_heads][256] activation dtype
  const void *key;    // [tokens][kv_heads][256]
  const void *value;  // [tokens][kv_heads][256]
  const void *gate;   // [tokens][query_heads][256]
  void *output;       // [tokens][query_heads][256]
  void *kv_cache;     // bf16 [2][kv_heads][max_ctx][256]
  std::uint32_t tokens;
  std::uint32_t past_tokens;
  std::uint32_t max_context_tokens;
  std::uint32_t query_heads;
  std::uint32_t kv_heads;
  bool activations_f32;
  // Head-sharded form: the tile stores go to `output_count` buffers (this rank's and its peers'), each
  // [tokens][output_heads][256], at head index output_head_offset.  output_count == 0 means `output` alone.
  // The tile is stored into the rank's own buffer and forwarded from there to the others.
  void *outputs[8];
  std::uint32_t output_count;
  std::uint32_t output_self; // index of this rank's own buffer
  std::uint32_t output_heads;
  std::uint32_t output_head_offset;
};
void launch_prefill_attention(const PrefillArgs &args, cudaStream_t stream);
// device-side rendezvous of the ranks of one box (peer.cu)
void launch_peer_rendezvous(std::uint32_t *const *flags, std::uint32_t world, std::uint32_t rank, std::uint32_t epoch,
                            cudaStream_t stream, long long limit_cycles);

// ---- gated delta rule (gdn_recurrent.cu, gdn_chunk.cu, gdn_layer.cu) -------------------------
// Operands of the recurrence for `sequences` independent sequences of `tokens` tokens each.
// Element (seq, t, head, i) of q lives at q[(seq * tokens + t) * q_stride + head * 128 + i]; likewise k, v.
struct GdnCoreArgs {
  const void *q, *k, *v;
  std::size_t q_stride, k_stride, v_stride; // elements between consecutive tokens
  bool qkv_f32;
  const float *beta;      // [(seq * tokens + t) * value_heads + head]
  const float *log_decay; // same indexing
  float *state;           // [value_heads][128][128] (single sequence) ...
  float *const *states;   // ... or one pointer per sequence (device array), when non-null
  float *out;             // [(seq * tokens + t)][value_heads][128]
  std::uint32_t tokens;
  std::uint32_t sequences;
  std::uint32_t key_heads;
  std::uint32_t value_heads;
};
void launch_gdn_recurrent(const GdnCoreArgs &args, cudaStream_t stream);
// Chunk-64 WY-form prefill (single sequence); scratch sized by gdn_chunk_workspace_bytes.
std::size_t gdn_chunk_workspace_bytes(std::size_t tokens, std::size_t key_heads, std::size_t value_heads);
void launch_gdn_chunked(const GdnCoreArgs &args, void *workspace, cudaStream_t stream);

// Steps either side of the recurrence inside qwen35_gated_delta (cpp/kernels/qwen35_delta.cu:236-276,
// 375-411,579-621).
struct GdnLayerArgs {
  const void *input; // [tokens][q | k | v | b | a | z], dtype
  const void *conv_weight, *recurrent_a, *dt_bias, *output_norm_weight;
  void *output;      // [tokens][hidden], dtype
  float *convolution_state;
  float *convolved;  // [tokens][conv_dim] fp32: q (normalised, scaled), k (normalised), v
  float *beta;       // [tokens][value_heads]
  float *log_decay;  // [tokens][value_heads]
  const float *raw;  // [tokens][hidden] recurrence output
  std::uint32_t tokens, key_heads, value_heads, conv_width;
  float epsilon;
  int32_t dtype, weight_dtype;
};
void launch_gdn_prologue(const GdnLayerArgs &args, cudaStream_t stream);
void launch_gdn_epilogue(const GdnLayerArgs &args, cudaStream_t stream);

} // namespace rib200
