/* rib200 - B200 (sm_100a) attention and gated-delta kernels behind RAFTInfer's kernel-launcher API.
 *
 * C ABI of librib200.so.  Plain pointers and sizes only.  Every entry point returns a status
 * {code, message}; `message` points into a thread-local buffer that stays valid until the next
 * call on the same thread.  Enum values are RAFTInfer's own
 * (cpp/include/raftinfer/tensor.h:10-15, cpp/include/raftinfer/status.h:7-20,
 * cpp/execution/qwen35_execution_policy.hpp:7-27) so the reference's structs convert field by field.
 *
 * Ownership and threading follow the reference launchers (cpp/kernels/qwen35_delta.cuh:76-86):
 * the caller owns every buffer (inputs, outputs, KV cache, gated-delta states, workspace); a call
 * only enqueues work on `stream`, never allocates, never creates a stream and never synchronises.
 * `stream` must be a real stream handle (NULL is rejected, as in cpp/kernels/qwen35_attention.cu:430).
 * Calls are re-entrant across different streams and buffers.
 *
 * There is no CPU fallback and no second backend: a signature these kernels do not cover returns
 * RIB200_STATUS_UNSUPPORTED.
 */
#ifndef RIB200_H
#define RIB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cpp/include/raftinfer/status.h:7-20 */
enum {
  RIB200_STATUS_OK = 0,
  RIB200_STATUS_INVALID_ARGUMENT = 1,
  RIB200_STATUS_UNAVAILABLE = 2,
  RIB200_STATUS_CUDA_ERROR = 3,
  RIB200_STATUS_INTERNAL = 4,
  RIB200_STATUS_UNSUPPORTED = 5,
  RIB200_STATUS_RESOURCE_EXHAUSTED = 6
};

typedef struct Rib200Status {
  int32_t code;
  const char *message; /* "" when code == RIB200_STATUS_OK */
} Rib200Status;

/* cpp/include/raftinfer/tensor.h:10-15 */
enum { RIB200_DTYPE_F32 = 1, RIB200_DTYPE_F16 = 2, RIB200_DTYPE_BF16 = 3 };
/* cpp/execution/qwen35_execution_policy.hpp:7-27 */
enum { RIB200_ATTENTION_MATERIALIZED_REFERENCE = 0, RIB200_ATTENTION_ONLINE_TILED = 1 };
enum { RIB200_DECODE_AUTO_SELECT = 0, RIB200_DECODE_SINGLE_BLOCK = 1, RIB200_DECODE_SPLIT_K_256 = 2,
       RIB200_DECODE_SPLIT_K_512 = 3 };
enum { RIB200_KV_CACHE_F32 = 0, RIB200_KV_CACHE_BF16 = 1 };
enum { RIB200_KV_LAYOUT_TOKEN_MAJOR = 0, RIB200_KV_LAYOUT_HEAD_MAJOR = 1 };
/* cpp/kernels/qwen35_delta.cuh:31-35 */
enum { RIB200_DELTA_SCHEDULE_CURRENT = 0, RIB200_DELTA_SCHEDULE_PREFILL_SM120 = 1,
       RIB200_DELTA_SCHEDULE_DECODE_SM120 = 2 };

/* Bits of the device status word (rib200_device_status).  They replace the device-side trap of
 * cpp/kernels/qwen35_online_attention.cu:714-717: the kernel records the condition and returns. */
enum {
  RIB200_DEVICE_DECODE_CAPACITY_EXCEEDED = 1u << 0, /* live context needs more partitions than the plan holds */
  RIB200_DEVICE_POSITION_OUT_OF_RANGE = 1u << 1,    /* *device_position >= max_context_tokens */
  RIB200_DEVICE_WAIT_TIMED_OUT = 1u << 2,           /* a bounded on-device wait gave up */
  RIB200_DEVICE_PAGE_OUT_OF_RANGE = 1u << 3,        /* a block table names a page the pool does not hold */
  RIB200_DEVICE_POINTER_MISALIGNED = 1u << 4        /* a pointer read on the device is off its required boundary */
};

/* cpp/kernels/qwen35_attention.cuh:14-21 */
typedef struct Rib200AttentionShape {
  size_t tokens;
  size_t query_heads;
  size_t kv_heads;
  size_t head_dim;
  size_t max_context_tokens;
  size_t past_tokens;
} Rib200AttentionShape;

/* cpp/kernels/qwen35_attention.cuh:23-27 */
typedef struct Rib200AttentionLaunchPolicy {
  uint8_t implementation;
  uint8_t kv_cache_dtype;
  uint8_t kv_cache_layout;
} Rib200AttentionLaunchPolicy;

/* QkNormRopeShape, cpp/kernels/qwen35_primitives.cuh:32-39 */
typedef struct Rib200QkNormRopeShape {
  size_t tokens;
  size_t heads;
  size_t head_dim;
  size_t rotary_dim;
  size_t position_offset;
  float rope_base;
} Rib200QkNormRopeShape;

/* cpp/kernels/qwen35_online_attention.cuh:12-21 */
typedef struct Rib200OnlineDecodePlan {
  uint8_t resolved_mode;
  size_t partition_tokens;
  size_t split_k_threshold_tokens;
  size_t context_bucket_tokens;
  size_t active_partition_capacity;
} Rib200OnlineDecodePlan;

/* cpp/kernels/qwen35_online_attention.cuh:23-31 */
typedef struct Rib200OnlineDecodeWorkspaceLayout {
  size_t partial_count;
  size_t max_offset_bytes;
  size_t sum_offset_bytes;
  size_t value_offset_bytes;
  size_t bytes;
} Rib200OnlineDecodeWorkspaceLayout;

/* cpp/kernels/qwen35_delta.cuh:20-29 */
typedef struct Rib200GatedDeltaShape {
  size_t tokens;
  size_t hidden_size;
  size_t key_heads;
  size_t value_heads;
  size_t key_dim;
  size_t value_dim;
  size_t conv_width;
  float epsilon;
} Rib200GatedDeltaShape;

/* cpp/kernels/qwen35_delta.cuh:37-41 */
typedef struct Rib200GatedDeltaLaunchPolicy {
  uint8_t schedule;
  uint32_t warps_per_block;
  uint8_t transposed_boundary_state;
} Rib200GatedDeltaLaunchPolicy;

/* cpp/kernels/qwen35_delta.cuh:43-60 (rejection_reason as a fixed buffer) */
typedef struct Rib200GatedDeltaScheduleDiagnostic {
  size_t bucket_tokens;
  size_t key_dim;
  size_t value_dim;
  uint8_t candidate_schedule;
  uint8_t schedule;
  uint32_t warps_per_block;
  uint8_t transposed_boundary_state;
  uint8_t candidate_accepted;
  uint8_t correctness_passed;
  float current_median_ms;
  float candidate_median_ms;
  char rejection_reason[32];
} Rib200GatedDeltaScheduleDiagnostic;

/* ---- sizes and plans (host only; no CUDA call) ------------------------------------------- */

/* qwen35_attention_workspace_floats, cpp/kernels/qwen35_attention.cuh:29 (cpp/kernels/qwen35_attention.cu).
 * Size of the logits buffer of the reference's materialized path: tokens * query_heads * context floats. */
Rib200Status rib200_attention_workspace_floats(const Rib200AttentionShape *shape, size_t *floats);
/* qwen35_attention_cache_bytes, cpp/kernels/qwen35_attention.cuh:31-32 (cpp/kernels/qwen35_attention.cu:417-428). */
Rib200Status rib200_attention_cache_bytes(const Rib200AttentionShape *shape, Rib200AttentionLaunchPolicy policy,
                                          size_t *bytes);
/* qwen35_attention_workspace_bytes (policy overload), cpp/kernels/qwen35_attention.cuh:33-35
 * (cpp/kernels/qwen35_attention.cu:430-443). */
Rib200Status rib200_attention_workspace_bytes(const Rib200AttentionShape *shape, Rib200AttentionLaunchPolicy policy,
                                              size_t *bytes);
/* qwen35_online_decode_plan, cpp/kernels/qwen35_online_attention.cuh:33-35
 * (cpp/kernels/qwen35_online_attention.cu:1071-1109). */
Rib200Status rib200_online_decode_plan(const Rib200AttentionShape *shape, uint8_t requested_mode,
                                       size_t context_tokens, Rib200OnlineDecodePlan *plan);
/* qwen35_online_decode_workspace_layout, cpp/kernels/qwen35_online_attention.cuh:37-38
 * (cpp/kernels/qwen35_online_attention.cu:1111-1143). */
Rib200Status rib200_online_decode_workspace_layout(const Rib200AttentionShape *shape, uint8_t resolved_mode,
                                                   Rib200OnlineDecodeWorkspaceLayout *layout);
/* qwen35_online_attention_prefill_supported, cpp/kernels/qwen35_online_attention.cuh:40-42.
 * Writes 1 when rib200_online_attention_prefill accepts the signature, else 0; never fails. */
Rib200Status rib200_online_attention_prefill_supported(const Rib200AttentionShape *shape, int32_t activation_dtype,
                                                       Rib200AttentionLaunchPolicy policy, int32_t *supported);
/* qwen35_online_attention_workspace_bytes, cpp/kernels/qwen35_online_attention.cuh:44-45 (always 0). */
Rib200Status rib200_online_attention_workspace_bytes(const Rib200AttentionShape *shape, size_t *bytes);
/* qwen35_gated_delta_workspace_bytes, cpp/kernels/qwen35_delta.cuh:65 (cpp/kernels/qwen35_delta.cu:755-757). */
Rib200Status rib200_gated_delta_workspace_bytes(const Rib200GatedDeltaShape *shape, size_t *bytes);
/* qwen35_gated_delta_select_policy, cpp/kernels/qwen35_delta.cuh:70-72. */
Rib200Status rib200_gated_delta_select_policy(const Rib200GatedDeltaShape *shape, size_t bucket_tokens,
                                              Rib200GatedDeltaLaunchPolicy *policy);
/* qwen35_gated_delta_schedule_diagnostic, cpp/kernels/qwen35_delta.cuh:74-76. */
Rib200Status rib200_gated_delta_schedule_diagnostic(const Rib200GatedDeltaShape *shape, size_t bucket_tokens,
                                                    Rib200GatedDeltaScheduleDiagnostic *diagnostic);

/* ---- launchers ---------------------------------------------------------------------------- */

/* qwen35_causal_attention (policy overload), cpp/kernels/qwen35_attention.cuh:37-44
 * (cpp/kernels/qwen35_attention.cu:565-613).  tokens == 1 runs single-block decode, tokens > 1 the
 * online prefill; a workspace is forbidden on the online path. */
Rib200Status rib200_causal_attention(const void *query, const void *key, const void *value, const void *gate,
                                     void *output, void *kv_cache, size_t kv_cache_bytes, void *workspace,
                                     size_t workspace_bytes, const Rib200AttentionShape *shape,
                                     int32_t activation_dtype, Rib200AttentionLaunchPolicy policy, void *stream);

/* qwen35_online_attention_prefill, cpp/kernels/qwen35_online_attention.cuh:47-53
 * (cpp/kernels/qwen35_online_attention.cu:1161-1218).  Appends this chunk's K,V to the cache at
 * past_tokens.. and writes out[t][h] = softmax_{j <= past+t}(q.k_j / sqrt(D)) . v * sigmoid(gate).
 * query, gate, output are [tokens][query_heads][head_dim]; key, value [tokens][kv_heads][head_dim]. */
Rib200Status rib200_online_attention_prefill(const void *query, const void *key, const void *value,
                                             const void *gate, void *output, void *kv_cache, size_t kv_cache_bytes,
                                             const Rib200AttentionShape *shape, int32_t activation_dtype,
                                             uint8_t cache_dtype, uint8_t cache_layout, void *stream);

/* qwen35_online_attention_decode (plan overload), cpp/kernels/qwen35_online_attention.cuh:55-63
 * (cpp/kernels/qwen35_online_attention.cu:1220-1314).  One token: append K,V at the position
 * (*device_position when non-NULL, else shape->past_tokens), then attend over 0..position.
 * With a split-k plan the partials (max, sum, acc) land in `workspace` in the layout of
 * rib200_online_decode_workspace_layout.  Safe to capture in a CUDA graph: the position is read
 * on the device and the grid is sized by plan->active_partition_capacity. */
Rib200Status rib200_online_attention_decode(const void *query, const void *key, const void *value,
                                            const void *gate, void *output, void *kv_cache, size_t kv_cache_bytes,
                                            void *workspace, size_t workspace_bytes,
                                            const Rib200AttentionShape *shape, int32_t activation_dtype,
                                            uint8_t cache_dtype, uint8_t cache_layout,
                                            const Rib200OnlineDecodePlan *plan, const uint32_t *device_position,
                                            void *stream);

/* qwen35_gated_delta (policy overload), cpp/kernels/qwen35_delta.cuh:95-102
 * (cpp/kernels/qwen35_delta.cu:811-897).  Packed input per token [q | k | v | b | a | z]. */
Rib200Status rib200_gated_delta(const void *input, const void *conv_weight, const void *recurrent_a,
                                const void *dt_bias, const void *output_norm_weight, void *output,
                                float *convolution_state, float *recurrent_state, void *workspace,
                                size_t workspace_bytes, const Rib200GatedDeltaShape *shape,
                                Rib200GatedDeltaLaunchPolicy policy, int32_t dtype, int32_t weight_dtype,
                                void *stream);

/* ---- additive entry points (no counterpart in the reference) ------------------------------ */

/* Gated delta-rule recurrence alone (the loop body of cpp/kernels/qwen35_delta.cu:482-576 /
 * cpp/reference/qwen35.cpp:459-518) on operands that are already convolved and normalised:
 * q, k [tokens][key_heads][key_dim] (q carries 1/sqrt(key_dim)), v [tokens][value_heads][value_dim], all of
 * qkv_dtype (RIB200_DTYPE_BF16 or RIB200_DTYPE_F32); beta and log_decay FP32 [tokens][value_heads]
 * (beta in (0,1), decay = exp(log_decay)); state FP32 [value_heads][key_dim][value_dim] updated in place;
 * out FP32 [tokens][value_heads][value_dim] (the vector before the output norm).  The key head of value
 * head h is h % key_heads.  tokens < 64 run the recurrent kernel (one pass over the state per token);
 * longer runs use the chunk-64 WY-form prefill and need rib200_gdn_core_workspace_bytes of scratch.
 * key_dim == value_dim == 128 only. */
Rib200Status rib200_gdn_core_workspace_bytes(size_t tokens, size_t key_heads, size_t value_heads, size_t key_dim,
                                             size_t value_dim, size_t *bytes);
Rib200Status rib200_gdn_core(const void *q, const void *k, const void *v, const float *beta,
                             const float *log_decay, float *state, float *out, void *workspace,
                             size_t workspace_bytes, size_t tokens, size_t key_heads, size_t value_heads,
                             size_t key_dim, size_t value_dim, int32_t qkv_dtype, void *stream);

/* One decode step for a batch of independent sequences (ragged contexts), one launch per stage.
 * Per sequence i: kv_caches[i] is its BF16 head-major cache of max_context_tokens[i] rows, positions[i]
 * the row the new token is appended at; query/gate/output are [batch][16][256], key/value [batch][4][256]
 * (BF16).  Arrays of pointers and sizes live in device memory.  workspace holds the split-k partials of
 * every sequence back to back; rib200_batched_decode_workspace_bytes sizes it for the largest context. */
Rib200Status rib200_batched_decode_workspace_bytes(size_t batch, size_t max_context_tokens, size_t *bytes);
Rib200Status rib200_batched_decode_attention(const void *query, const void *key, const void *value,
                                             const void *gate, void *output, void *const *kv_caches,
                                             const uint32_t *max_context_tokens, const uint32_t *positions,
                                             size_t batch, size_t largest_max_context_tokens, void *workspace,
                                             size_t workspace_bytes, void *stream);
/* Paged form of the batched decode step (no counterpart in the reference, which holds one contiguous cache per
 * sequence).  The KV rows live in a pool of pages of 256 tokens; a page is laid out like a head-major cache of 256
 * rows, [2][4][256][256] BF16 = 1 MiB, and block_tables[i][b] (device memory, rows of max_blocks_per_sequence
 * entries) names the page that holds rows [256 b, 256 b + 256) of sequence i.  positions[i] is the row the new
 * token is appended at; its page must be in the table already.  Entries past a sequence's live context are not
 * read.  An entry >= pool_pages sets RIB200_DEVICE_PAGE_OUT_OF_RANGE and leaves that sequence's output undefined;
 * positions[i] >= 256 * max_blocks_per_sequence sets RIB200_DEVICE_POSITION_OUT_OF_RANGE.  The workspace is that of
 * rib200_batched_decode_workspace_bytes(batch, 256 * max_blocks_per_sequence). */
Rib200Status rib200_paged_decode_attention(const void *query, const void *key, const void *value, const void *gate,
                                           void *output, void *page_pool, size_t pool_pages,
                                           const uint32_t *block_tables, size_t max_blocks_per_sequence,
                                           const uint32_t *positions, size_t batch, void *workspace,
                                           size_t workspace_bytes, void *stream);
/* Recurrent gated-delta decode step for a batch of sequences: states[i] FP32 [value_heads][128][128], 16-byte
 * aligned (array of device pointers, itself in device memory); q,k BF16 [batch][key_heads][128], v BF16
 * [batch][value_heads][128], beta/log_decay FP32 [batch][value_heads], out FP32 [batch][value_heads][128].
 * A states[i] off a 16-byte boundary sets RIB200_DEVICE_POINTER_MISALIGNED; the states and outputs of that call are
 * then undefined. */
Rib200Status rib200_batched_gdn_decode(const void *q, const void *k, const void *v, const float *beta,
                                       const float *log_decay, float *const *states, float *out, size_t batch,
                                       size_t key_heads, size_t value_heads, void *stream);

/* No counterpart in the reference.  The same split-k decode step as rib200_online_attention_decode (partition
 * size 256, grid sized for the whole cache so one launch shape serves every position), for hosts that may
 * not allocate device memory on the decode path and have no workspace to hand over: a runtime that gave all
 * of its device memory to a pool at start-up and treats any later allocation as a bug (RAFTInfer's executor
 * asserts zero allocations after construction, cpp/tests/qwen35_executor_test.cu:1426-1441), a plugin that is
 * only given the tensors of the operator it replaces, or a latency-critical serving thread for which the
 * implicit device synchronisation of cudaMalloc is not acceptable.  The partials go to an array built into the
 * library (2 113 536 bytes of device memory per GPU that loads it, held until the process exits), so:
 *   - shape->max_context_tokens may be at most 32768; larger caches are refused with
 *     RIB200_STATUS_INVALID_ARGUMENT (use the workspace entry point for those);
 *   - the call allocates nothing and frees nothing;
 *   - the first call on each device looks up the array's device address; make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array, which keeps whatever the previous call left in it.  Nothing
 *     in it needs clearing (every partial that is read was written by the same call), but two calls whose
 *     kernels overlap on the GPU (different streams, or graphs launched concurrently) race on it: serialise
 *     them.
 * Other arguments as rib200_online_attention_decode; the cache must be BF16 head-major. */
Rib200Status rib200_online_attention_decode_static_scratch(const void *query, const void *key, const void *value,
                                                           const void *gate, void *output, void *kv_cache,
                                                           size_t kv_cache_bytes, const Rib200AttentionShape *shape,
                                                           int32_t activation_dtype, const uint32_t *device_position,
                                                           void *stream);

/* ---- the step in front of the attention kernels ----------------------------------------------------
 * qwen35_qk_norm_rope, cpp/kernels/qwen35_primitives.cuh:61-66 (cpp/kernels/qwen35_primitives.cu:574-626):
 * per head vector RMSNorm (mean square + epsilon) times weight[head_dim], then NeoX-style RoPE on the first
 * rotary_dim dims, pairs (i, i + rotary_dim / 2), angle (position_offset or *device_position, plus the token
 * index) / rope_base^(2 i / rotary_dim).  input, output [tokens][heads][head_dim] in `dtype`.
 * head_dim 128 or 256; FP32 or BF16 weights. */
Rib200Status rib200_qk_norm_rope(const void *input, const void *weight, void *output,
                                 const Rib200QkNormRopeShape *shape, float epsilon, int32_t dtype,
                                 int32_t weight_dtype, void *stream, const uint32_t *device_position);
/* qwen35_split_full_query_gate, cpp/kernels/qwen35_primitives.cuh:90-93
 * (cpp/kernels/qwen35_primitives.cu:743-766): query_gate [tokens][heads][2 * head_dim] -> query, gate
 * [tokens][heads][head_dim]. */
Rib200Status rib200_split_full_query_gate(const void *query_gate, void *query, void *gate, size_t tokens,
                                          size_t heads, size_t head_dim, int32_t dtype, void *stream);
/* The three calls the executor makes in front of attention (cpp/execution/qwen35_executor.cu:1989-2015:
 * split_full_query_gate, qk_norm_rope on q, qk_norm_rope on k) as one launch, which also casts v: reads
 * query_gate [tokens][query_heads][2 * head_dim], key and value [tokens][kv_heads][head_dim] in `dtype`
 * once and writes query, gate, key_out, value_out in output_dtype (BF16, or `dtype`), ready for
 * rib200_online_attention_prefill / _decode.  Positions start at shape->past_tokens or *device_position.
 * No counterpart in the reference as a single entry point. */
Rib200Status rib200_attention_prologue(const void *query_gate, const void *key, const void *value,
                                       const void *query_norm_weight, const void *key_norm_weight, void *query,
                                       void *gate, void *key_out, void *value_out,
                                       const Rib200AttentionShape *shape, size_t rotary_dim, float rope_base,
                                       float epsilon, int32_t dtype, int32_t weight_dtype, int32_t output_dtype,
                                       const uint32_t *device_position, void *stream);

/* ---- head-sharded prefill across the GPUs of one box (no counterpart in the reference) --------------
 * Each rank runs the prefill kernel on its own slice of the heads (its own query/key/value/gate and its
 * own KV cache holding its KV heads) and the kernel's epilogue stores every output tile straight into
 * the full-width output buffer of every rank - peer stores over NVLink, no separate all-gather.
 * outputs[r] (host array, `world` device pointers valid on this device) is rank r's buffer
 * [tokens][total_query_heads][head_dim] in the activation dtype, outputs[rank] this rank's own; this
 * rank's shape->query_heads heads land at head index head_offset.  world <= 8. */
Rib200Status rib200_online_attention_prefill_scatter(const void *query, const void *key, const void *value,
                                                     const void *gate, void *const *outputs, size_t world,
                                                     size_t rank, size_t total_query_heads, size_t head_offset,
                                                     void *kv_cache,
                                                     size_t kv_cache_bytes, const Rib200AttentionShape *shape,
                                                     int32_t activation_dtype, uint8_t cache_dtype,
                                                     uint8_t cache_layout, void *stream);
/* Rendezvous of the ranks after such a step, on the device: stores `epoch` into slot `rank` of every
 * rank's flag array (flags[r], host array of `world` device pointers to uint32[world], zero at start),
 * then waits, for a bounded time, until every slot of this rank's own array holds at least `epoch`.
 * Enqueued behind the prefill on `stream`: when it completes, every peer's tiles are in this rank's
 * buffer.  epoch must grow from call to call.  A wait that runs out sets RIB200_DEVICE_WAIT_TIMED_OUT. */
Rib200Status rib200_peer_rendezvous(uint32_t *const *flags, size_t world, size_t rank, uint32_t epoch,
                                    void *stream);
/* The same rendezvous with the caller's bound on the wait, in SM clock cycles (rib200_peer_rendezvous waits for
 * 2^31, about a second).  For callers that would rather learn of a missing peer after milliseconds, and for the
 * test that makes the wait run out: the kernel then sets RIB200_DEVICE_WAIT_TIMED_OUT and returns, and the CUDA
 * context stays usable.
 * The rendezvous only says that the peers' tiles of THIS step have arrived.  A peer that has passed it may start
 * its next step and store into this rank's buffer while this rank's readers of the current step are still
 * running, so a buffer may be rewritten only after every rank has consumed it: put a second rendezvous (a new
 * epoch) behind the consumers, or alternate between two buffers. */
Rib200Status rib200_peer_rendezvous_bounded(uint32_t *const *flags, size_t world, size_t rank, uint32_t epoch,
                                            uint64_t limit_cycles, void *stream);
/* Device memory that other processes on the box can map: allocation (zero-filled) with its 64-byte
 * handle, mapping of a peer's handle, and their releases. */
Rib200Status rib200_shared_alloc(size_t bytes, void **pointer, uint8_t handle[64]);
Rib200Status rib200_shared_open(const uint8_t handle[64], void **pointer);
Rib200Status rib200_shared_close(void *pointer);
Rib200Status rib200_shared_free(void *pointer);

/* One decode step driven from host memory (no counterpart in the reference, whose callers hold device
 * buffers): copies the token's rows q | k | v | gate ([16+4+4+16][256] in the activation dtype, back to back,
 * ideally pinned) into device_token (same size), runs rib200_online_attention_decode with them and returns once
 * the [16][256] output is in host_output (it synchronises `stream`).  When host_output is page-locked memory the
 * device can address, the kernel writes it there itself and device_output is left untouched; otherwise the output
 * goes to device_output and is copied.  The other arguments are those of rib200_online_attention_decode. */
Rib200Status rib200_online_attention_decode_from_host(const void *host_token, void *host_output, void *device_token,
                                                      void *device_output, void *kv_cache, size_t kv_cache_bytes,
                                                      void *workspace, size_t workspace_bytes,
                                                      const Rib200AttentionShape *shape, int32_t activation_dtype,
                                                      uint8_t cache_dtype, uint8_t cache_layout,
                                                      const Rib200OnlineDecodePlan *plan,
                                                      const uint32_t *device_position, void *stream);

/* rib200_online_attention_decode with the early cache fetch (no counterpart in the reference); host position
 * only.  A decode step reads cache rows [0, past_tokens) that earlier calls wrote and four token rows the kernel
 * in front of it produced.  Through this entry point the kernel starts fetching the cache rows as soon as it is
 * resident -- under programmatic dependent launch that can be while the kernel in front of it is still running --
 * and waits for that kernel only before it touches the token's rows, before it writes anything and before it lets
 * the kernel behind it become resident.  The caller promises in return that whatever wrote rows [0, past_tokens)
 * of that KV cache has completed, or is separated from this step by at least one ordinary kernel launch on the
 * stream (a kernel that does not release its dependents early; the decode kernels of this library do release them
 * early).  True for the reference's executor, where the previous writer of a layer's cache is the previous
 * token's step, a whole model pass earlier; false for two steps enqueued directly one after the other on the same
 * cache with advancing positions.  The choice is per call: nothing is remembered between calls. */
Rib200Status rib200_online_attention_decode_early_kv_fetch(const void *query, const void *key, const void *value,
                                                           const void *gate, void *output, void *kv_cache,
                                                           size_t kv_cache_bytes, void *workspace,
                                                           size_t workspace_bytes, const Rib200AttentionShape *shape,
                                                           int32_t activation_dtype, uint8_t cache_dtype,
                                                           uint8_t cache_layout, const Rib200OnlineDecodePlan *plan,
                                                           void *stream);

/* Reads and clears the status word the kernels of this library set on the current device.  It
 * synchronises `stream` first, so it is not for use inside a graph capture. */
Rib200Status rib200_device_status(void *stream, uint32_t *bits);

/* "rib200 <version> sm_100a" */
const char *rib200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RIB200_H */
