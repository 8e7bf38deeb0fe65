// Runs the two call sequences of RAFTInfer's executor on a GPU through the C++ drop-in headers alone
// (<raftinfer_b200/kernels.hpp>, <raftinfer_b200/primitives.hpp>), with plain cudaMalloc buffers, one stream and
// FP32 activations, the dtype the executor passes (cpp/execution/qwen35_executor.cu:697):
//
//   full-attention layer, cpp/execution/qwen35_executor.cu:1989-2055
//       qwen35_split_full_query_gate -> qwen35_qk_norm_rope (q) -> qwen35_qk_norm_rope (k) -> qwen35_causal_attention
//     for a chunk of tokens behind a past, then one decode step: the same three calls with a device position and
//     qwen35_online_attention_decode with a split-k plan (the executor's graph variant, :2191-2225);
//   linear layer, cpp/execution/qwen35_executor.cu:2118-2126
//       qwen35_gated_delta on a chunk, then on one token, same states.
//
// Inputs are read from <dir>/<name>.bin and outputs written there; tests/test_cpp_dropin.py makes the inputs and
// compares the outputs with the CPU oracle.  Usage: dropin_gpu_test <dir> <tokens> <past> <max_ctx> <delta_tokens>
#include <raftinfer_b200/kernels.hpp>
#include <raftinfer_b200/primitives.hpp>

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace rk = raftinfer::kernels;

namespace {

void cuda(cudaError_t err, const char *what) {
  if (err != cudaSuccess) {
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
  }
}

std::vector<unsigned char> read_file(const std::string &path, std::size_t expect_bytes) {
  std::ifstream in(path, std::ios::binary);
  if (!in) {
    throw std::runtime_error("cannot open " + path);
  }
  std::vector<unsigned char> data((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  if (data.size() != expect_bytes) {
    throw std::runtime_error(path + ": expected " + std::to_string(expect_bytes) + " bytes, found " +
                             std::to_string(data.size()));
  }
  return data;
}

// A device buffer that knows its size; optionally filled from a file, optionally written back to one.
struct Buffer {
  void *ptr = nullptr;
  std::size_t bytes = 0;
  explicit Buffer(std::size_t n) : bytes(n) {
    cuda(cudaMalloc(&ptr, n), "cudaMalloc");
    cuda(cudaMemset(ptr, 0, n), "cudaMemset");
  }
  Buffer(const std::string &path, std::size_t n) : Buffer(n) {
    const std::vector<unsigned char> host = read_file(path, n);
    cuda(cudaMemcpy(ptr, host.data(), n, cudaMemcpyHostToDevice), "upload");
  }
  Buffer(const Buffer &) = delete;
  Buffer &operator=(const Buffer &) = delete;
  ~Buffer() { cudaFree(ptr); }
  void dump(const std::string &path) const {
    std::vector<unsigned char> host(bytes);
    cuda(cudaMemcpy(host.data(), ptr, bytes, cudaMemcpyDeviceToHost), "download");
    std::ofstream out(path, std::ios::binary);
    out.write(reinterpret_cast<const char *>(host.data()), static_cast<std::streamsize>(bytes));
    if (!out) {
      throw std::runtime_error("cannot write " + path);
    }
  }
  template <class T> T *as() const { return static_cast<T *>(ptr); }
};

constexpr std::size_t kQueryHeads = 16, kKvHeads = 4, kHeadDim = 256, kRotary = 64;
constexpr float kRopeBase = 1.0e7F, kEpsilon = 1.0e-6F;
constexpr std::size_t kKeyHeads = 16, kValueHeads = 32, kDeltaDim = 128, kConvWidth = 4;

void full_attention_layer(const std::string &dir, std::size_t tokens, std::size_t past, std::size_t max_ctx,
                          cudaStream_t stream) {
  const auto f32 = RAFTINFER_DTYPE_F32;
  const std::size_t q_floats = kQueryHeads * kHeadDim, kv_floats = kKvHeads * kHeadDim;
  const rk::Qwen35AttentionLaunchPolicy policy{raftinfer::Qwen35AttentionImplementation::online_tiled,
                                               raftinfer::Qwen35KvCacheDType::bf16,
                                               raftinfer::Qwen35KvCacheLayout::head_major};
  rk::Qwen35AttentionShape shape{tokens, kQueryHeads, kKvHeads, kHeadDim, max_ctx, past};
  const std::size_t cache_bytes = rk::qwen35_attention_cache_bytes(shape, policy);
  if (!rk::qwen35_online_attention_prefill_supported(shape, f32, policy)) {
    throw std::runtime_error("the executor's prefill signature is reported as unsupported");
  }
  Buffer query_gate(dir + "/query_gate.bin", tokens * 2 * q_floats * 4);
  Buffer key(dir + "/key.bin", tokens * kv_floats * 4), value(dir + "/value.bin", tokens * kv_floats * 4);
  Buffer q_weight(dir + "/q_norm_weight.bin", kHeadDim * 4), k_weight(dir + "/k_norm_weight.bin", kHeadDim * 4);
  Buffer cache(dir + "/kv_cache.bin", cache_bytes);
  Buffer query(tokens * q_floats * 4), gate(tokens * q_floats * 4), query_normed(tokens * q_floats * 4);
  Buffer key_normed(tokens * kv_floats * 4), output(tokens * q_floats * 4);

  // prefill chunk: the executor's sequence, activations FP32, no workspace on the online path
  rk::qwen35_split_full_query_gate(query_gate.ptr, query.ptr, gate.ptr, tokens, kQueryHeads, kHeadDim, f32, stream);
  rk::qwen35_qk_norm_rope(query.ptr, q_weight.ptr, query_normed.ptr,
                          rk::QkNormRopeShape{tokens, kQueryHeads, kHeadDim, kRotary, past, kRopeBase}, kEpsilon, f32,
                          f32, stream);
  rk::qwen35_qk_norm_rope(key.ptr, k_weight.ptr, key_normed.ptr,
                          rk::QkNormRopeShape{tokens, kKvHeads, kHeadDim, kRotary, past, kRopeBase}, kEpsilon, f32, f32,
                          stream);
  rk::qwen35_causal_attention(query_normed.ptr, key_normed.ptr, value.ptr, gate.ptr, output.ptr, cache.ptr,
                              cache_bytes, nullptr, 0, shape, f32, policy, stream);

  // one decode step behind it: position on the device, split-k plan sized for the whole cache
  const std::uint32_t position = static_cast<std::uint32_t>(past + tokens);
  Buffer device_position(sizeof(std::uint32_t));
  cuda(cudaMemcpyAsync(device_position.ptr, &position, sizeof(position), cudaMemcpyHostToDevice, stream), "position");
  Buffer d_query_gate(dir + "/decode_query_gate.bin", 2 * q_floats * 4);
  Buffer d_key(dir + "/decode_key.bin", kv_floats * 4), d_value(dir + "/decode_value.bin", kv_floats * 4);
  Buffer d_query(q_floats * 4), d_gate(q_floats * 4), d_query_normed(q_floats * 4), d_key_normed(kv_floats * 4);
  Buffer d_output(q_floats * 4);
  rk::Qwen35AttentionShape one{1, kQueryHeads, kKvHeads, kHeadDim, max_ctx, 0};
  const rk::Qwen35OnlineDecodePlan plan =
      rk::qwen35_online_decode_plan(one, raftinfer::Qwen35DecodeAttentionMode::split_k_256, max_ctx);
  const rk::Qwen35OnlineDecodeWorkspaceLayout layout = rk::qwen35_online_decode_workspace_layout(one, plan.resolved_mode);
  Buffer workspace(layout.bytes);
  rk::qwen35_split_full_query_gate(d_query_gate.ptr, d_query.ptr, d_gate.ptr, 1, kQueryHeads, kHeadDim, f32, stream);
  rk::qwen35_qk_norm_rope(d_query.ptr, q_weight.ptr, d_query_normed.ptr,
                          rk::QkNormRopeShape{1, kQueryHeads, kHeadDim, kRotary, 0, kRopeBase}, kEpsilon, f32, f32,
                          stream, device_position.as<std::uint32_t>());
  rk::qwen35_qk_norm_rope(d_key.ptr, k_weight.ptr, d_key_normed.ptr,
                          rk::QkNormRopeShape{1, kKvHeads, kHeadDim, kRotary, 0, kRopeBase}, kEpsilon, f32, f32, stream,
                          device_position.as<std::uint32_t>());
  rk::qwen35_online_attention_decode(d_query_normed.ptr, d_key_normed.ptr, d_value.ptr, d_gate.ptr, d_output.ptr,
                                     cache.ptr, cache_bytes, workspace.ptr, layout.bytes, one, f32,
                                     raftinfer::Qwen35KvCacheDType::bf16, raftinfer::Qwen35KvCacheLayout::head_major,
                                     plan, device_position.as<std::uint32_t>(), stream);
  cuda(cudaStreamSynchronize(stream), "full-attention layer");
  output.dump(dir + "/attention_output.bin");
  d_output.dump(dir + "/decode_output.bin");
  cache.dump(dir + "/kv_cache_after.bin");
}

void linear_layer(const std::string &dir, std::size_t tokens, cudaStream_t stream) {
  const auto f32 = RAFTINFER_DTYPE_F32;
  const std::size_t hidden = kValueHeads * kDeltaDim;
  const std::size_t conv_dim = 2 * kKeyHeads * kDeltaDim + hidden;
  const std::size_t stride = conv_dim + 2 * kValueHeads + hidden;
  Buffer input(dir + "/delta_input.bin", (tokens + 1) * stride * 4);
  Buffer conv_weight(dir + "/conv_weight.bin", conv_dim * kConvWidth * 4);
  Buffer recurrent_a(dir + "/recurrent_a.bin", kValueHeads * 4), dt_bias(dir + "/dt_bias.bin", kValueHeads * 4);
  Buffer norm_weight(dir + "/output_norm_weight.bin", kDeltaDim * 4);
  Buffer conv_state(dir + "/conv_state.bin", conv_dim * (kConvWidth - 1) * 4);
  Buffer recurrent_state(dir + "/recurrent_state.bin", kValueHeads * kDeltaDim * kDeltaDim * 4);
  Buffer output((tokens + 1) * hidden * 4);
  const rk::GatedDeltaShape chunk{tokens, hidden, kKeyHeads, kValueHeads, kDeltaDim, kDeltaDim, kConvWidth, kEpsilon};
  const rk::GatedDeltaShape one{1, hidden, kKeyHeads, kValueHeads, kDeltaDim, kDeltaDim, kConvWidth, kEpsilon};
  // the executor sizes one workspace for its largest call and reuses it
  Buffer workspace(rk::qwen35_gated_delta_workspace_bytes(chunk));
  rk::qwen35_gated_delta(input.ptr, conv_weight.ptr, recurrent_a.ptr, dt_bias.ptr, norm_weight.ptr, output.ptr,
                         conv_state.as<float>(), recurrent_state.as<float>(), workspace.ptr, workspace.bytes, chunk,
                         rk::qwen35_gated_delta_select_policy(chunk, tokens), f32, f32, stream);
  rk::qwen35_gated_delta(input.as<float>() + tokens * stride, conv_weight.ptr, recurrent_a.ptr, dt_bias.ptr,
                         norm_weight.ptr, output.as<float>() + tokens * hidden, conv_state.as<float>(),
                         recurrent_state.as<float>(), workspace.ptr, workspace.bytes, one,
                         rk::qwen35_gated_delta_select_policy(one, 1), f32, f32, stream);
  cuda(cudaStreamSynchronize(stream), "linear layer");
  output.dump(dir + "/delta_output.bin");
  conv_state.dump(dir + "/conv_state_after.bin");
  recurrent_state.dump(dir + "/recurrent_state_after.bin");
}

} // namespace

int main(int argc, char **argv) {
  if (argc != 6) {
    std::fprintf(stderr, "usage: %s <dir> <tokens> <past> <max_ctx> <delta_tokens>\n", argv[0]);
    return 2;
  }
  try {
    const std::string dir = argv[1];
    const std::size_t tokens = std::strtoull(argv[2], nullptr, 10), past = std::strtoull(argv[3], nullptr, 10);
    const std::size_t max_ctx = std::strtoull(argv[4], nullptr, 10), delta_tokens = std::strtoull(argv[5], nullptr, 10);
    cudaStream_t stream = nullptr;
    cuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
    full_attention_layer(dir, tokens, past, max_ctx, stream);
    linear_layer(dir, delta_tokens, stream);
    std::uint32_t bits = 0;
    const Rib200Status status = rib200_device_status(stream, &bits);
    if (status.code != RIB200_STATUS_OK || bits != 0) {
      std::fprintf(stderr, "device status %u (%s)\n", bits, status.message);
      return 1;
    }
    cuda(cudaStreamDestroy(stream), "cudaStreamDestroy");
    std::printf("dropin gpu ok\n");
    return 0;
  } catch (const std::exception &error) {
    std::fprintf(stderr, "dropin gpu test failed: %s\n", error.what());
    return 1;
  }
}
