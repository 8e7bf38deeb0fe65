// TEST INFRASTRUCTURE ONLY.  CPU restatement of the RAFTInfer CPU reference
// operators for the attention + gated-delta hot path.  Nothing in the shipped
// library links, loads or calls this file; only the test-suite, the smoke
// check and the benchmark's cpu-baseline leg may use it, and only as the
// checker.
//
// Parity pin: every function here is checked (tests/test_oracle_pins.py)
//   * against the reference's literal known-answer vectors
//     (cpp/tests/qwen35_reference_test.cpp:59-156),
//   * against the Hugging Face golden layer fixture the reference ships
//     (tests/fixtures/qwen35/tiny-layer-v1.bin, read by
//     cpp/tests/qwen35_fixture_test.cpp:105-161), and
//   * against the reference's own cpp/reference library compiled unmodified
//     into oracle/_ref (when that library was built).
//
// Each routine names the reference lines it restates.  Accumulation types are
// kept identical to the reference (double dot products, float probabilities,
// float value accumulation) so that the restatement agrees with the reference
// to rounding, not merely to tolerance.
//
// The "core" entry points take already normalised / rotated operands and a
// KV cache, which the fused reference layer cannot do: the reference has no
// decode entry, so a 32K-token decode would cost a full O(L^2) prefill there.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

// cpp/reference/bf16.hpp:12-32 (round to nearest even, NaN kept NaN).
inline float bf16_bits_to_float(std::uint16_t bits) {
  std::uint32_t wide = static_cast<std::uint32_t>(bits) << 16U;
  float out;
  std::memcpy(&out, &wide, sizeof(out));
  return out;
}

inline std::uint16_t float_to_bf16_bits(float value) {
  std::uint32_t bits;
  std::memcpy(&bits, &value, sizeof(bits));
  if ((bits & 0x7F800000U) == 0x7F800000U) {
    const std::uint16_t top =
        static_cast<std::uint16_t>((bits >> 16U) & 0xFF80U);
    if ((bits & 0x007FFFFFU) == 0) {
      return top;
    }
    std::uint16_t payload = static_cast<std::uint16_t>((bits >> 16U) & 0x7FU);
    if (payload == 0) {
      payload = 1;
    }
    return static_cast<std::uint16_t>(top | payload);
  }
  const std::uint32_t lsb = (bits >> 16U) & 1U;
  return static_cast<std::uint16_t>((bits + 0x7FFFU + lsb) >> 16U);
}

// cpp/reference/qwen35.cpp:35-47.
inline float sigmoid_f(float v) { return 1.0F / (1.0F + std::exp(-v)); }
inline float silu_f(float v) { return v / (1.0F + std::exp(-v)); }
inline float softplus_f(float v) {
  if (v > 20.0F) {
    return v;
  }
  if (v < -20.0F) {
    return std::exp(v);
  }
  return std::log1p(std::exp(v));
}

// cpp/reference/qwen35.cpp:125-155 with weight_base = 0.
void rms_norm_rows(const float *in, const float *weight, float *out,
                   std::size_t rows, std::size_t cols, float eps) {
  for (std::size_t r = 0; r < rows; ++r) {
    double sq = 0.0;
    for (std::size_t c = 0; c < cols; ++c) {
      const double v = in[r * cols + c];
      sq += v * v;
    }
    const float scale =
        1.0F /
        std::sqrt(static_cast<float>(sq / static_cast<double>(cols)) + eps);
    for (std::size_t c = 0; c < cols; ++c) {
      out[r * cols + c] = in[r * cols + c] * scale * (0.0F + weight[c]);
    }
  }
}

// cpp/reference/qwen35.cpp:157-167.
void l2_normalize(float *v, std::size_t n, float eps) {
  double sq = 0.0;
  for (std::size_t i = 0; i < n; ++i) {
    sq += static_cast<double>(v[i]) * static_cast<double>(v[i]);
  }
  const float scale = 1.0F / std::sqrt(static_cast<float>(sq) + eps);
  for (std::size_t i = 0; i < n; ++i) {
    v[i] *= scale;
  }
}

// cpp/reference/qwen35.cpp:169-186 (NeoX pairing: (i, i + rotary/2)).
void partial_rope(float *v, std::size_t rotary, std::size_t pos, float base) {
  const std::size_t pairs = rotary / 2;
  for (std::size_t p = 0; p < pairs; ++p) {
    const double expo =
        static_cast<double>(2 * p) / static_cast<double>(rotary);
    const double theta = static_cast<double>(pos) / std::pow(base, expo);
    const float c = static_cast<float>(std::cos(theta));
    const float s = static_cast<float>(std::sin(theta));
    const float x0 = v[p];
    const float x1 = v[p + pairs];
    v[p] = x0 * c - x1 * s;
    v[p + pairs] = x0 * s + x1 * c;
  }
}

template <class Fn> void parallel_for(std::size_t n, int threads, Fn fn) {
  if (threads <= 1 || n <= 1) {
    for (std::size_t i = 0; i < n; ++i) {
      fn(i);
    }
    return;
  }
  std::atomic<std::size_t> next{0};
  std::vector<std::thread> pool;
  const int count = static_cast<int>(std::min<std::size_t>(threads, n));
  pool.reserve(count);
  for (int t = 0; t < count; ++t) {
    pool.emplace_back([&] {
      for (;;) {
        const std::size_t i = next.fetch_add(1);
        if (i >= n) {
          return;
        }
        fn(i);
      }
    });
  }
  for (auto &th : pool) {
    th.join();
  }
}

// KV accessor over either a dense float [ctx][Hkv][D] array or the BF16
// head-major cache [plane K|V][Hkv][max_ctx][D] of
// cpp/kernels/qwen35_online_attention.cu:240-252,316.
struct KvView {
  const float *k_f32{};
  const float *v_f32{};
  const std::uint16_t *cache_bf16{};
  std::size_t kv_heads{};
  std::size_t head_dim{};
  std::size_t max_ctx{};

  float k(std::size_t tok, std::size_t head, std::size_t dim) const {
    if (cache_bf16 != nullptr) {
      return bf16_bits_to_float(
          cache_bf16[(head * max_ctx + tok) * head_dim + dim]);
    }
    return k_f32[(tok * kv_heads + head) * head_dim + dim];
  }
  float v(std::size_t tok, std::size_t head, std::size_t dim) const {
    if (cache_bf16 != nullptr) {
      const std::size_t plane = max_ctx * kv_heads * head_dim;
      return bf16_bits_to_float(
          cache_bf16[plane + (head * max_ctx + tok) * head_dim + dim]);
    }
    return v_f32[(tok * kv_heads + head) * head_dim + dim];
  }
};

// One (query row, query head) of cpp/reference/qwen35.cpp:316-364:
// double dot, logit = float(dot / sqrt(double(D))), float running max,
// double shifted exp stored as float, double sum of the float
// probabilities, float(p / sum), float accumulation of p * v in key order.
void attention_row_head(const float *q_row, const KvView &kv,
                        std::size_t kv_head, std::size_t visible,
                        float *head_out, std::vector<float> &logits,
                        std::vector<float> &probs) {
  const std::size_t d = kv.head_dim;
  logits.resize(visible);
  probs.resize(visible);
  float max_logit = -std::numeric_limits<float>::infinity();
  const double root = std::sqrt(static_cast<double>(d));
  for (std::size_t j = 0; j < visible; ++j) {
    double dot = 0.0;
    for (std::size_t c = 0; c < d; ++c) {
      dot += static_cast<double>(q_row[c]) *
             static_cast<double>(kv.k(j, kv_head, c));
    }
    const float logit = static_cast<float>(dot / root);
    logits[j] = logit;
    max_logit = std::max(max_logit, logit);
  }
  double sum = 0.0;
  for (std::size_t j = 0; j < visible; ++j) {
    const double shifted =
        static_cast<double>(logits[j]) - static_cast<double>(max_logit);
    probs[j] = static_cast<float>(std::exp(shifted));
    sum += probs[j];
  }
  for (std::size_t j = 0; j < visible; ++j) {
    probs[j] = static_cast<float>(static_cast<double>(probs[j]) / sum);
  }
  for (std::size_t c = 0; c < d; ++c) {
    head_out[c] = 0.0F;
  }
  for (std::size_t j = 0; j < visible; ++j) {
    const float p = probs[j];
    for (std::size_t c = 0; c < d; ++c) {
      head_out[c] += p * kv.v(j, kv_head, c);
    }
  }
}

void attention_core(const float *q, const float *gate, float *out,
                    const KvView &kv, std::size_t tokens, std::size_t q_heads,
                    std::size_t past, int threads) {
  const std::size_t d = kv.head_dim;
  const std::size_t group = q_heads / kv.kv_heads;
  parallel_for(tokens * q_heads, threads, [&](std::size_t item) {
    const std::size_t t = item / q_heads;
    const std::size_t h = item % q_heads;
    std::vector<float> logits;
    std::vector<float> probs;
    const std::size_t base = (t * q_heads + h) * d;
    attention_row_head(q + base, kv, h / group, past + t + 1, out + base,
                       logits, probs);
    // cpp/reference/qwen35.cpp:366-370: gate applied after normalisation.
    for (std::size_t c = 0; c < d; ++c) {
      out[base + c] *= sigmoid_f(gate[base + c]);
    }
  });
}

} // namespace

extern "C" {

// cpp/reference/bf16.hpp:16-32.
void orc_round_to_bf16(const float *in, float *out, std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) {
    out[i] = bf16_bits_to_float(float_to_bf16_bits(in[i]));
  }
}

void orc_float_to_bf16_bits(const float *in, std::uint16_t *out,
                            std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) {
    out[i] = float_to_bf16_bits(in[i]);
  }
}

void orc_bf16_bits_to_float(const std::uint16_t *in, float *out,
                            std::size_t n) {
  for (std::size_t i = 0; i < n; ++i) {
    out[i] = bf16_bits_to_float(in[i]);
  }
}

// Attention core of cpp/reference/qwen35.cpp:316-370 over dense float K/V
// [past+tokens][Hkv][D].  q, gate, out are [tokens][Hq][D]; query row t sees
// keys 0 .. past+t.
void orc_attention_core_f32(const float *q, const float *k, const float *v,
                            const float *gate, float *out, std::size_t tokens,
                            std::size_t q_heads, std::size_t kv_heads,
                            std::size_t head_dim, std::size_t past,
                            int threads) {
  KvView kv;
  kv.k_f32 = k;
  kv.v_f32 = v;
  kv.kv_heads = kv_heads;
  kv.head_dim = head_dim;
  attention_core(q, gate, out, kv, tokens, q_heads, past, threads);
}

// Same arithmetic, keys and values read from the BF16 head-major cache
// (cpp/kernels/qwen35_online_attention.cu:240-252).  The cache must already
// hold rows 0 .. past+tokens-1.
void orc_attention_core_cache(const float *q, const float *gate, float *out,
                              const std::uint16_t *cache, std::size_t tokens,
                              std::size_t q_heads, std::size_t kv_heads,
                              std::size_t head_dim, std::size_t max_ctx,
                              std::size_t past, int threads) {
  KvView kv;
  kv.cache_bf16 = cache;
  kv.kv_heads = kv_heads;
  kv.head_dim = head_dim;
  kv.max_ctx = max_ctx;
  attention_core(q, gate, out, kv, tokens, q_heads, past, threads);
}

// Host recomputation of the split-k partial contract checked by
// cpp/tests/qwen35_cuda_attention_test.cu:883-957: for q head h and
// partition p over tokens [p*part, min(ctx, (p+1)*part)):
//   max = max_j s_j, sum = sum_j exp(s_j - max), acc = sum_j exp(s_j-max) v_j
// with s_j = (q . k_j) / sqrt(D).  Outputs are laid out as
// cpp/kernels/qwen35_online_attention.cu:1111-1143 (index h*max_parts + p).
void orc_decode_partials(const float *q, const std::uint16_t *cache,
                         float *part_max, float *part_sum, float *part_val,
                         std::size_t q_heads, std::size_t kv_heads,
                         std::size_t head_dim, std::size_t max_ctx,
                         std::size_t ctx, std::size_t part_tokens,
                         int threads) {
  KvView kv;
  kv.cache_bf16 = cache;
  kv.kv_heads = kv_heads;
  kv.head_dim = head_dim;
  kv.max_ctx = max_ctx;
  const std::size_t max_parts = (max_ctx + part_tokens - 1) / part_tokens;
  const std::size_t parts = (ctx + part_tokens - 1) / part_tokens;
  const std::size_t group = q_heads / kv_heads;
  const double root = std::sqrt(static_cast<double>(head_dim));
  parallel_for(q_heads * parts, threads, [&](std::size_t item) {
    const std::size_t h = item / parts;
    const std::size_t p = item % parts;
    const std::size_t begin = p * part_tokens;
    const std::size_t end = std::min(ctx, begin + part_tokens);
    std::vector<double> s(end - begin);
    double mx = -std::numeric_limits<double>::infinity();
    for (std::size_t j = begin; j < end; ++j) {
      double dot = 0.0;
      for (std::size_t c = 0; c < head_dim; ++c) {
        dot += static_cast<double>(q[h * head_dim + c]) *
               static_cast<double>(kv.k(j, h / group, c));
      }
      s[j - begin] = static_cast<double>(static_cast<float>(dot / root));
      mx = std::max(mx, s[j - begin]);
    }
    std::vector<double> acc(head_dim, 0.0);
    double sum = 0.0;
    for (std::size_t j = begin; j < end; ++j) {
      const double w = std::exp(s[j - begin] - mx);
      sum += w;
      for (std::size_t c = 0; c < head_dim; ++c) {
        acc[c] += w * static_cast<double>(kv.v(j, h / group, c));
      }
    }
    const std::size_t idx = h * max_parts + p;
    part_max[idx] = static_cast<float>(mx);
    part_sum[idx] = static_cast<float>(sum);
    for (std::size_t c = 0; c < head_dim; ++c) {
      part_val[idx * head_dim + c] = static_cast<float>(acc[c]);
    }
  });
}

// Whole fused layer of cpp/reference/qwen35.cpp:254-382: per-head RMSNorm
// with weight, partial RoPE, causal attention, sigmoid gate, output
// projection accumulated in double.  input is [tokens][q | k | v | gate].
void orc_full_attention_layer(const float *input, float *output,
                              const float *q_norm_w, const float *k_norm_w,
                              const float *out_w, std::size_t tokens,
                              std::size_t hidden, std::size_t q_heads,
                              std::size_t kv_heads, std::size_t head_dim,
                              std::size_t rotary, std::size_t pos_offset,
                              float rope_base, float eps, int threads) {
  const std::size_t q_size = q_heads * head_dim;
  const std::size_t kv_size = kv_heads * head_dim;
  const std::size_t stride = q_size + 2 * kv_size + hidden;
  std::vector<float> q(tokens * q_size);
  std::vector<float> k(tokens * kv_size);
  std::vector<float> v(tokens * kv_size);
  std::vector<float> gate(tokens * hidden);
  for (std::size_t t = 0; t < tokens; ++t) {
    const float *row = input + t * stride;
    std::copy(row, row + q_size, q.begin() + t * q_size);
    std::copy(row + q_size, row + q_size + kv_size, k.begin() + t * kv_size);
    std::copy(row + q_size + kv_size, row + q_size + 2 * kv_size,
              v.begin() + t * kv_size);
    std::copy(row + q_size + 2 * kv_size, row + stride,
              gate.begin() + t * hidden);
    for (std::size_t h = 0; h < q_heads; ++h) {
      float *qh = q.data() + t * q_size + h * head_dim;
      rms_norm_rows(qh, q_norm_w, qh, 1, head_dim, eps);
      partial_rope(qh, rotary, pos_offset + t, rope_base);
    }
    for (std::size_t h = 0; h < kv_heads; ++h) {
      float *kh = k.data() + t * kv_size + h * head_dim;
      rms_norm_rows(kh, k_norm_w, kh, 1, head_dim, eps);
      partial_rope(kh, rotary, pos_offset + t, rope_base);
    }
  }
  std::vector<float> attn(tokens * hidden);
  orc_attention_core_f32(q.data(), k.data(), v.data(), gate.data(),
                         attn.data(), tokens, q_heads, kv_heads, head_dim, 0,
                         threads);
  // cpp/reference/qwen35.cpp:372-380: weight is [in][out], double sum.
  parallel_for(tokens, threads, [&](std::size_t t) {
    for (std::size_t oc = 0; oc < hidden; ++oc) {
      double sum = 0.0;
      for (std::size_t ic = 0; ic < hidden; ++ic) {
        sum += static_cast<double>(attn[t * hidden + ic]) *
               static_cast<double>(out_w[ic * hidden + oc]);
      }
      output[t * hidden + oc] = static_cast<float>(sum);
    }
  });
}

// Pre-attention step alone (cpp/reference/qwen35.cpp:298-313): RMSNorm with
// weight then partial RoPE on [tokens][heads][D] in place.
void orc_qk_norm_rope(float *x, const float *norm_w, std::size_t tokens,
                      std::size_t heads, std::size_t head_dim,
                      std::size_t rotary, std::size_t pos_offset,
                      float rope_base, float eps) {
  for (std::size_t t = 0; t < tokens; ++t) {
    for (std::size_t h = 0; h < heads; ++h) {
      float *xh = x + (t * heads + h) * head_dim;
      rms_norm_rows(xh, norm_w, xh, 1, head_dim, eps);
      partial_rope(xh, rotary, pos_offset + t, rope_base);
    }
  }
}

// Recurrence core of cpp/reference/qwen35.cpp:459-518 for `tokens` steps.
// q [T][Hk][dk] must already carry the 1/sqrt(dk) scale (reference
// :448-456), k [T][Hk][dk] already L2-normalised, v [T][Hv][dv],
// beta [T][Hv] already sigmoid'ed, decay [T][Hv] already exp'ed.
// state [Hv][dk][dv] is updated in place; out is [T][Hv][dv] (the "raw"
// vector before the output norm).  key head of value head h is h % Hk.
void orc_gdn_core(const float *q, const float *k, const float *v,
                  const float *beta, const float *decay, float *state,
                  float *out, std::size_t tokens, std::size_t key_heads,
                  std::size_t value_heads, std::size_t key_dim,
                  std::size_t value_dim, int threads) {
  parallel_for(value_heads, threads, [&](std::size_t vh) {
    const std::size_t kh = vh % key_heads;
    float *s = state + vh * key_dim * value_dim;
    std::vector<float> delta(value_dim);
    for (std::size_t t = 0; t < tokens; ++t) {
      const float *qh = q + (t * key_heads + kh) * key_dim;
      const float *kk = k + (t * key_heads + kh) * key_dim;
      const float *vv = v + (t * value_heads + vh) * value_dim;
      const float b = beta[t * value_heads + vh];
      const float dc = decay[t * value_heads + vh];
      for (std::size_t i = 0; i < key_dim * value_dim; ++i) {
        s[i] *= dc;
      }
      for (std::size_t c = 0; c < value_dim; ++c) {
        double mem = 0.0;
        for (std::size_t r = 0; r < key_dim; ++r) {
          mem += static_cast<double>(s[r * value_dim + c]) *
                 static_cast<double>(kk[r]);
        }
        delta[c] = (vv[c] - static_cast<float>(mem)) * b;
      }
      for (std::size_t r = 0; r < key_dim; ++r) {
        for (std::size_t c = 0; c < value_dim; ++c) {
          s[r * value_dim + c] += kk[r] * delta[c];
        }
      }
      float *o = out + (t * value_heads + vh) * value_dim;
      for (std::size_t c = 0; c < value_dim; ++c) {
        double sum = 0.0;
        for (std::size_t r = 0; r < key_dim; ++r) {
          sum += static_cast<double>(s[r * value_dim + c]) *
                 static_cast<double>(qh[r]);
        }
        o[c] = static_cast<float>(sum);
      }
    }
  });
}

// Whole gated-delta layer of cpp/reference/qwen35.cpp:384-549: depthwise
// causal conv + SiLU with state [channel][W-1], L2 norm of q,k (eps 1e-6)
// and q * 1/sqrt(dk), beta = sigmoid(b), decay = exp(A * softplus(a + dt)),
// recurrence, per-head RMSNorm(dv) * w * SiLU(z).
// input is [T][q | k | v | b | a | z].
void orc_gated_delta_layer(const float *input, float *output,
                           const float *conv_w, const float *rec_a,
                           const float *dt_bias, const float *out_norm_w,
                           float *conv_state, float *rec_state,
                           std::size_t tokens, std::size_t hidden,
                           std::size_t key_heads, std::size_t value_heads,
                           std::size_t key_dim, std::size_t value_dim,
                           std::size_t conv_width, float eps, int threads) {
  const std::size_t key_size = key_heads * key_dim;
  const std::size_t value_size = value_heads * value_dim;
  const std::size_t conv_dim = 2 * key_size + value_size;
  const std::size_t stride = conv_dim + 2 * value_heads + hidden;
  const std::size_t hist = conv_width - 1;
  std::vector<float> q(tokens * key_size);
  std::vector<float> k(tokens * key_size);
  std::vector<float> v(tokens * value_size);
  std::vector<float> beta(tokens * value_heads);
  std::vector<float> decay(tokens * value_heads);
  std::vector<float> conv(conv_dim);
  const float q_scale = 1.0F / std::sqrt(static_cast<float>(key_dim));
  for (std::size_t t = 0; t < tokens; ++t) {
    const float *row = input + t * stride;
    // :417-427 last tap multiplies the current token.
    for (std::size_t ch = 0; ch < conv_dim; ++ch) {
      float sum = row[ch] * conv_w[ch * conv_width + conv_width - 1];
      for (std::size_t hi = 0; hi + 1 < conv_width; ++hi) {
        sum += conv_state[ch * hist + hi] * conv_w[ch * conv_width + hi];
      }
      conv[ch] = silu_f(sum);
    }
    // :429-438 shift history.
    if (conv_width > 1) {
      for (std::size_t ch = 0; ch < conv_dim; ++ch) {
        for (std::size_t hi = 0; hi + 2 < conv_width; ++hi) {
          conv_state[ch * hist + hi] = conv_state[ch * hist + hi + 1];
        }
        conv_state[ch * hist + conv_width - 2] = row[ch];
      }
    }
    // :447-457.
    for (std::size_t h = 0; h < key_heads; ++h) {
      float *qh = conv.data() + h * key_dim;
      float *kh = conv.data() + key_size + h * key_dim;
      l2_normalize(qh, key_dim, 1.0e-6F);
      l2_normalize(kh, key_dim, 1.0e-6F);
      for (std::size_t c = 0; c < key_dim; ++c) {
        qh[c] *= q_scale;
      }
    }
    std::copy(conv.begin(), conv.begin() + key_size, q.begin() + t * key_size);
    std::copy(conv.begin() + key_size, conv.begin() + 2 * key_size,
              k.begin() + t * key_size);
    std::copy(conv.begin() + 2 * key_size, conv.end(),
              v.begin() + t * value_size);
    const float *b = row + conv_dim;
    const float *a = row + conv_dim + value_heads;
    for (std::size_t h = 0; h < value_heads; ++h) {
      beta[t * value_heads + h] = sigmoid_f(b[h]);
      decay[t * value_heads + h] =
          std::exp(rec_a[h] * softplus_f(a[h] + dt_bias[h]));
    }
  }
  std::vector<float> raw(tokens * value_size);
  orc_gdn_core(q.data(), k.data(), v.data(), beta.data(), decay.data(),
               rec_state, raw.data(), tokens, key_heads, value_heads, key_dim,
               value_dim, threads);
  // :520-525.
  for (std::size_t t = 0; t < tokens; ++t) {
    const float *z = input + t * stride + conv_dim + 2 * value_heads;
    rms_norm_rows(raw.data() + t * value_size, out_norm_w,
                  output + t * hidden, value_heads, value_dim, eps);
    for (std::size_t i = 0; i < hidden; ++i) {
      output[t * hidden + i] *= silu_f(z[i]);
    }
  }
}

// cpp/reference/correctness.cpp:18-75 (max abs, max rel with floor, cosine,
// non-finite mismatches) plus the relative L2 error the parity gates use.
void orc_compare(const float *cand, const float *ref, std::size_t n,
                 double rel_floor, double *out5) {
  double max_abs = 0.0;
  double max_rel = 0.0;
  double dot = 0.0;
  double cn = 0.0;
  double rn = 0.0;
  double dn = 0.0;
  double mismatches = 0.0;
  for (std::size_t i = 0; i < n; ++i) {
    const float c = cand[i];
    const float r = ref[i];
    if (!std::isfinite(c) || !std::isfinite(r)) {
      const bool same_inf = std::isinf(c) && std::isinf(r) &&
                            std::signbit(c) == std::signbit(r);
      if (!same_inf) {
        mismatches += 1.0;
      }
      continue;
    }
    const double cd = c;
    const double rd = r;
    const double err = std::fabs(cd - rd);
    max_abs = std::max(max_abs, err);
    max_rel = std::max(max_rel, err / std::max(std::fabs(rd), rel_floor));
    dot += cd * rd;
    cn += cd * cd;
    rn += rd * rd;
    dn += (cd - rd) * (cd - rd);
  }
  double cosine = 1.0;
  if (cn == 0.0 && rn == 0.0) {
    cosine = 1.0;
  } else if (cn == 0.0 || rn == 0.0) {
    cosine = 0.0;
  } else {
    cosine = std::clamp(dot / (std::sqrt(cn) * std::sqrt(rn)), -1.0, 1.0);
  }
  out5[0] = max_abs;
  out5[1] = max_rel;
  out5[2] = cosine;
  out5[3] = mismatches;
  out5[4] = rn > 0.0 ? std::sqrt(dn / rn) : std::sqrt(dn);
}

} // extern "C"
