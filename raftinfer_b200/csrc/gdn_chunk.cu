// Chunk-64 WY-form prefill of the gated delta rule for key_dim = value_dim = 128.  The reference has only the
// token-sequential recurrence (cpp/kernels/qwen35_delta.cu:482-576, cpp/reference/qwen35.cpp:459-518); this is the
// same recurrence regrouped so that the dense work runs on the tensor cores.
//
// Per value head (key head = head % key_heads), for a chunk of C = 64 tokens entering with state S0 [128][128],
// with G_i the running sum of the log decays inside the chunk (decay applied before the read, as the reference):
//   A_ij  = beta_i exp(G_i - G_j) (k_i . k_j)   for j < i            T = (I + A)^-1
//   W     = T diag(beta exp(G)) K                U = T diag(beta) V
//   Delta = U - W S0
//   O     = diag(exp(G)) Q S0 + P Delta,         P_ij = exp(G_i - G_j) (q_i . k_j) for j <= i
//   S_C   = exp(G_C) S0 + K^T diag(exp(G_C - G)) Delta
// Every decay factor is exp of a non-positive number.  A ragged last chunk is padded with inert rows
// (beta = 0, log decay = 0, k = q = v = 0), which leave the state untouched.
//
// Two kernels.  `prepare` is parallel over (chunk, value head): T by forward substitution in FP32, the four
// dense products on mma.sync TF32 tensor-core tiles, results (W, U, P, G) to the workspace.  `apply` walks the
// chunks in order for one (value head, 32-column slice of the state): the slice lives in shared memory, and
// W S0, Q S0, P Delta and K^T Delta are TF32 tensor-core products.  State columns are independent, so the
// four slices of a head never talk to each other.  TF32 (10-bit mantissa, FP32 accumulate) rather than BF16
// keeps the FP32 state within 1e-3 relative L2 of the sequential recurrence over 64 chunks.
//
// Dense flops per launch: chunks * value_heads * [2 C^2 (3 dk + 2 dv) + 6 C dk dv].

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

namespace rib200 {
namespace {

constexpr int kDim = 128;
constexpr int kChunk = 64;
constexpr int kSlice = 32;          // state columns per apply CTA
constexpr int kPitchRow = 132;      // [row][k] operands read along k by lane%4: pitch = 4 mod 32
constexpr int kPitchCol = 136;      // [k][n] operands read along n by lane/4: pitch = 8 mod 32
constexpr int kPitchSq = 68;        // 64-wide [row][k] operands
constexpr int kPitchSlice = 40;     // 32-wide [k][n] operands
// Workspace record of one (chunk, value head), in floats.  Every block is stored at the padded pitch the apply
// kernel reads it at, so that one bulk copy brings a block into shared memory ready for conflict-free fragment reads.
constexpr std::size_t kRecW = 0;                                   // [64][132], rounded to TF32
constexpr std::size_t kRecGamma = kRecW + kChunk * kPitchRow;      // [64] exp(G_i)
constexpr std::size_t kRecE = kRecGamma + kChunk;                  // [64] exp(G_C - G_i)
constexpr std::size_t kRecP = kRecE + kChunk;                      // [64][68], rounded to TF32
constexpr std::size_t kRecU = kRecP + kChunk * kPitchSq;           // [4 slices][64][40]
constexpr std::size_t kRecFloats = kRecU + (kDim / kSlice) * kChunk * kPitchSlice;
// FP32 (TF32-rounded) copy of one (chunk, key head)'s q and k rows, zero rows past the last token
constexpr std::size_t kCopyQ = 0;                                  // [64][132]
constexpr std::size_t kCopyK = kCopyQ + kChunk * kPitchRow;        // [64][136]
constexpr std::size_t kCopyFloats = kCopyK + kChunk * kPitchCol;
static_assert(kRecFloats % 4 == 0 && kCopyFloats % 4 == 0 && kRecP % 4 == 0 && kRecU % 4 == 0, "16-byte blocks");

struct ChunkParams {
  const void *q, *k, *v;
  std::size_t q_stride, k_stride, v_stride;
  const float *beta;
  const float *log_decay;
  float *state;
  float *out;
  float *workspace;
  float *qk_copy; // [chunk][key_head] copy records, after the chunk records
  unsigned int *status;
  std::uint32_t tokens;
  std::uint32_t chunks;
  std::uint32_t key_heads;
  std::uint32_t value_heads;
};

__device__ __forceinline__ std::uint32_t tf32(float x) {
  std::uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const std::uint32_t (&a)[4], std::uint32_t b0,
                                         std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Rows [tok0, tok0 + 64) of a [token][heads][128] operand (head `head`) go to dst[64][pitch] as FP32 in two halves,
// so that other work can run while the loads are in flight: fetch_rows reads this thread's 32 elements of its row
// into registers (zeros at or past `tokens`), store_rows converts and writes them.  256 threads.
template <bool F32> struct RowRegs {
  uint4 v[F32 ? 8 : 4];
};

template <bool F32>
__device__ __forceinline__ RowRegs<F32> fetch_rows(const void *src, std::size_t stride, std::uint32_t head,
                                                   std::uint32_t tok0, std::uint32_t tokens) {
  RowRegs<F32> regs;
  const int row = threadIdx.x >> 2;
  const int part = threadIdx.x & 3; // 32 elements each
  const std::uint32_t tok = tok0 + row;
  constexpr int kVectors = F32 ? 8 : 4;
  if (tok >= tokens) {
#pragma unroll
    for (int i = 0; i < kVectors; ++i) {
      regs.v[i] = make_uint4(0U, 0U, 0U, 0U);
    }
    return regs;
  }
  const std::size_t base = static_cast<std::size_t>(tok) * stride + head * kDim + part * 32;
  const uint4 *s = F32 ? reinterpret_cast<const uint4 *>(static_cast<const float *>(src) + base)
                       : reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(src) + base);
#pragma unroll
  for (int i = 0; i < kVectors; ++i) {
    regs.v[i] = s[i];
  }
  return regs;
}

template <bool F32> __device__ __forceinline__ void store_rows(float *dst, int pitch, const RowRegs<F32> &regs) {
  const int row = threadIdx.x >> 2;
  const int part = threadIdx.x & 3;
  float *d = dst + row * pitch + part * 32;
  if constexpr (F32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      *reinterpret_cast<uint4 *>(d + 4 * i) = regs.v[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const std::uint32_t w[4] = {regs.v[i].x, regs.v[i].y, regs.v[i].z, regs.v[i].w};
      float4 lo;
      float4 hi;
      lo.x = __uint_as_float(w[0] << 16);
      lo.y = __uint_as_float(w[0] & 0xFFFF0000U);
      lo.z = __uint_as_float(w[1] << 16);
      lo.w = __uint_as_float(w[1] & 0xFFFF0000U);
      hi.x = __uint_as_float(w[2] << 16);
      hi.y = __uint_as_float(w[2] & 0xFFFF0000U);
      hi.z = __uint_as_float(w[3] << 16);
      hi.w = __uint_as_float(w[3] & 0xFFFF0000U);
      *reinterpret_cast<float4 *>(d + 8 * i) = lo;
      *reinterpret_cast<float4 *>(d + 8 * i + 4) = hi;
    }
  }
}

// Copies a dense [rows][cols] FP32 block from global memory into dst[rows][pitch].  256 threads.
__device__ __forceinline__ void load_block(float *dst, int pitch, const float *src, int rows, int cols,
                                           int src_pitch) {
  const int vec_per_row = cols / 4;
  for (int i = threadIdx.x; i < rows * vec_per_row; i += 256) {
    const int r = i / vec_per_row;
    const int c = (i % vec_per_row) * 4;
    *reinterpret_cast<float4 *>(dst + r * pitch + c) = *reinterpret_cast<const float4 *>(src + r * src_pitch + c);
  }
}

// Optional timeline probe (compile with -DRIB200_TRACE): thread 0 of the first CTA stamps clock64() at eight points
// per chunk, the producer's lane 0 at four more; the first prepare CTA stamps row 127.
#ifdef RIB200_TRACE
__device__ long long g_gdn_trace[128 * 16];
#define RIB200_GDN_STAMP(chunk, slot)                                  \
  do {                                                                 \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (chunk) < 128) {         \
      g_gdn_trace[(chunk) * 16 + (slot)] = clock64();                  \
    }                                                                  \
  } while (0)
#else
#define RIB200_GDN_STAMP(chunk, slot) \
  do {                                \
  } while (0)
#endif

// ---- prepare: per (chunk, value head) ---------------------------------------------------------------
constexpr int kPrepSmemFloats = kChunk * kPitchRow + kChunk * kPitchCol + 2 * kChunk * kPitchSq + 3 * kChunk;

template <bool F32>
__global__ void __launch_bounds__(256, 2) gdn_chunk_prepare_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) float prep_smem[];
  float *sK = prep_smem;                      // [64][132]
  float *sX = sK + kChunk * kPitchRow;        // [64][136]  Q, later V
  float *sA = sX + kChunk * kPitchCol;        // [64][68]
  float *sT = sA + kChunk * kPitchSq;         // [64][68]
  float *sG = sT + kChunk * kPitchSq;         // [64] inclusive running log decay
  float *sBeta = sG + kChunk;                 // [64]
  float *sBg = sBeta + kChunk;                // [64] beta * exp(G)

  const std::uint32_t chunk = blockIdx.x;
  const std::uint32_t head = blockIdx.y;
  const std::uint32_t key_head = head % p.key_heads;
  const std::uint32_t tok0 = chunk * kChunk;
  float *rec = p.workspace + (static_cast<std::size_t>(chunk) * p.value_heads + head) * kRecFloats;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;

  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 0);
  }
  {
    const RowRegs<F32> k_regs = fetch_rows<F32>(p.k, p.k_stride, key_head, tok0, p.tokens);
    const RowRegs<F32> q_regs = fetch_rows<F32>(p.q, p.q_stride, key_head, tok0, p.tokens);
    if (warp == 0) { // running sum of the log decays: two tokens per lane, warp scan
      const std::uint32_t tok_a = tok0 + lane;
      const std::uint32_t tok_b = tok_a + 32;
      float a = tok_a < p.tokens ? p.log_decay[static_cast<std::size_t>(tok_a) * p.value_heads + head] : 0.0F;
      float b = tok_b < p.tokens ? p.log_decay[static_cast<std::size_t>(tok_b) * p.value_heads + head] : 0.0F;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float ua = __shfl_up_sync(0xFFFFFFFFU, a, d);
        const float ub = __shfl_up_sync(0xFFFFFFFFU, b, d);
        if (lane >= d) {
          a += ua;
          b += ub;
        }
      }
      b += __shfl_sync(0xFFFFFFFFU, a, 31);
      sG[lane] = a;
      sG[lane + 32] = b;
    } else if (warp <= 2) {
      const std::uint32_t tok = tok0 + lane + 32 * (warp - 1);
      sBeta[lane + 32 * (warp - 1)] =
          tok < p.tokens ? p.beta[static_cast<std::size_t>(tok) * p.value_heads + head] : 0.0F;
    }
    store_rows<F32>(sK, kPitchRow, k_regs);
    store_rows<F32>(sX, kPitchRow, q_regs); // Q is read along k like K: same pitch; V will use the full pitch
  }
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 1);
  }
  if (head < p.key_heads) { // the first value head of each key head leaves the q and k rows for the apply kernel
    float *copy = p.qk_copy + (static_cast<std::size_t>(chunk) * p.key_heads + head) * kCopyFloats;
    for (int i = threadIdx.x; i < kChunk * (kDim / 4); i += 256) {
      const int r = i / (kDim / 4);
      const int c = (i % (kDim / 4)) * 4;
      const float4 kv = *reinterpret_cast<const float4 *>(sK + r * kPitchRow + c);
      const float4 qv = *reinterpret_cast<const float4 *>(sX + r * kPitchRow + c);
      *reinterpret_cast<float4 *>(copy + kCopyK + r * kPitchCol + c) =
          make_float4(__uint_as_float(tf32(kv.x)), __uint_as_float(tf32(kv.y)), __uint_as_float(tf32(kv.z)),
                      __uint_as_float(tf32(kv.w)));
      *reinterpret_cast<float4 *>(copy + kCopyQ + r * kPitchRow + c) =
          make_float4(__uint_as_float(tf32(qv.x)), __uint_as_float(tf32(qv.y)), __uint_as_float(tf32(qv.z)),
                      __uint_as_float(tf32(qv.w)));
    }
  }
  if (threadIdx.x < kChunk) {
    const float gamma = expf(sG[threadIdx.x]);
    sBg[threadIdx.x] = sBeta[threadIdx.x] * gamma;
    rec[kRecGamma + threadIdx.x] = gamma;
    rec[kRecE + threadIdx.x] = expf(sG[kChunk - 1] - sG[threadIdx.x]);
  }

  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 2);
  }
  // K K^T and Q K^T, 64 x 64 each, contraction over the 128 dims.  Warp: rows 16*(warp&3).., columns 32*(warp>>2)..
  {
    const int mt = warp & 3;
    const int nt0 = (warp >> 2) * 4;
    float acc_k[4][4] = {};
    float acc_q[4][4] = {};
#pragma unroll 4
    for (int ks = 0; ks < 16; ++ks) {
      std::uint32_t ak[4];
      std::uint32_t aq[4];
      const int col = ks * 8 + t;
      ak[0] = tf32(sK[(16 * mt + g) * kPitchRow + col]);
      ak[1] = tf32(sK[(16 * mt + g + 8) * kPitchRow + col]);
      ak[2] = tf32(sK[(16 * mt + g) * kPitchRow + col + 4]);
      ak[3] = tf32(sK[(16 * mt + g + 8) * kPitchRow + col + 4]);
      aq[0] = tf32(sX[(16 * mt + g) * kPitchRow + col]);
      aq[1] = tf32(sX[(16 * mt + g + 8) * kPitchRow + col]);
      aq[2] = tf32(sX[(16 * mt + g) * kPitchRow + col + 4]);
      aq[3] = tf32(sX[(16 * mt + g + 8) * kPitchRow + col + 4]);
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int j = 8 * (nt0 + n) + g;
        const std::uint32_t b0 = tf32(sK[j * kPitchRow + col]);
        const std::uint32_t b1 = tf32(sK[j * kPitchRow + col + 4]);
        mma_tf32(acc_k[n], ak, b0, b1);
        mma_tf32(acc_q[n], aq, b0, b1);
      }
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 16 * mt + g + (e >> 1) * 8;
        const int j = 8 * (nt0 + n) + 2 * t + (e & 1);
        const float decay = j <= i ? expf(sG[i] - sG[j]) : 0.0F;
        sA[i * kPitchSq + j] = j < i ? sBeta[i] * decay * acc_k[n][e] : 0.0F;
        rec[kRecP + i * kPitchSq + j] = __uint_as_float(tf32(decay * acc_q[n][e]));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 3);
  }

  // V replaces Q; T = (I + A)^-1 by forward substitution in FP32.  Column c belongs to four neighbouring lanes
  // that split the sum over j in groups of four (lane `part` holds T[16 q + 4 part + r][c] in mine[4 q + r], and
  // reads its four A_ij with one 16-byte load) and add their parts with two shuffles.
  const RowRegs<F32> v_regs = fetch_rows<F32>(p.v, p.v_stride, head, tok0, p.tokens); // lands during the substitution
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 4);
  }
  {
    const int c = threadIdx.x >> 2;
    const int part = threadIdx.x & 3;
    float mine[kChunk / 4];
#pragma unroll
    for (int m = 0; m < kChunk / 4; ++m) {
      mine[m] = 0.0F;
    }
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      float acc0 = 0.0F;
      float acc1 = 0.0F;
#pragma unroll
      for (int q = 0; 16 * q < i; ++q) { // A is zero on and above the diagonal, entries not yet known are zero
        const float4 a = *reinterpret_cast<const float4 *>(sA + i * kPitchSq + 16 * q + 4 * part);
        acc0 -= a.x * mine[4 * q];
        acc1 -= a.y * mine[4 * q + 1];
        acc0 -= a.z * mine[4 * q + 2];
        acc1 -= a.w * mine[4 * q + 3];
      }
      float acc = acc0 + acc1;
      acc += __shfl_xor_sync(0xFFFFFFFFU, acc, 1);
      acc += __shfl_xor_sync(0xFFFFFFFFU, acc, 2);
      const float value = (i == c ? 1.0F : 0.0F) + acc;
      if (part == ((i >> 2) & 3)) {
        mine[4 * (i >> 4) + (i & 3)] = value;
      }
    }
    // stores after the loop: none of the loads above has to wait for one
#pragma unroll
    for (int m = 0; m < kChunk / 4; ++m) {
      sT[(16 * (m >> 2) + 4 * part + (m & 3)) * kPitchSq + c] = mine[m];
    }
  }
  store_rows<F32>(sX, kPitchCol, v_regs);
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 5);
  }

  // W = T (diag(beta exp(G)) K), U = T (diag(beta) V): 64 x 128 each, contraction over the 64 tokens.
  // Warp: rows 16*(warp&3).., columns 64*(warp>>2)...  T is lower triangular: k-steps above the tile are skipped.
  {
    const int mt = warp & 3;
    const int n0 = (warp >> 2) * 64;
    float acc_w[8][4] = {};
    float acc_u[8][4] = {};
    const int ks_end = 2 * mt + 2;
    for (int ks = 0; ks < ks_end; ++ks) {
      std::uint32_t a[4];
      const int col = ks * 8 + t;
      a[0] = tf32(sT[(16 * mt + g) * kPitchSq + col]);
      a[1] = tf32(sT[(16 * mt + g + 8) * kPitchSq + col]);
      a[2] = tf32(sT[(16 * mt + g) * kPitchSq + col + 4]);
      a[3] = tf32(sT[(16 * mt + g + 8) * kPitchSq + col + 4]);
      const float bg0 = sBg[col];
      const float bg1 = sBg[col + 4];
      const float be0 = sBeta[col];
      const float be1 = sBeta[col + 4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int d = n0 + 8 * n + g;
        mma_tf32(acc_w[n], a, tf32(sK[col * kPitchRow + d] * bg0), tf32(sK[(col + 4) * kPitchRow + d] * bg1));
        mma_tf32(acc_u[n], a, tf32(sX[col * kPitchCol + d] * be0), tf32(sX[(col + 4) * kPitchCol + d] * be1));
      }
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int d = n0 + 8 * n + 2 * t;
      const int i = 16 * mt + g;
      // W only ever feeds TF32 products: round it here, once
      *reinterpret_cast<float2 *>(rec + kRecW + i * kPitchRow + d) =
          make_float2(__uint_as_float(tf32(acc_w[n][0])), __uint_as_float(tf32(acc_w[n][1])));
      *reinterpret_cast<float2 *>(rec + kRecW + (i + 8) * kPitchRow + d) =
          make_float2(__uint_as_float(tf32(acc_w[n][2])), __uint_as_float(tf32(acc_w[n][3])));
      float *u = rec + kRecU + (d / kSlice) * (kChunk * kPitchSlice) + d % kSlice;
      *reinterpret_cast<float2 *>(u + i * kPitchSlice) = make_float2(acc_u[n][0], acc_u[n][1]);
      *reinterpret_cast<float2 *>(u + (i + 8) * kPitchSlice) = make_float2(acc_u[n][2], acc_u[n][3]);
    }
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 6);
  }
}

// ---- apply: per (state slice, value head), chunks in order ---------------------------------------------
// Eight consumer warps and one producer warp.  The producer streams each chunk's operands into shared memory with
// TMA bulk row copies (cp.async.bulk, bytes counted on an mbarrier), one chunk ahead of the consumers: W, K, the U
// slice and G sit in a two-stage ring, Q and P in single buffers that are refilled as soon as their last reader is
// done.  Rows land at padded pitches so that every tensor-core fragment read is free of bank conflicts.
// Every mbarrier wait is bounded; when one runs out the CTA records RIB200_DEVICE_WAIT_TIMED_OUT, stops waiting
// and copying, and runs to its end (its results are then meaningless, as the status word says).
constexpr int kApplyConsumers = 256;
constexpr int kApplyThreads = kApplyConsumers + 32;
constexpr int kStageW = 0;                                   // W, gamma, e: one block of the record
constexpr int kStageGamma = kStageW + kChunk * kPitchRow;
constexpr int kStageE = kStageGamma + kChunk;
constexpr int kStageK = kStageE + kChunk;
constexpr int kStageD = kStageK + kChunk * kPitchCol;
constexpr int kStageFloats = kStageD + kChunk * kPitchSlice;
constexpr int kApplyS = 0;
constexpr int kApplyStage = kApplyS + kDim * kPitchSlice;
constexpr int kApplyQ = kApplyStage + 2 * kStageFloats;
constexpr int kApplyP = kApplyQ + kChunk * kPitchRow;
constexpr int kApplyFloats = kApplyP + kChunk * kPitchSq;
constexpr int kApplyBars = 8; // full[2], empty[2], q_full, q_empty, p_full, p_empty
constexpr int kApplySmemBytes = kApplyFloats * 4 + kApplyBars * 8 + 16;
static_assert(kApplySmemBytes <= 232448, "apply kernel exceeds the shared memory of an SM");
constexpr long long kWaitLimitCycles = 1LL << 28;

__device__ __forceinline__ std::uint32_t smem_address(const void *p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarrier_init(std::uint32_t bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive(std::uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(std::uint32_t bar, std::uint32_t parity) {
  std::uint32_t done;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(std::uint32_t dst, const void *src, std::uint32_t bytes,
                                              std::uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }

__global__ void __launch_bounds__(kApplyThreads, 1) gdn_chunk_apply_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) float apply_smem[];
  float *sS = apply_smem + kApplyS;  // [128][40] state slice
  float *sQ = apply_smem + kApplyQ;  // [64][132]
  float *sP = apply_smem + kApplyP;  // [64][68]
  const std::uint32_t bars = smem_address(apply_smem + kApplyFloats);
  volatile std::uint32_t *abort_flag = reinterpret_cast<volatile std::uint32_t *>(apply_smem + kApplyFloats) +
                                       2 * kApplyBars;
  const std::uint32_t bar_full0 = bars, bar_empty0 = bars + 16, bar_q_full = bars + 32, bar_q_empty = bars + 40,
                      bar_p_full = bars + 48, bar_p_empty = bars + 56;

  const std::uint32_t slice = blockIdx.x;
  const std::uint32_t head = blockIdx.y;
  const std::uint32_t key_head = head % p.key_heads;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  float *state = p.state + static_cast<std::size_t>(head) * kDim * kDim + slice * kSlice;

  if (threadIdx.x == 0) {
    mbarrier_init(bar_full0, 1);
    mbarrier_init(bar_full0 + 8, 1);
    mbarrier_init(bar_empty0, 8);
    mbarrier_init(bar_empty0 + 8, 8);
    mbarrier_init(bar_q_full, 1);
    mbarrier_init(bar_q_empty, 8);
    mbarrier_init(bar_p_full, 1);
    mbarrier_init(bar_p_empty, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (threadIdx.x < kApplyConsumers) {
    load_block(sS, kPitchSlice, state, kDim, kSlice, kDim);
  }
  fence_proxy_async();
  __syncthreads();

  // bounded wait; once the CTA has given up nobody waits any more
  auto wait = [&](std::uint32_t bar, std::uint32_t parity) {
    if (*abort_flag != 0 || mbarrier_try_wait(bar, parity)) {
      return;
    }
    const long long started = clock64();
    while (!mbarrier_try_wait(bar, parity)) {
      if (*abort_flag != 0) {
        return;
      }
      if (clock64() - started > kWaitLimitCycles) {
        *abort_flag = 1;
        atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
        return;
      }
    }
  };

  if (warp == kApplyConsumers / 32) {
    // ---- producer ----
    // One lane issues five bulk copies per chunk; every block of the records is stored ready-padded.
    std::uint32_t issued[4] = {0, 0, 0, 0}; // fills of stage 0, stage 1, Q, P
    if (lane == 0) {
      for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
        const float *rec = p.workspace + (static_cast<std::size_t>(chunk) * p.value_heads + head) * kRecFloats;
        const float *copy = p.qk_copy + (static_cast<std::size_t>(chunk) * p.key_heads + key_head) * kCopyFloats;
        const std::uint32_t s = chunk & 1U;
        float *stage = apply_smem + kApplyStage + s * kStageFloats;
        // stage: W with gamma and e, K, U slice
        if (chunk >= 2) {
          wait(bar_empty0 + 8 * s, ((chunk >> 1) - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        RIB200_GDN_STAMP(chunk, 8);
        fence_proxy_async();
        constexpr std::uint32_t kWBytes = (kChunk * kPitchRow + 2 * kChunk) * 4;
        constexpr std::uint32_t kKBytes = kChunk * kPitchCol * 4;
        constexpr std::uint32_t kUBytes = kChunk * kPitchSlice * 4;
        mbarrier_expect_tx(bar_full0 + 8 * s, kWBytes + kKBytes + kUBytes);
        bulk_copy_g2s(smem_address(stage + kStageW), rec + kRecW, kWBytes, bar_full0 + 8 * s);
        bulk_copy_g2s(smem_address(stage + kStageD), rec + kRecU + slice * (kChunk * kPitchSlice), kUBytes,
                      bar_full0 + 8 * s);
        bulk_copy_g2s(smem_address(stage + kStageK), copy + kCopyK, kKBytes, bar_full0 + 8 * s);
        ++issued[s];
        RIB200_GDN_STAMP(chunk, 9);
        // Q
        if (chunk >= 1) {
          wait(bar_q_empty, (chunk - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        fence_proxy_async();
        mbarrier_expect_tx(bar_q_full, kChunk * kPitchRow * 4);
        bulk_copy_g2s(smem_address(sQ), copy + kCopyQ, kChunk * kPitchRow * 4, bar_q_full);
        ++issued[2];
        RIB200_GDN_STAMP(chunk, 10);
        // P
        if (chunk >= 1) {
          wait(bar_p_empty, (chunk - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        fence_proxy_async();
        mbarrier_expect_tx(bar_p_full, kChunk * kPitchSq * 4);
        bulk_copy_g2s(smem_address(sP), rec + kRecP, kChunk * kPitchSq * 4, bar_p_full);
        ++issued[3];
        RIB200_GDN_STAMP(chunk, 11);
      }
    }
    // after giving up: let the copies already issued land before the CTA's shared memory goes away
    if (lane == 0 && *abort_flag != 0) {
      const std::uint32_t full_bars[4] = {bar_full0, bar_full0 + 8, bar_q_full, bar_p_full};
      for (int b = 0; b < 4; ++b) {
        if (issued[b] > 0) {
          const std::uint32_t parity = (issued[b] - 1) & 1U;
          const long long started = clock64();
          while (!mbarrier_try_wait(full_bars[b], parity) && clock64() - started < kWaitLimitCycles) {
          }
        }
      }
    }
    return;
  }

  // ---- consumers ----
  const int g = lane >> 2;
  const int t = lane & 3;
  const int mt = warp & 3;
  const int nc0 = (warp >> 2) * 16;
  for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
    const std::uint32_t tok0 = chunk * kChunk;
    const std::uint32_t s = chunk & 1U;
    float *stage = apply_smem + kApplyStage + s * kStageFloats;
    const float *sW = stage + kStageW;
    const float *sK = stage + kStageK;
    float *sD = stage + kStageD;
    const float *sGamma = stage + kStageGamma;
    const float *sE = stage + kStageE;

    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 0);
    }
    wait(bar_full0 + 8 * s, (chunk >> 1) & 1U);
    wait(bar_q_full, chunk & 1U);
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 1);
    }
    consumer_sync(); // the previous chunk's state update is complete
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 2);
    }

    // W S0 and Q S0: 64 x 32, contraction over 128.  Warp: rows 16*(warp&3).., columns 16*(warp>>2)..
    // W and Q arrive already rounded to TF32.
    float acc_w[2][4] = {};
    float acc_o[2][4] = {};
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      std::uint32_t aw[4];
      std::uint32_t aq[4];
      const int col = ks * 8 + t;
      aw[0] = __float_as_uint(sW[(16 * mt + g) * kPitchRow + col]);
      aw[1] = __float_as_uint(sW[(16 * mt + g + 8) * kPitchRow + col]);
      aw[2] = __float_as_uint(sW[(16 * mt + g) * kPitchRow + col + 4]);
      aw[3] = __float_as_uint(sW[(16 * mt + g + 8) * kPitchRow + col + 4]);
      aq[0] = __float_as_uint(sQ[(16 * mt + g) * kPitchRow + col]);
      aq[1] = __float_as_uint(sQ[(16 * mt + g + 8) * kPitchRow + col]);
      aq[2] = __float_as_uint(sQ[(16 * mt + g) * kPitchRow + col + 4]);
      aq[3] = __float_as_uint(sQ[(16 * mt + g + 8) * kPitchRow + col + 4]);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const std::uint32_t b0 = tf32(sS[col * kPitchSlice + nc0 + 8 * n + g]);
        const std::uint32_t b1 = tf32(sS[(col + 4) * kPitchSlice + nc0 + 8 * n + g]);
        mma_tf32(acc_w[n], aw, b0, b1);
        mma_tf32(acc_o[n], aq, b0, b1);
      }
    }
    __syncwarp();
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 3);
    }
    if (lane == 0) {
      mbarrier_arrive(bar_q_empty);
    }
    // Delta = U - W S0 (in place over the U slice); the output starts as exp(G_i) * (Q S0)_i
    {
      const int i0 = 16 * mt + g;
      const float gamma0 = sGamma[i0];
      const float gamma1 = sGamma[i0 + 8];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int c = nc0 + 8 * n + 2 * t;
        float2 lo = *reinterpret_cast<float2 *>(sD + i0 * kPitchSlice + c);
        float2 hi = *reinterpret_cast<float2 *>(sD + (i0 + 8) * kPitchSlice + c);
        lo.x -= acc_w[n][0];
        lo.y -= acc_w[n][1];
        hi.x -= acc_w[n][2];
        hi.y -= acc_w[n][3];
        *reinterpret_cast<float2 *>(sD + i0 * kPitchSlice + c) = lo;
        *reinterpret_cast<float2 *>(sD + (i0 + 8) * kPitchSlice + c) = hi;
        acc_o[n][0] *= gamma0;
        acc_o[n][1] *= gamma0;
        acc_o[n][2] *= gamma1;
        acc_o[n][3] *= gamma1;
      }
    }
    consumer_sync(); // Delta is complete
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 4);
    }

    // S = exp(G_C) S + K^T (diag(exp(G_C - G)) Delta): 128 x 32, contraction over the 64 tokens.
    // Warp: state rows 16*warp.., all 32 columns.  This is the step the next chunk waits for, so it runs first.
    {
      const float gamma_c = sGamma[kChunk - 1];
      float acc[4][4];
      const int r0 = 16 * warp + g;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int c = 8 * n + 2 * t;
        const float2 lo = *reinterpret_cast<const float2 *>(sS + r0 * kPitchSlice + c);
        const float2 hi = *reinterpret_cast<const float2 *>(sS + (r0 + 8) * kPitchSlice + c);
        acc[n][0] = lo.x * gamma_c;
        acc[n][1] = lo.y * gamma_c;
        acc[n][2] = hi.x * gamma_c;
        acc[n][3] = hi.y * gamma_c;
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        std::uint32_t a[4];
        const int tok = ks * 8 + t;
        a[0] = __float_as_uint(sK[tok * kPitchCol + 16 * warp + g]);
        a[1] = __float_as_uint(sK[tok * kPitchCol + 16 * warp + g + 8]);
        a[2] = __float_as_uint(sK[(tok + 4) * kPitchCol + 16 * warp + g]);
        a[3] = __float_as_uint(sK[(tok + 4) * kPitchCol + 16 * warp + g + 8]);
        const float e0 = sE[tok];
        const float e1 = sE[tok + 4];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const std::uint32_t b0 = tf32(sD[tok * kPitchSlice + 8 * n + g] * e0);
          const std::uint32_t b1 = tf32(sD[(tok + 4) * kPitchSlice + 8 * n + g] * e1);
          mma_tf32(acc[n], a, b0, b1);
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int c = 8 * n + 2 * t;
        *reinterpret_cast<float2 *>(sS + r0 * kPitchSlice + c) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2 *>(sS + (r0 + 8) * kPitchSlice + c) = make_float2(acc[n][2], acc[n][3]);
      }
    }

    // O += P Delta: 64 x 32, contraction over the 64 tokens (P is lower triangular: stop at the diagonal tile;
    // P arrives already rounded to TF32)
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 5);
    }
    wait(bar_p_full, chunk & 1U);
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 6);
    }
    for (int ks = 0; ks < 2 * mt + 2; ++ks) {
      std::uint32_t a[4];
      const int col = ks * 8 + t;
      a[0] = __float_as_uint(sP[(16 * mt + g) * kPitchSq + col]);
      a[1] = __float_as_uint(sP[(16 * mt + g + 8) * kPitchSq + col]);
      a[2] = __float_as_uint(sP[(16 * mt + g) * kPitchSq + col + 4]);
      a[3] = __float_as_uint(sP[(16 * mt + g + 8) * kPitchSq + col + 4]);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const std::uint32_t b0 = tf32(sD[col * kPitchSlice + nc0 + 8 * n + g]);
        const std::uint32_t b1 = tf32(sD[(col + 4) * kPitchSlice + nc0 + 8 * n + g]);
        mma_tf32(acc_o[n], a, b0, b1);
      }
    }
    __syncwarp();
    if (threadIdx.x == 0) {
      RIB200_GDN_STAMP(chunk, 7);
    }
    if (lane == 0) {
      mbarrier_arrive(bar_p_empty);
      mbarrier_arrive(bar_empty0 + 8 * s);
    }
    {
      const std::uint32_t r0 = tok0 + 16 * mt + g;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const std::size_t c = static_cast<std::size_t>(head) * kDim + slice * kSlice + nc0 + 8 * n + 2 * t;
        const std::size_t row_pitch = static_cast<std::size_t>(p.value_heads) * kDim;
        if (r0 < p.tokens) {
          *reinterpret_cast<float2 *>(p.out + r0 * row_pitch + c) = make_float2(acc_o[n][0], acc_o[n][1]);
        }
        if (r0 + 8 < p.tokens) {
          *reinterpret_cast<float2 *>(p.out + (r0 + 8) * row_pitch + c) = make_float2(acc_o[n][2], acc_o[n][3]);
        }
      }
    }
  }
  consumer_sync();
  for (int i = threadIdx.x; i < kDim * (kSlice / 4); i += kApplyConsumers) {
    const int r = i / (kSlice / 4);
    const int c = (i % (kSlice / 4)) * 4;
    *reinterpret_cast<float4 *>(state + r * kDim + c) = *reinterpret_cast<const float4 *>(sS + r * kPitchSlice + c);
  }
}

template <bool F32> void configure_once() {
  static std::once_flag flags[64];
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  std::call_once(flags[device], [] {
    cuda_ok(cudaFuncSetAttribute(gdn_chunk_prepare_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kPrepSmemFloats * 4),
            "gated-delta prepare shared-memory opt-in");
    cuda_ok(cudaFuncSetAttribute(gdn_chunk_apply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kApplySmemBytes),
            "gated-delta apply shared-memory opt-in");
  });
}

template <bool F32> void launch(const ChunkParams &params, cudaStream_t stream) {
  configure_once<F32>();
  gdn_chunk_prepare_kernel<F32>
      <<<dim3(params.chunks, params.value_heads), 256, kPrepSmemFloats * 4, stream>>>(params);
  cuda_ok(cudaGetLastError(), "gated-delta prepare launch");
  gdn_chunk_apply_kernel<<<dim3(kDim / kSlice, params.value_heads), kApplyThreads, kApplySmemBytes, stream>>>(params);
  cuda_ok(cudaGetLastError(), "gated-delta apply launch");
}

} // namespace

#ifdef RIB200_TRACE
extern "C" int rib200_debug_read_gdn_trace(long long *host, std::size_t count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_gdn_trace, count * sizeof(long long)));
}
#endif

std::size_t gdn_chunk_workspace_bytes(std::size_t tokens, std::size_t key_heads, std::size_t value_heads) {
  const std::size_t chunks = ceil_div(tokens, kChunk, "gated-delta chunk count overflows");
  const std::size_t records = mul(mul(chunks, value_heads, "gated-delta chunk workspace overflows"),
                                  kRecFloats * sizeof(float), "gated-delta chunk workspace overflows");
  const std::size_t copies = mul(mul(chunks, key_heads, "gated-delta chunk workspace overflows"),
                                 kCopyFloats * sizeof(float), "gated-delta chunk workspace overflows");
  return add(records, copies, "gated-delta chunk workspace overflows");
}

void launch_gdn_chunked(const GdnCoreArgs &a, void *workspace, cudaStream_t stream) {
  require(workspace != nullptr, "gated-delta chunked prefill needs its workspace");
  require(reinterpret_cast<std::uintptr_t>(workspace) % 16 == 0, "gated-delta chunk workspace is not 16-byte aligned");
  ChunkParams p{};
  p.q = a.q;
  p.k = a.k;
  p.v = a.v;
  p.q_stride = a.q_stride;
  p.k_stride = a.k_stride;
  p.v_stride = a.v_stride;
  p.beta = a.beta;
  p.log_decay = a.log_decay;
  p.state = a.state;
  p.out = a.out;
  p.workspace = static_cast<float *>(workspace);
  p.tokens = a.tokens;
  p.chunks = (a.tokens + kChunk - 1) / kChunk;
  p.key_heads = a.key_heads;
  p.value_heads = a.value_heads;
  p.status = device_status_word();
  p.qk_copy = p.workspace + static_cast<std::size_t>(p.chunks) * a.value_heads * kRecFloats;
  if (a.qkv_f32) {
    launch<true>(p, stream);
  } else {
    launch<false>(p, stream);
  }
}

} // namespace rib200
