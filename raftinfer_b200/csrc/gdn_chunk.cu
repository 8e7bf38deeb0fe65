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
// workspace record of one (chunk, value head), in floats
constexpr std::size_t kRecW = 0;
constexpr std::size_t kRecU = kChunk * kDim;
constexpr std::size_t kRecP = 2 * kChunk * kDim;
constexpr std::size_t kRecG = 2 * kChunk * kDim + kChunk * kChunk;
constexpr std::size_t kRecFloats = kRecG + kChunk;

struct ChunkParams {
  const void *q, *k, *v;
  std::size_t q_stride, k_stride, v_stride;
  const float *beta;
  const float *log_decay;
  float *state;
  float *out;
  float *workspace;
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

// Copies rows [tok0, tok0 + 64) of a [token][heads][128] operand (head `head`) into dst[64][pitch] as FP32;
// rows at or past `tokens` become zeros.  256 threads.
template <bool F32>
__device__ __forceinline__ void load_rows(float *dst, int pitch, const void *src, std::size_t stride,
                                          std::uint32_t head, std::uint32_t tok0, std::uint32_t tokens) {
  const int row = threadIdx.x >> 2;
  const int part = threadIdx.x & 3; // 32 elements each
  const std::uint32_t tok = tok0 + row;
  float *d = dst + row * pitch + part * 32;
  if (tok >= tokens) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      *reinterpret_cast<float4 *>(d + i) = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    }
    return;
  }
  const std::size_t base = static_cast<std::size_t>(tok) * stride + head * kDim + part * 32;
  if constexpr (F32) {
    const float *s = static_cast<const float *>(src) + base;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      *reinterpret_cast<float4 *>(d + i) = *reinterpret_cast<const float4 *>(s + i);
    }
  } else {
    const __nv_bfloat16 *s = static_cast<const __nv_bfloat16 *>(src) + base;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(s + i);
      const std::uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
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
      *reinterpret_cast<float4 *>(d + i) = lo;
      *reinterpret_cast<float4 *>(d + i + 4) = hi;
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

  load_rows<F32>(sK, kPitchRow, p.k, p.k_stride, key_head, tok0, p.tokens);
  load_rows<F32>(sX, kPitchCol, p.q, p.q_stride, key_head, tok0, p.tokens);
  if (threadIdx.x < kChunk) {
    const std::uint32_t tok = tok0 + threadIdx.x;
    const bool live = tok < p.tokens;
    sBeta[threadIdx.x] = live ? p.beta[static_cast<std::size_t>(tok) * p.value_heads + head] : 0.0F;
    sG[threadIdx.x] = live ? p.log_decay[static_cast<std::size_t>(tok) * p.value_heads + head] : 0.0F;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.0F;
    for (int i = 0; i < kChunk; ++i) {
      run += sG[i];
      sG[i] = run;
    }
  }
  __syncthreads();
  if (threadIdx.x < kChunk) {
    sBg[threadIdx.x] = sBeta[threadIdx.x] * expf(sG[threadIdx.x]);
    rec[kRecG + threadIdx.x] = sG[threadIdx.x];
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
      aq[0] = tf32(sX[(16 * mt + g) * kPitchCol + col]);
      aq[1] = tf32(sX[(16 * mt + g + 8) * kPitchCol + col]);
      aq[2] = tf32(sX[(16 * mt + g) * kPitchCol + col + 4]);
      aq[3] = tf32(sX[(16 * mt + g + 8) * kPitchCol + col + 4]);
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
        rec[kRecP + i * kChunk + j] = decay * acc_q[n][e];
      }
    }
  }
  __syncthreads();

  // V replaces Q; T = (I + A)^-1 by forward substitution, thread c owning column c
  load_rows<F32>(sX, kPitchCol, p.v, p.v_stride, head, tok0, p.tokens);
  if (threadIdx.x < kChunk) {
    const int c = threadIdx.x;
    float col[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      float acc0 = i == c ? 1.0F : 0.0F;
      float acc1 = 0.0F;
#pragma unroll
      for (int j = 0; j + 1 < i; j += 2) {
        acc0 -= sA[i * kPitchSq + j] * col[j];
        acc1 -= sA[i * kPitchSq + j + 1] * col[j + 1];
      }
      if (i & 1) {
        acc0 -= sA[i * kPitchSq + i - 1] * col[i - 1];
      }
      col[i] = acc0 + acc1;
      sT[i * kPitchSq + c] = col[i];
    }
  }
  __syncthreads();

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
      *reinterpret_cast<float2 *>(rec + kRecW + i * kDim + d) = make_float2(acc_w[n][0], acc_w[n][1]);
      *reinterpret_cast<float2 *>(rec + kRecW + (i + 8) * kDim + d) = make_float2(acc_w[n][2], acc_w[n][3]);
      *reinterpret_cast<float2 *>(rec + kRecU + i * kDim + d) = make_float2(acc_u[n][0], acc_u[n][1]);
      *reinterpret_cast<float2 *>(rec + kRecU + (i + 8) * kDim + d) = make_float2(acc_u[n][2], acc_u[n][3]);
    }
  }
}

// ---- apply: per (state slice, value head), chunks in order ---------------------------------------------
constexpr int kApplySmemFloats = kDim * kPitchSlice + 2 * kChunk * kPitchRow + kChunk * kPitchCol +
                                 kChunk * kPitchSq + kChunk * kPitchSlice + 2 * kChunk;

template <bool F32>
__global__ void __launch_bounds__(256, 1) gdn_chunk_apply_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) float apply_smem[];
  float *sS = apply_smem;                     // [128][40] state slice
  float *sW = sS + kDim * kPitchSlice;        // [64][132]
  float *sQ = sW + kChunk * kPitchRow;        // [64][132]
  float *sK = sQ + kChunk * kPitchRow;        // [64][136]
  float *sP = sK + kChunk * kPitchCol;        // [64][68]
  float *sD = sP + kChunk * kPitchSq;         // [64][40]  U slice, then Delta
  float *sG = sD + kChunk * kPitchSlice;      // [64]
  float *sE = sG + kChunk;                    // [64] exp(G_C - G_i)

  const std::uint32_t slice = blockIdx.x;
  const std::uint32_t head = blockIdx.y;
  const std::uint32_t key_head = head % p.key_heads;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  float *state = p.state + static_cast<std::size_t>(head) * kDim * kDim + slice * kSlice;

  load_block(sS, kPitchSlice, state, kDim, kSlice, kDim);

  for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
    const std::uint32_t tok0 = chunk * kChunk;
    const float *rec = p.workspace + (static_cast<std::size_t>(chunk) * p.value_heads + head) * kRecFloats;
    load_block(sW, kPitchRow, rec + kRecW, kChunk, kDim, kDim);
    load_rows<F32>(sQ, kPitchRow, p.q, p.q_stride, key_head, tok0, p.tokens);
    load_rows<F32>(sK, kPitchCol, p.k, p.k_stride, key_head, tok0, p.tokens);
    load_block(sP, kPitchSq, rec + kRecP, kChunk, kChunk, kChunk);
    load_block(sD, kPitchSlice, rec + kRecU + slice * kSlice, kChunk, kSlice, kDim);
    if (threadIdx.x < kChunk) {
      sG[threadIdx.x] = rec[kRecG + threadIdx.x];
    }
    __syncthreads(); // also orders the previous chunk's state update before this chunk's reads
    if (threadIdx.x < kChunk) {
      sE[threadIdx.x] = expf(sG[kChunk - 1] - sG[threadIdx.x]);
    }

    // W S0 and Q S0: 64 x 32, contraction over 128.  Warp: rows 16*(warp&3).., columns 16*(warp>>2)..
    const int mt = warp & 3;
    const int nc0 = (warp >> 2) * 16;
    float acc_w[2][4] = {};
    float acc_o[2][4] = {};
#pragma unroll 4
    for (int ks = 0; ks < 16; ++ks) {
      std::uint32_t aw[4];
      std::uint32_t aq[4];
      const int col = ks * 8 + t;
      aw[0] = tf32(sW[(16 * mt + g) * kPitchRow + col]);
      aw[1] = tf32(sW[(16 * mt + g + 8) * kPitchRow + col]);
      aw[2] = tf32(sW[(16 * mt + g) * kPitchRow + col + 4]);
      aw[3] = tf32(sW[(16 * mt + g + 8) * kPitchRow + col + 4]);
      aq[0] = tf32(sQ[(16 * mt + g) * kPitchRow + col]);
      aq[1] = tf32(sQ[(16 * mt + g + 8) * kPitchRow + col]);
      aq[2] = tf32(sQ[(16 * mt + g) * kPitchRow + col + 4]);
      aq[3] = tf32(sQ[(16 * mt + g + 8) * kPitchRow + col + 4]);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const std::uint32_t b0 = tf32(sS[col * kPitchSlice + nc0 + 8 * n + g]);
        const std::uint32_t b1 = tf32(sS[(col + 4) * kPitchSlice + nc0 + 8 * n + g]);
        mma_tf32(acc_w[n], aw, b0, b1);
        mma_tf32(acc_o[n], aq, b0, b1);
      }
    }
    // Delta = U - W S0 (in place over the U slice); the output starts as exp(G_i) * (Q S0)_i
    {
      const int i0 = 16 * mt + g;
      const float gamma0 = expf(sG[i0]);
      const float gamma1 = expf(sG[i0 + 8]);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int c = nc0 + 8 * n + 2 * t;
        sD[i0 * kPitchSlice + c] -= acc_w[n][0];
        sD[i0 * kPitchSlice + c + 1] -= acc_w[n][1];
        sD[(i0 + 8) * kPitchSlice + c] -= acc_w[n][2];
        sD[(i0 + 8) * kPitchSlice + c + 1] -= acc_w[n][3];
        acc_o[n][0] *= gamma0;
        acc_o[n][1] *= gamma0;
        acc_o[n][2] *= gamma1;
        acc_o[n][3] *= gamma1;
      }
    }
    __syncthreads();

    // O += P Delta: 64 x 32, contraction over the 64 tokens (P is lower triangular: stop at the diagonal tile)
    for (int ks = 0; ks < 2 * mt + 2; ++ks) {
      std::uint32_t a[4];
      const int col = ks * 8 + t;
      a[0] = tf32(sP[(16 * mt + g) * kPitchSq + col]);
      a[1] = tf32(sP[(16 * mt + g + 8) * kPitchSq + col]);
      a[2] = tf32(sP[(16 * mt + g) * kPitchSq + col + 4]);
      a[3] = tf32(sP[(16 * mt + g + 8) * kPitchSq + col + 4]);
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const std::uint32_t b0 = tf32(sD[col * kPitchSlice + nc0 + 8 * n + g]);
        const std::uint32_t b1 = tf32(sD[(col + 4) * kPitchSlice + nc0 + 8 * n + g]);
        mma_tf32(acc_o[n], a, b0, b1);
      }
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

    // S = exp(G_C) S + K^T (diag(exp(G_C - G)) Delta): 128 x 32, contraction over the 64 tokens.
    // Warp: state rows 16*warp.., all 32 columns.
    {
      const float gamma_c = expf(sG[kChunk - 1]);
      float acc[4][4];
      const int r0 = 16 * warp + g;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int c = 8 * n + 2 * t;
        acc[n][0] = sS[r0 * kPitchSlice + c] * gamma_c;
        acc[n][1] = sS[r0 * kPitchSlice + c + 1] * gamma_c;
        acc[n][2] = sS[(r0 + 8) * kPitchSlice + c] * gamma_c;
        acc[n][3] = sS[(r0 + 8) * kPitchSlice + c + 1] * gamma_c;
      }
#pragma unroll 2
      for (int ks = 0; ks < 8; ++ks) {
        std::uint32_t a[4];
        const int tok = ks * 8 + t;
        a[0] = tf32(sK[tok * kPitchCol + 16 * warp + g]);
        a[1] = tf32(sK[tok * kPitchCol + 16 * warp + g + 8]);
        a[2] = tf32(sK[(tok + 4) * kPitchCol + 16 * warp + g]);
        a[3] = tf32(sK[(tok + 4) * kPitchCol + 16 * warp + g + 8]);
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
        sS[r0 * kPitchSlice + c] = acc[n][0];
        sS[r0 * kPitchSlice + c + 1] = acc[n][1];
        sS[(r0 + 8) * kPitchSlice + c] = acc[n][2];
        sS[(r0 + 8) * kPitchSlice + c + 1] = acc[n][3];
      }
    }
    __syncthreads(); // the chunk's operands may now be overwritten
  }

  for (int i = threadIdx.x; i < kDim * (kSlice / 4); i += 256) {
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
    cuda_ok(cudaFuncSetAttribute(gdn_chunk_apply_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kApplySmemFloats * 4),
            "gated-delta apply shared-memory opt-in");
  });
}

template <bool F32> void launch(const ChunkParams &params, cudaStream_t stream) {
  configure_once<F32>();
  gdn_chunk_prepare_kernel<F32>
      <<<dim3(params.chunks, params.value_heads), 256, kPrepSmemFloats * 4, stream>>>(params);
  cuda_ok(cudaGetLastError(), "gated-delta prepare launch");
  gdn_chunk_apply_kernel<F32>
      <<<dim3(kDim / kSlice, params.value_heads), 256, kApplySmemFloats * 4, stream>>>(params);
  cuda_ok(cudaGetLastError(), "gated-delta apply launch");
}

} // namespace

std::size_t gdn_chunk_workspace_bytes(std::size_t tokens, std::size_t key_heads, std::size_t value_heads) {
  (void)key_heads;
  const std::size_t chunks = ceil_div(tokens, kChunk, "gated-delta chunk count overflows");
  return mul(mul(chunks, value_heads, "gated-delta chunk workspace overflows"), kRecFloats * sizeof(float),
             "gated-delta chunk workspace overflows");
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
  if (a.qkv_f32) {
    launch<true>(p, stream);
  } else {
    launch<false>(p, stream);
  }
}

} // namespace rib200
