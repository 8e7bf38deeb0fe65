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
// dense products on mma.sync TF32 tensor-core tiles; it leaves every operand the apply kernel multiplies with as a
// ready shared-memory image (K-major, 128-byte swizzle) in the workspace.  `apply` walks the chunks in order for one
// (value head, 32-column slice of the state): the slice lives in registers (FP32) and, rounded to TF32, in shared
// memory as the B operand; [Q; W] S0, P Delta and K^T diag(e) Delta are tcgen05.mma.kind::tf32 products with
// accumulators in tensor memory.  State columns are independent, so the four slices of a head never talk to each
// other.  TF32 (10-bit mantissa, FP32 accumulate) rather than BF16 keeps the FP32 state within 1e-3 relative L2 of
// the sequential recurrence over 64 chunks.
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
// Workspace record of one (chunk, value head), in bytes.  A1, A2 and A3 are images of tcgen05 shared-memory
// operands: K-major, 32 TF32 elements (128 bytes) per row and k-block, [k-block][row][128 bytes], the 16-byte chunk
// index of a row XORed with row % 8 (SWIZZLE_128B).
constexpr std::uint32_t kRowBytes = 128;
constexpr std::uint32_t kA1Block = 128 * kRowBytes;               // rows 0..63 Q, rows 64..127 W; 4 k-blocks
constexpr std::uint32_t kA1Bytes = 4 * kA1Block;
constexpr std::uint32_t kA2Block = kChunk * kRowBytes;            // P, 64 rows; 2 k-blocks
constexpr std::uint32_t kA2Bytes = 2 * kA2Block;
constexpr std::uint32_t kA3Block = kDim * kRowBytes;              // (K diag(e))^T, 128 rows; 2 k-blocks
constexpr std::uint32_t kA3Bytes = 2 * kA3Block;
constexpr int kPitchU = 36;                                        // U slice [64][36] FP32, then gamma [64]
constexpr std::uint32_t kUBytes = (kChunk * kPitchU + kChunk) * 4;
constexpr std::uint32_t kRecA1 = 0;
constexpr std::uint32_t kRecA2 = kRecA1 + kA1Bytes;
constexpr std::uint32_t kRecA3 = kRecA2 + kA2Bytes;
constexpr std::uint32_t kRecU = kRecA3 + kA3Bytes;                // [4 slices] of kUBytes
constexpr std::uint32_t kRecBytes = kRecU + (kDim / kSlice) * kUBytes;
static_assert(kRecBytes % 16 == 0 && kUBytes % 16 == 0, "16-byte blocks");

// Byte offset of element (row, k) inside an operand image whose k-blocks are block_bytes apart.
__host__ __device__ constexpr std::uint32_t image_offset(std::uint32_t row, std::uint32_t k, std::uint32_t block_bytes) {
  return (k >> 5) * block_bytes + row * kRowBytes + ((((k & 31U) >> 2) ^ (row & 7U)) << 4) + ((k & 3U) << 2);
}

struct ChunkParams {
  const void *q, *k, *v;
  std::size_t q_stride, k_stride, v_stride;
  const float *beta;
  const float *log_decay;
  float *state;
  float *out;
  unsigned char *workspace;
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
// into registers (zeros at or past `tokens`), store_rows converts and writes them.  256 threads, four per row.
// The four threads of a row take 8-element pieces in turn (piece 4 a + part for a = 0..3), so that the 16-byte
// stores of a quarter-warp (two rows) fall into 32 different banks at a pitch of 4 mod 32 words.
template <bool F32> struct RowRegs {
  uint4 v[F32 ? 8 : 4];
};

template <bool F32>
__device__ __forceinline__ RowRegs<F32> fetch_rows(const void *src, std::size_t stride, std::uint32_t head,
                                                   std::uint32_t tok0, std::uint32_t tokens) {
  RowRegs<F32> regs;
  const int row = threadIdx.x >> 2;
  const int part = threadIdx.x & 3;
  const std::uint32_t tok = tok0 + row;
  constexpr int kVectors = F32 ? 8 : 4;
  if (tok >= tokens) {
#pragma unroll
    for (int i = 0; i < kVectors; ++i) {
      regs.v[i] = make_uint4(0U, 0U, 0U, 0U);
    }
    return regs;
  }
  const std::size_t base = static_cast<std::size_t>(tok) * stride + head * kDim + part * 8;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    if constexpr (F32) {
      const uint4 *s = reinterpret_cast<const uint4 *>(static_cast<const float *>(src) + base + 32 * a);
      regs.v[2 * a] = s[0];
      regs.v[2 * a + 1] = s[1];
    } else {
      regs.v[a] = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(src) + base + 32 * a);
    }
  }
  return regs;
}

template <bool F32> __device__ __forceinline__ void store_rows(float *dst, int pitch, const RowRegs<F32> &regs) {
  const int row = threadIdx.x >> 2;
  const int part = threadIdx.x & 3;
  float *d = dst + row * pitch + part * 8;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    if constexpr (F32) {
      *reinterpret_cast<uint4 *>(d + 32 * a) = regs.v[2 * a];
      *reinterpret_cast<uint4 *>(d + 32 * a + 4) = regs.v[2 * a + 1];
    } else {
      const std::uint32_t w[4] = {regs.v[a].x, regs.v[a].y, regs.v[a].z, regs.v[a].w};
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
      *reinterpret_cast<float4 *>(d + 32 * a) = lo;
      *reinterpret_cast<float4 *>(d + 32 * a + 4) = hi;
    }
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
constexpr int kPrepSmemFloats = kChunk * kPitchRow + kChunk * kPitchCol + 2 * kChunk * kPitchSq + 4 * kChunk;

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
  float *sE = sBg + kChunk;                   // [64] exp(G_C - G)

  const std::uint32_t chunk = blockIdx.x;
  const std::uint32_t head = blockIdx.y;
  const std::uint32_t key_head = head % p.key_heads;
  const std::uint32_t tok0 = chunk * kChunk;
  unsigned char *rec = p.workspace + (static_cast<std::size_t>(chunk) * p.value_heads + head) * kRecBytes;
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
  // Q rows of the [Q; W] operand image, rounded to TF32 (zero rows past the last token)
  for (int i = threadIdx.x; i < kChunk * (kDim / 4); i += 256) {
    const int r = i / (kDim / 4);
    const int c = (i % (kDim / 4)) * 4;
    const float4 qv = *reinterpret_cast<const float4 *>(sX + r * kPitchRow + c);
    *reinterpret_cast<float4 *>(rec + kRecA1 + image_offset(r, c, kA1Block)) =
        make_float4(__uint_as_float(tf32(qv.x)), __uint_as_float(tf32(qv.y)), __uint_as_float(tf32(qv.z)),
                    __uint_as_float(tf32(qv.w)));
  }
  if (threadIdx.x < kChunk) {
    const float gamma = expf(sG[threadIdx.x]);
    sBg[threadIdx.x] = sBeta[threadIdx.x] * gamma;
    sE[threadIdx.x] = expf(sG[kChunk - 1] - sG[threadIdx.x]);
#pragma unroll
    for (int slice = 0; slice < kDim / kSlice; ++slice) {
      reinterpret_cast<float *>(rec + kRecU + slice * kUBytes)[kChunk * kPitchU + threadIdx.x] = gamma;
    }
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
      for (int half = 0; half < 2; ++half) {
        const int i = 16 * mt + g + half * 8;
        const int j0 = 8 * (nt0 + n) + 2 * t;
        float pv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = j0 + e;
          const float decay = j <= i ? __expf(sG[i] - sG[j]) : 0.0F;
          sA[i * kPitchSq + j] = j < i ? sBeta[i] * decay * acc_k[n][2 * half + e] : 0.0F;
          pv[e] = __uint_as_float(tf32(decay * acc_q[n][2 * half + e]));
        }
        *reinterpret_cast<float2 *>(rec + kRecA2 + image_offset(i, j0, kA2Block)) = make_float2(pv[0], pv[1]);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 3);
  }

  // V replaces Q; T = (I + A)^-1 by forward substitution in FP32.
  const RowRegs<F32> v_regs = fetch_rows<F32>(p.v, p.v_stride, head, tok0, p.tokens); // lands during the substitution
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 4);
  }
  if (threadIdx.x < kChunk) {
    // Two warps, a column of T per thread, all of it in registers: row i costs i multiply-adds in four
    // independent chains and no exchange between lanes; only the term with T[i-1] waits for the row before.
    const int c = threadIdx.x;
    float tcol[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      tcol[i] = 0.0F;
    }
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      float acc0 = 0.0F;
      float acc1 = 0.0F;
      float acc2 = 0.0F;
      float acc3 = 0.0F;
#pragma unroll
      for (int j = 0; j < i; j += 4) { // A is zero on and above the diagonal, entries not yet known are zero
        const float4 a = *reinterpret_cast<const float4 *>(sA + i * kPitchSq + j);
        acc0 -= a.x * tcol[j];
        acc1 -= a.y * tcol[j + 1];
        acc2 -= a.z * tcol[j + 2];
        acc3 -= a.w * tcol[j + 3];
      }
      tcol[i] = (i == c ? 1.0F : 0.0F) + ((acc0 + acc1) + (acc2 + acc3));
    }
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      sT[i * kPitchSq + c] = tcol[i];
    }
    if (threadIdx.x == 0 && blockIdx.x == 0) {
      RIB200_GDN_STAMP(127, 7);
    }
  } else {
    // The other six warps meanwhile: their share of V, and the (K diag(e))^T operand image (row = key dim,
    // k = token).  A thread gathers four tokens of one dim from sK; a warp covers 16 dims x 2 token quads per item,
    // which reads 32 different banks and writes whole 32-byte sectors.
    store_rows<F32>(sX, kPitchCol, v_regs);
    for (int item = warp - 2; item < 64; item += 6) {
      const int d = 16 * (item & 7) + (lane & 15);
      const int j = 4 * (2 * (item >> 3) + (lane >> 4));
      const float4 e4 = *reinterpret_cast<const float4 *>(sE + j);
      *reinterpret_cast<float4 *>(rec + kRecA3 + image_offset(d, j, kA3Block)) =
          make_float4(__uint_as_float(tf32(sK[j * kPitchRow + d] * e4.x)),
                      __uint_as_float(tf32(sK[(j + 1) * kPitchRow + d] * e4.y)),
                      __uint_as_float(tf32(sK[(j + 2) * kPitchRow + d] * e4.z)),
                      __uint_as_float(tf32(sK[(j + 3) * kPitchRow + d] * e4.w)));
    }
    if (threadIdx.x == 64 && blockIdx.x == 0) {
      RIB200_GDN_STAMP(127, 8);
    }
  }
  if (threadIdx.x < kChunk) {
    store_rows<F32>(sX, kPitchCol, v_regs);
  }
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
      *reinterpret_cast<float2 *>(rec + kRecA1 + image_offset(kChunk + i, d, kA1Block)) =
          make_float2(__uint_as_float(tf32(acc_w[n][0])), __uint_as_float(tf32(acc_w[n][1])));
      *reinterpret_cast<float2 *>(rec + kRecA1 + image_offset(kChunk + i + 8, d, kA1Block)) =
          make_float2(__uint_as_float(tf32(acc_w[n][2])), __uint_as_float(tf32(acc_w[n][3])));
      float *u = reinterpret_cast<float *>(rec + kRecU + (d / kSlice) * kUBytes) + d % kSlice;
      *reinterpret_cast<float2 *>(u + i * kPitchU) = make_float2(acc_u[n][0], acc_u[n][1]);
      *reinterpret_cast<float2 *>(u + (i + 8) * kPitchU) = make_float2(acc_u[n][2], acc_u[n][3]);
    }
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    RIB200_GDN_STAMP(127, 6);
  }
}

// ---- apply: per (state slice, value head), chunks in order ---------------------------------------------
// 192 threads.  Warps 0-3 own the 128 lanes of tensor memory (thread = row of every product), warp 4 issues the
// tcgen05 products (whole warp in step, one elected lane issuing), lane 0 of warp 5 streams the operand images of
// each chunk into shared memory with bulk copies counted on mbarriers.  Per chunk:
//   X  = [Q; W] S0            M 128 (rows 0..63 Q S0, rows 64..127 W S0), N 32, K 128
//   warps 2-3: Delta = U - X[64..]  ->  B operand (TF32);   warps 0-1: keep gamma_i (Q S0)_i
//   SD = (K diag(e))^T Delta  M 128, N 32, K 64
//   O2 = P Delta              M 128 (rows 64..127 are don't-care), N 32, K 64
//   all: S = gamma_C S + SD (FP32 registers) -> B operand (TF32): the next chunk's first product waits for this
//   warps 0-1: O = gamma_i (Q S0)_i + O2, each row through shared memory and out with a bulk copy
// Every mbarrier wait is bounded; when one runs out the CTA records RIB200_DEVICE_WAIT_TIMED_OUT, stops waiting
// and copying, and runs to its end (its results are then meaningless, as the status word says).
constexpr int kApplyThreads = 192;
constexpr std::uint32_t kSmA1 = 0;                         // two stages of the [Q; W] image
constexpr std::uint32_t kSmA23 = kSmA1 + 2 * kA1Bytes;     // P image, then the (K diag(e))^T image
constexpr std::uint32_t kSmB1 = kSmA23 + kA2Bytes + kA3Bytes; // S^T, [4 k-blocks][32 rows][128 bytes]
constexpr std::uint32_t kB1Block = kSlice * kRowBytes;
constexpr std::uint32_t kSmBD = kSmB1 + 4 * kB1Block;      // Delta^T, [2 k-blocks][32 rows][128 bytes]
constexpr std::uint32_t kSmU = kSmBD + 2 * kB1Block;       // two stages of U slice + gamma
constexpr std::uint32_t kUStage = 10240;                   // stage stride: the output tile that reuses a stage wants 1 KiB alignment
constexpr std::uint32_t kSmBars = kSmU + 2 * kUStage;
enum : std::uint32_t {
  kBarA1Full = 0,   // [2] bytes of a [Q; W] image
  kBarA1Empty = 2,  // [2] the product that read it has completed
  kBarA23Full = 4,
  kBarA23Empty = 5,
  kBarUFull = 6,    // [2]
  kBarUEmpty = 8,   // [2] 128 readers
  kBarXDone = 10,   // X is in tensor memory
  kBarDReady = 11,  // Delta^T is in shared memory (64 writers)
  kBarSdDone = 12,  // SD is in tensor memory
  kBarSReady = 13,  // S^T is in shared memory, X and SD have been read (128 threads)
  kBarO2Done = 14,  // O2 is in tensor memory
  kBarO2Free = 15,  // O2 has been read (64 threads)
  kBarCount = 16
};
constexpr std::uint32_t kSmTmemSlot = kSmBars + kBarCount * 8;
constexpr std::uint32_t kSmAbort = kSmTmemSlot + 4;
constexpr std::uint32_t kApplySmemBytes = kSmAbort + 4 + 1024; // + room to align the base to 1 KiB
static_assert(kUStage >= kUBytes && kSmA23 % 1024 == 0 && kSmB1 % 1024 == 0 && kSmBD % 1024 == 0 && kSmU % 1024 == 0 &&
                  kSmBars % 8 == 0,
              "operand images sit on 1 KiB boundaries");
static_assert(kApplySmemBytes <= 232448, "apply kernel exceeds the shared memory of an SM");
constexpr long long kWaitLimitCycles = 1LL << 28;
constexpr std::uint32_t kTmemColumns = 128; // X at 0, O2 at 32, SD at 64
constexpr std::uint32_t kPrefetchAhead = 3;   // chunks between an L2 prefetch and the copy that uses it
constexpr std::uint32_t kCopyPiece = 16384;  // the operand images come in as several bulk copies in flight at once

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
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ bool elect_one() {
  std::uint32_t chosen;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "elect.sync _|p, 0xFFFFFFFF;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(chosen));
  return chosen != 0;
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1 KiB apart, descriptor version 1.
__device__ __forceinline__ std::uint64_t smem_desc(std::uint32_t addr) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((addr & 0x3FFFFU) >> 4);
  d |= static_cast<std::uint64_t>(1) << 16;            // leading-dimension offset: unused by this layout
  d |= static_cast<std::uint64_t>(1024 >> 4) << 32;    // stride between 8-row groups
  d |= static_cast<std::uint64_t>(1) << 46;            // version
  d |= static_cast<std::uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}
// Instruction descriptor: TF32 x TF32 -> FP32, both operands K-major, M 128, N 32.
constexpr std::uint32_t kIdesc = (1U << 4) | (2U << 7) | (2U << 10) | (static_cast<std::uint32_t>(kSlice >> 3) << 17) |
                                 (static_cast<std::uint32_t>(128 >> 4) << 24);
__device__ __forceinline__ void umma_tf32(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                          std::uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_commit(std::uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(std::uint32_t taddr, float (&v)[32]) {
  std::uint32_t r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                 "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                 "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                 "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __uint_as_float(r[i]);
  }
}
__device__ __forceinline__ void sts32(std::uint32_t addr, std::uint32_t value) {
  asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(addr), "r"(value) : "memory");
}
// Shared-memory loads by 32-bit shared address: unlike loads through a generic pointer they are known not to
// alias global stores, so a run of them is issued back to back.
__device__ __forceinline__ void sts128(std::uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float lds32(std::uint32_t addr) {
  float value;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(value) : "r"(addr));
  return value;
}
__device__ __forceinline__ float4 lds128(std::uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

__global__ void __launch_bounds__(kApplyThreads, 1)
    gdn_chunk_apply_kernel(const ChunkParams p, const __grid_constant__ TensorMapBytes out_map) {
  extern __shared__ unsigned char apply_smem_raw[];
  const std::uint32_t base = (smem_address(apply_smem_raw) + 1023U) & ~1023U;
  unsigned char *smem = apply_smem_raw + (base - smem_address(apply_smem_raw));
  const std::uint32_t bars = base + kSmBars;
  auto bar = [&](std::uint32_t index) { return bars + index * 8; };
  volatile std::uint32_t *tmem_slot = reinterpret_cast<volatile std::uint32_t *>(smem + kSmTmemSlot);
  volatile std::uint32_t *abort_flag = reinterpret_cast<volatile std::uint32_t *>(smem + kSmAbort);

  const std::uint32_t slice = blockIdx.x;
  const std::uint32_t head = blockIdx.y;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  float *state = p.state + static_cast<std::size_t>(head) * kDim * kDim + slice * kSlice;

  if (threadIdx.x == 0) {
    for (std::uint32_t i = 0; i < kBarCount; ++i) {
      std::uint32_t count = 1;
      if (i == kBarSReady) {
        count = 128;
      } else if (i == kBarUEmpty || i == kBarUEmpty + 1) {
        count = 65; // the 64 readers of U rows, and thread 0 once the output tile has left the stage
      } else if (i == kBarDReady || i == kBarO2Free) {
        count = 64;
      }
      mbarrier_init(bar(i), count);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(base + kSmTmemSlot),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }

  // State slice: row `key` of S in this thread's registers (FP32), S^T rounded to TF32 as the B operand.
  float s_reg[kSlice];
  const std::uint32_t key = threadIdx.x; // warps 0-3
  // element (n, k) of a B operand image with 32-row k-blocks
  auto b_offset = [](std::uint32_t n, std::uint32_t k) { return image_offset(n, k, kB1Block); };
  if (warp < 4) {
#pragma unroll
    for (int c = 0; c < kSlice; c += 4) {
      const float4 v = *reinterpret_cast<const float4 *>(state + static_cast<std::size_t>(key) * kDim + c);
      s_reg[c] = v.x;
      s_reg[c + 1] = v.y;
      s_reg[c + 2] = v.z;
      s_reg[c + 3] = v.w;
    }
#pragma unroll
    for (int n = 0; n < kSlice; ++n) {
      sts32(base + kSmB1 + b_offset(n, key), tf32(s_reg[n]));
    }
    fence_proxy_async();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const std::uint32_t tmem = *tmem_slot;

  // bounded wait; once the CTA has given up nobody waits any more
  auto wait = [&](std::uint32_t b, std::uint32_t parity) {
    if (*abort_flag != 0 || mbarrier_try_wait(b, parity)) {
      return;
    }
    const long long started = clock64();
    while (!mbarrier_try_wait(b, parity)) {
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

  if (warp == 5) {
    // ---- producer: three bulk copies per chunk ----
    if (lane == 0) {
      std::uint32_t issued[5] = {0, 0, 0, 0, 0}; // A1 stage 0/1, A23, U stage 0/1
      for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
        const unsigned char *rec =
            p.workspace + (static_cast<std::size_t>(chunk) * p.value_heads + head) * kRecBytes;
        const std::uint32_t s = chunk & 1U;
        if (slice == (chunk & 3U) && chunk + kPrefetchAhead < p.chunks) {
          // Pull a later chunk's images into L2 (the four slices of a head take turns): the copies below then hit L2.
          const unsigned char *ahead = rec + static_cast<std::size_t>(kPrefetchAhead) * p.value_heads * kRecBytes;
#pragma unroll
          for (std::uint32_t part = 0; part < kRecU; part += kCopyPiece) {
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(ahead + part), "r"(kCopyPiece) : "memory");
          }
        }
        if (chunk >= 2) {
          wait(bar(kBarA1Empty + s), ((chunk >> 1) - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        mbarrier_expect_tx(bar(kBarA1Full + s), kA1Bytes);
#pragma unroll
        for (std::uint32_t part = 0; part < kA1Bytes; part += kCopyPiece) {
          bulk_copy_g2s(base + kSmA1 + s * kA1Bytes + part, rec + kRecA1 + part, kCopyPiece, bar(kBarA1Full + s));
        }
        ++issued[s];
        if (chunk >= 2) {
          wait(bar(kBarUEmpty + s), ((chunk >> 1) - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        fence_proxy_async(); // the readers of this stage used ordinary loads
        mbarrier_expect_tx(bar(kBarUFull + s), kUBytes);
        bulk_copy_g2s(base + kSmU + s * kUStage, rec + kRecU + slice * kUBytes, kUBytes, bar(kBarUFull + s));
        ++issued[3 + s];
        if (chunk >= 1) {
          wait(bar(kBarA23Empty), (chunk - 1) & 1U);
        }
        if (*abort_flag != 0) {
          break;
        }
        mbarrier_expect_tx(bar(kBarA23Full), kA2Bytes + kA3Bytes);
#pragma unroll
        for (std::uint32_t part = 0; part < kA2Bytes + kA3Bytes; part += kCopyPiece) {
          bulk_copy_g2s(base + kSmA23 + part, rec + kRecA2 + part, kCopyPiece, bar(kBarA23Full));
        }
        ++issued[2];
      }
      // after giving up: let the copies already issued land before the CTA's shared memory goes away
      if (*abort_flag != 0) {
        const std::uint32_t full_bars[5] = {bar(kBarA1Full), bar(kBarA1Full + 1), bar(kBarA23Full), bar(kBarUFull),
                                            bar(kBarUFull + 1)};
        for (int b = 0; b < 5; ++b) {
          if (issued[b] > 0) {
            const std::uint32_t parity = (issued[b] - 1) & 1U;
            const long long started = clock64();
            while (!mbarrier_try_wait(full_bars[b], parity) && clock64() - started < kWaitLimitCycles) {
            }
          }
        }
      }
    }
  } else if (warp == 4) {
    // ---- tensor-core issue: the whole warp walks the chunks, one elected lane issues ----
    const bool issuer = elect_one();
    const std::uint64_t b1_desc = smem_desc(base + kSmB1);
    const std::uint64_t bd_desc = smem_desc(base + kSmBD);
    const std::uint64_t a2_desc = smem_desc(base + kSmA23);
    const std::uint64_t a3_desc = smem_desc(base + kSmA23 + kA2Bytes);
    // descriptor address field counts 16-byte units: a k-step inside a k-block is 32 bytes = 2 units
    auto step = [](std::uint32_t ks, std::uint32_t block_bytes) {
      return static_cast<std::uint64_t>(((ks >> 2) * block_bytes + (ks & 3U) * 32U) >> 4);
    };
    for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
      const std::uint32_t s = chunk & 1U;
      wait(bar(kBarA1Full + s), (chunk >> 1) & 1U);
      if (chunk >= 1) {
        wait(bar(kBarSReady), (chunk - 1) & 1U);
      }
      tcgen05_fence_after();
      if (issuer) {
        RIB200_GDN_STAMP(chunk, 5);
      }
      if (issuer && *abort_flag == 0) {
        const std::uint64_t a1_desc = smem_desc(base + kSmA1 + s * kA1Bytes);
#pragma unroll
        for (std::uint32_t ks = 0; ks < 16; ++ks) {
          umma_tf32(tmem, a1_desc + step(ks, kA1Block), b1_desc + step(ks, kB1Block), ks);
        }
        umma_commit(bar(kBarXDone));
        umma_commit(bar(kBarA1Empty + s));
      }
      __syncwarp();
      wait(bar(kBarDReady), chunk & 1U);
      if (issuer) {
        RIB200_GDN_STAMP(chunk, 6);
      }
      wait(bar(kBarA23Full), chunk & 1U);
      if (issuer) {
        RIB200_GDN_STAMP(chunk, 7);
      }
      tcgen05_fence_after();
      if (issuer && *abort_flag == 0) {
#pragma unroll
        for (std::uint32_t ks = 0; ks < 8; ++ks) {
          umma_tf32(tmem + 64, a3_desc + step(ks, kA3Block), bd_desc + step(ks, kB1Block), ks);
        }
        umma_commit(bar(kBarSdDone));
      }
      __syncwarp();
      if (chunk >= 1) {
        wait(bar(kBarO2Free), (chunk - 1) & 1U);
      }
      tcgen05_fence_after();
      if (issuer && *abort_flag == 0) {
#pragma unroll
        for (std::uint32_t ks = 0; ks < 8; ++ks) {
          umma_tf32(tmem + 32, a2_desc + step(ks, kA2Block), bd_desc + step(ks, kB1Block), ks);
        }
        umma_commit(bar(kBarO2Done));
        umma_commit(bar(kBarA23Empty));
      }
      __syncwarp();
      if (*abort_flag != 0) {
        break;
      }
    }
  } else {
    // ---- warps 0-3: thread = lane of tensor memory ----
    const std::uint32_t lane_base = static_cast<std::uint32_t>(warp * 32) << 16;
    const bool upper = warp >= 2;                  // rows 64..127 of X: W S0 of token threadIdx.x - 64
    const std::uint32_t token = threadIdx.x & 63U; // the token this thread serves in X and O2
    for (std::uint32_t chunk = 0; chunk < p.chunks; ++chunk) {
      const std::uint32_t s = chunk & 1U;
      const std::uint32_t u_stage = base + kSmU + s * kUStage; // U slice [64][36] FP32, then gamma [64]
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 0);
      }
      wait(bar(kBarUFull + s), (chunk >> 1) & 1U);
      wait(bar(kBarXDone), chunk & 1U);
      tcgen05_fence_after();
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 1);
      }
      if (threadIdx.x == 64) {
        RIB200_GDN_STAMP(chunk, 12);
      }
      float x[kSlice];
      tmem_ld32(tmem + lane_base, x);
      if (threadIdx.x == 64) {
        RIB200_GDN_STAMP(chunk, 14);
      }
      const float gamma_c = lds32(u_stage + (kChunk * kPitchU + kChunk - 1) * 4);
      if (upper) {
        // Delta = U - W S0, written as the B operand of the two products that follow.  All loads first, then the
        // arithmetic, then the stores: the store helper is a compiler barrier for memory accesses.
        float4 u[kSlice / 4];
#pragma unroll
        for (int c = 0; c < kSlice / 4; ++c) {
          u[c] = lds128(u_stage + (token * kPitchU + 4 * c) * 4);
        }
        std::uint32_t d[kSlice];
#pragma unroll
        for (int c = 0; c < kSlice / 4; ++c) {
          d[4 * c] = tf32(u[c].x - x[4 * c]);
          d[4 * c + 1] = tf32(u[c].y - x[4 * c + 1]);
          d[4 * c + 2] = tf32(u[c].z - x[4 * c + 2]);
          d[4 * c + 3] = tf32(u[c].w - x[4 * c + 3]);
        }
#pragma unroll
        for (int n = 0; n < kSlice; ++n) {
          sts32(base + kSmBD + b_offset(n, token), d[n]);
        }
        if (threadIdx.x == 64) {
          RIB200_GDN_STAMP(chunk, 15);
        }
        fence_proxy_async();
        tcgen05_fence_before();
        mbarrier_arrive(bar(kBarDReady));
        if (threadIdx.x == 64) {
          RIB200_GDN_STAMP(chunk, 13);
        }
        mbarrier_arrive(bar(kBarUEmpty + s)); // the lower half hands the stage back after using it for the output
      } else {
        const float gamma = lds32(u_stage + (kChunk * kPitchU + token) * 4);
#pragma unroll
        for (int c = 0; c < kSlice; ++c) {
          x[c] *= gamma;
        }
      }
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 2);
      }

      wait(bar(kBarSdDone), chunk & 1U);
      tcgen05_fence_after();
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 3);
      }
      {
        float sd[kSlice];
        tmem_ld32(tmem + lane_base + 64, sd);
        std::uint32_t rounded[kSlice];
#pragma unroll
        for (int n = 0; n < kSlice; ++n) {
          s_reg[n] = s_reg[n] * gamma_c + sd[n];
          rounded[n] = tf32(s_reg[n]);
        }
#pragma unroll
        for (int n = 0; n < kSlice; ++n) {
          sts32(base + kSmB1 + b_offset(n, key), rounded[n]);
        }
      }
      fence_proxy_async();
      tcgen05_fence_before();
      mbarrier_arrive(bar(kBarSReady));
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 4);
      }
      if (!upper) {
        // O = gamma_i (Q S0)_i + (P Delta)_i; the thread owns a row.
        wait(bar(kBarO2Done), chunk & 1U);
        tcgen05_fence_after();
        if (threadIdx.x == 0) {
          RIB200_GDN_STAMP(chunk, 8);
        }
        float o2[kSlice];
        tmem_ld32(tmem + lane_base + 32, o2);
        tcgen05_fence_before();
        mbarrier_arrive(bar(kBarO2Free));
        // The 64 x 32 tile goes through the U stage (dead since the Delta step) in the 128-byte-swizzled layout of
        // the output's tensor map, and out with one tiled bulk store; rows past the last token are clipped by it.
#pragma unroll
        for (std::uint32_t c = 0; c < kSlice / 4; ++c) {
          sts128(u_stage + token * kRowBytes + ((c ^ (token & 7U)) << 4), x[4 * c] + o2[4 * c],
                 x[4 * c + 1] + o2[4 * c + 1], x[4 * c + 2] + o2[4 * c + 2], x[4 * c + 3] + o2[4 * c + 3]);
        }
        fence_proxy_async();
        asm volatile("bar.sync 1, 64;\n" ::: "memory");
        if (threadIdx.x == 0) {
          if (*abort_flag == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n" ::"l"(
                             reinterpret_cast<std::uint64_t>(&out_map)),
                         "r"(static_cast<int>(head * kDim + slice * kSlice)), "r"(static_cast<int>(chunk * kChunk)),
                         "r"(u_stage)
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
          RIB200_GDN_STAMP(chunk, 9);
          asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); // the tile has been read
          mbarrier_arrive(bar(kBarUEmpty + s));
        }
      }
      if (threadIdx.x == 0) {
        RIB200_GDN_STAMP(chunk, 11);
      }
      if (*abort_flag != 0) {
        break;
      }
    }
#pragma unroll
    for (int c = 0; c < kSlice; c += 4) {
      *reinterpret_cast<float4 *>(state + static_cast<std::size_t>(key) * kDim + c) =
          make_float4(s_reg[c], s_reg[c + 1], s_reg[c + 2], s_reg[c + 3]);
    }
  }

  // every role comes here; the products issued so far have completed or the CTA has given up waiting for them
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 4) {
    // warps 0-3 waited for the last commit, so nothing is still writing tensor memory
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemColumns) : "memory");
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
  TensorMapBytes out_map;
  encode_f32_rows_map(&out_map, params.out, static_cast<std::uint64_t>(params.value_heads) * kDim, params.tokens,
                      kSlice, kChunk);
  gdn_chunk_apply_kernel<<<dim3(kDim / kSlice, params.value_heads), kApplyThreads, kApplySmemBytes, stream>>>(
      params, out_map);
  cuda_ok(cudaGetLastError(), "gated-delta apply launch");
}

} // namespace

#ifdef RIB200_TRACE
extern "C" int rib200_debug_read_gdn_trace(long long *host, std::size_t count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_gdn_trace, count * sizeof(long long)));
}
#endif

std::size_t gdn_chunk_workspace_bytes(std::size_t tokens, std::size_t key_heads, std::size_t value_heads) {
  (void)key_heads;
  const std::size_t chunks = ceil_div(tokens, kChunk, "gated-delta chunk count overflows");
  return mul(mul(chunks, value_heads, "gated-delta chunk workspace overflows"), kRecBytes,
             "gated-delta chunk workspace overflows");
}

void launch_gdn_chunked(const GdnCoreArgs &a, void *workspace, cudaStream_t stream) {
  require(workspace != nullptr, "gated-delta chunked prefill needs its workspace");
  require(reinterpret_cast<std::uintptr_t>(workspace) % 16 == 0, "gated-delta chunk workspace is not 16-byte aligned");
  require(reinterpret_cast<std::uintptr_t>(a.out) % 16 == 0 && reinterpret_cast<std::uintptr_t>(a.state) % 16 == 0,
          "gated-delta chunked prefill: output and state must be 16-byte aligned");
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
  p.workspace = static_cast<unsigned char *>(workspace);
  p.tokens = a.tokens;
  p.chunks = (a.tokens + kChunk - 1) / kChunk;
  p.key_heads = a.key_heads;
  p.value_heads = a.value_heads;
  p.status = device_status_word();
  if (a.qkv_f32) {
    launch<true>(p, stream);
  } else {
    launch<false>(p, stream);
  }
}

} // namespace rib200
