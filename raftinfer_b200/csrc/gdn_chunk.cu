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
// Two kernels, both on tcgen05 TF32 products with accumulators in tensor memory.  `prepare` is parallel over
// (chunk, value head), one persistent CTA per SM: the raw K, Q, V rows of an item arrive by tensor-map copies issued
// while the item before it is in its last third (into areas of shared memory that are idle by then); [K; Q] K^T is
// one product; T comes from a blocked inversion at FP32 accuracy (16 x 16 diagonal blocks by substitution, then the
// blocks below them by doubling, -M22^-1 M21 M11^-1, on warp-level tensor tiles with operands split in two TF32
// parts); then [T diag(beta exp(G)); T diag(beta)] times K and times V, whose B operands are K and V exactly as
// they are stored (token rows, dims contiguous: "MN-major" operands, no transposition).  It leaves every operand the
// apply kernel multiplies with as a ready shared-memory image in the workspace.  `apply` walks the chunks in order for one (value head, 32-column slice
// of the state): the slice lives in registers (FP32) and, rounded to TF32, in shared memory as the B operand;
// [Q; W] S0, P Delta and (diag(e) K)^T Delta are the products.  State columns are independent, so the four slices
// of a head never talk to each other.  TF32 (10-bit mantissa, FP32 accumulate) rather than BF16 keeps the FP32
// state within 1e-3 relative L2 of the sequential recurrence over 64 chunks.
//
// Dense flops per launch: chunks * value_heads * [2 C^2 (3 dk + 2 dv) + 6 C dk dv].

#include "common.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <type_traits>

namespace rib200 {
namespace {

constexpr int kDim = 128;
constexpr int kChunk = 64;
constexpr int kSlice = 32;          // state columns per apply CTA
constexpr int kPitchSq = 68;        // 64-wide FP32 matrices of the inversion: pitch = 4 mod 32 words
// Workspace record of one (chunk, value head), in bytes.  A1 and A2 are images of K-major tcgen05 operands:
// 32 TF32 elements (128 bytes) per row and k-block, [k-block][row][128 bytes], the 16-byte piece index of a row
// XORed with row % 8 (SWIZZLE_128B).  A3 is the image of an MN-major operand (see mn_offset).
constexpr std::uint32_t kRowBytes = 128;
constexpr std::uint32_t kA1Block = 128 * kRowBytes;               // rows 0..63 Q, rows 64..127 W; 4 k-blocks
constexpr std::uint32_t kA1Bytes = 4 * kA1Block;
constexpr std::uint32_t kA2Block = kChunk * kRowBytes;            // P, 64 rows; 2 k-blocks
constexpr std::uint32_t kA2Bytes = 2 * kA2Block;
constexpr std::uint32_t kA3AtomBytes = kChunk * kRowBytes;        // diag(e) K: 4 groups of 32 key dims x 64 tokens
constexpr std::uint32_t kA3Bytes = 4 * kA3AtomBytes;
constexpr int kPitchU = 36;                                        // U slice [64][36] FP32, then gamma [64]
constexpr std::uint32_t kUBytes = (kChunk * kPitchU + kChunk) * 4;
constexpr std::uint32_t kRecA1 = 0;
constexpr std::uint32_t kRecA2 = kRecA1 + kA1Bytes;
constexpr std::uint32_t kRecA3 = kRecA2 + kA2Bytes;
constexpr std::uint32_t kRecU = kRecA3 + kA3Bytes;                // [4 slices] of kUBytes
constexpr std::uint32_t kRecBytes = kRecU + (kDim / kSlice) * kUBytes;
static_assert(kRecBytes % 16 == 0 && kUBytes % 16 == 0, "16-byte blocks");

// Byte offset of element (row, k) inside a K-major operand image whose k-blocks are block_bytes apart.
__host__ __device__ constexpr std::uint32_t image_offset(std::uint32_t row, std::uint32_t k, std::uint32_t block_bytes) {
  return (k >> 5) * block_bytes + row * kRowBytes + ((((k & 31U) >> 2) ^ (row & 7U)) << 4) + ((k & 3U) << 2);
}
// Byte offset of element (token, dim) of a [token][128 dims] matrix stored as an MN-major operand: groups of 32
// dims `atom_bytes` apart, inside a group one 128-byte row per token, the 32-byte piece index XORed with token % 4.
__host__ __device__ constexpr std::uint32_t mn_offset(std::uint32_t token, std::uint32_t dim, std::uint32_t atom_bytes) {
  return (dim >> 5) * atom_bytes + token * kRowBytes + ((((dim & 31U) >> 3) ^ (token & 3U)) << 5) + ((dim & 7U) << 2);
}

// The prepare kernel writes piece `part` (dims 32 kb + 4 part ..) of row `row` with these offsets spelled out:
static_assert(mn_offset(5, 32 + 4 * 3, kA3AtomBytes) ==
                  kA3AtomBytes + 5 * kRowBytes + ((((3U >> 1) ^ (5U & 3U)) << 5) | ((3U & 1U) << 4)),
              "MN-major piece offset");
static_assert(image_offset(13, 64 + 4 * 6, kA1Block) == 2 * kA1Block + 13 * kRowBytes + ((6U ^ (13U & 7U)) << 4),
              "K-major piece offset");

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

// Round to TF32 (10 mantissa bits), nearest with ties away from zero, as cvt.rna.tf32.f32 does for finite numbers:
// half a unit of the last kept place is added to the magnitude and the 13 low bits are dropped.  Two integer
// instructions at full rate; the conversion instruction goes through the slow conversion pipe, and the kernels
// below round tens of thousands of values per item.
__device__ __forceinline__ std::uint32_t tf32(float x) { return (__float_as_uint(x) + 0x1000U) & 0xFFFFE000U; }
__device__ __forceinline__ float tf32f(float x) { return __uint_as_float(tf32(x)); }
// e^x through the base-2 unit; results below the normal range are flushed to zero, which is what every use here
// (decay factors <= 1 and their products with bounded numbers) wants, and spares the code around a subnormal result.
__device__ __forceinline__ float exp_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x * 1.4426950408889634F));
  return y;
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
// the prepare kernel's first CTA: rows 100.. of the probe, one per item it walks
#define PREP_STAMP(slot)                              \
  do {                                                \
    if (threadIdx.x == 0) {                           \
      RIB200_GDN_STAMP(100 + iteration, slot);        \
    }                                                 \
  } while (0)

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
// tiled tensor-map load of one box, completion counted on an mbarrier
__device__ __forceinline__ void tma_load_2d(std::uint32_t dst, const void *map, int c0, int c1, std::uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
                   "r"(dst),
               "l"(reinterpret_cast<std::uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
               : "memory");
}
// bulk copy shared -> global, completion tracked by the issuing thread's bulk groups
__device__ __forceinline__ void bulk_copy_s2g(void *dst, std::uint32_t src, std::uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes)
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
// Shared-memory matrix descriptor of an operand whose M (or N) index is the contiguous one ("MN-major"), 32-bit
// elements: rows of 128 bytes hold 32 consecutive M/N elements of one k index, four such rows (512 bytes) form an
// atom inside which the 32-byte piece index is XORed with the row index (the 32-byte-base form of the 128-byte
// swizzle, the only MN-major form for 32-bit elements); atoms follow each other `k_atom_bytes` apart along k and
// `mn_atom_bytes` apart along M/N.
__device__ __forceinline__ std::uint64_t smem_desc_mn(std::uint32_t addr, std::uint32_t mn_atom_bytes,
                                                      std::uint32_t k_atom_bytes) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((addr & 0x3FFFFU) >> 4);
  d |= static_cast<std::uint64_t>(mn_atom_bytes >> 4) << 16; // leading-dimension offset: between M/N atoms
  d |= static_cast<std::uint64_t>(k_atom_bytes >> 4) << 32;  // stride offset: between k atoms
  d |= static_cast<std::uint64_t>(1) << 46;                  // version
  d |= static_cast<std::uint64_t>(1) << 61;                  // SWIZZLE_128B with a 32-byte base
  return d;
}
// Instruction descriptor: TF32 x TF32 -> FP32, M 128, N columns; bit 15 / bit 16 mark an MN-major A / B operand.
__host__ __device__ constexpr std::uint32_t idesc_tf32(std::uint32_t n, bool a_mn_major, bool b_mn_major) {
  return (1U << 4) | (2U << 7) | (2U << 10) | (a_mn_major ? 1U << 15 : 0U) | (b_mn_major ? 1U << 16 : 0U) |
         ((n >> 3) << 17) | (static_cast<std::uint32_t>(128 >> 4) << 24);
}
constexpr std::uint32_t kIdesc = idesc_tf32(kSlice, false, false);
constexpr std::uint32_t kIdescMnA = idesc_tf32(kSlice, true, false);
__device__ __forceinline__ void umma_tf32(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                          std::uint32_t accumulate, std::uint32_t idesc = kIdesc) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
               "}\n" ::"r"(d_tmem),
               "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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
__device__ __forceinline__ uint4 lds128u(std::uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds128(std::uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// ---- prepare: per (chunk, value head), persistent CTAs --------------------------------------------------
// 512 threads.  Thread (row = tid / 8, part = tid % 8) owns dims 64 a + 8 part .. + 7 (a = 0, 1) of token `row` of
// K, Q and V; the rows of the next item are already in flight while the current one is worked on.  Per item:
//   images   K and Q rounded to TF32 into the K-major image [K; Q] (A and B of the first product); K and V into
//            MN-major images (B of the last two); Q and diag(e) K also go to the workspace record from registers
//   G        = [K; Q] K^T            M 128, N 64, K 128   -> rows 0..63 K K^T, rows 64..127 Q K^T
//   rows 0..63: A = beta_i decay_ij (K K^T)_ij below the diagonal -> shared memory;  rows 64..127: P -> record
//            (a warp reads 32 rows x 16 columns of tensor memory; decay_ij = exp(G_i - G_j) is one exponential per
//            element only inside the diagonal 16 x 16 blocks, elsewhere the product of a row and a column factor
//            taken against the running sum at the end of the column block, both <= 1)
//   T        = (I + A)^-1 in FP32, all warps
//   [W; *]   = [T diag(beta gamma); T diag(beta)] K      M 128, N 128, K 64   (rows 0..63 are W)
//   [*; U]   = [T diag(beta gamma); T diag(beta)] V      M 128, N 128, K 64   (rows 64..127 are U)
//   rows 0..63: W -> record (TF32 image);  rows 64..127: U, gamma -> record (a warp reads 32 rows x 32 columns)
// Record pieces leave through shared-memory staging and bulk copies.  Every mbarrier wait is bounded as in the
// apply kernel.
constexpr int kPrepThreads = 512;
constexpr std::uint32_t kPsKQ = 0;                          // [K; Q] image, 64 KiB; later:
constexpr std::uint32_t kPsTstack = kPsKQ;                  //   [T diag(beta gamma); T diag(beta)] image, 32 KiB
constexpr std::uint32_t kPsWstage = kPsKQ;                  //   W image on its way to the record, 32 KiB
constexpr std::uint32_t kPsKb = 65536;                      // K as an MN-major operand, 32 KiB
constexpr std::uint32_t kPsVb = kPsKb + 32768;              // V as an MN-major operand, 32 KiB
constexpr std::uint32_t kPsUstage = kPsKb;                  //   later: the four U slices on their way to the record
constexpr std::uint32_t kPsKe = kPsVb + 32768;              // diag(e) K on its way to the record, 32 KiB
constexpr std::uint32_t kPsPstage = kPsKe + 32768;          // P image on its way to the record, 16 KiB
constexpr std::uint32_t kPsA = kPsPstage + 16384;           // A, FP32 [64][68]
constexpr std::uint32_t kPsT = kPsA + kChunk * kPitchSq * 4; // T, FP32 [64][68]
constexpr std::uint32_t kPsVec = kPsT + kChunk * kPitchSq * 4; // G, beta, beta gamma, column factors: 4 x 64 floats
constexpr std::uint32_t kPsGateNext = kPsVec + 1024;         // the next item's log decays [64] and betas [64]
constexpr std::uint32_t kPsBars = kPsGateNext + 512;
constexpr std::uint32_t kPsTmemSlot = kPsBars + 32;
// The raw rows of the next item land, by tensor-map copies issued while the current item is in its last third, in
// areas that are idle by then: K in the diag(e) K staging area, Q in the upper half of the [K; Q] image, V in the P
// staging area and A.  FP32 rows take 32 KiB per operand, BF16 rows 16 KiB.
constexpr std::uint32_t kPsRawK = kPsKe;
constexpr std::uint32_t kPsRawQ = kPsKQ + 32768;
constexpr std::uint32_t kPsRawV = kPsPstage;
static_assert(kPsA + kChunk * kPitchSq * 4 - kPsPstage >= 32768, "raw V rows fit in the P staging area and A");
constexpr std::uint32_t kPsAbort = kPsTmemSlot + 4;
constexpr std::uint32_t kPrepSmemBytes = kPsAbort + 4 + 1024; // + room to align the base to 1 KiB
static_assert((kDim / kSlice) * kUBytes <= 65536 && kPsA % 16 == 0 && kPsBars % 8 == 0, "staging fits, alignment");
static_assert(kPrepSmemBytes <= 232448, "prepare kernel exceeds the shared memory of an SM");
constexpr long long kPrepWaitLimitCycles = 1LL << 28;
constexpr std::uint32_t kPrepTmemColumns = 512;  // G at 0 (64 columns), [W; *] at 64, [*; U] at 192
constexpr std::uint32_t kIdescG = idesc_tf32(kChunk, false, false);
constexpr std::uint32_t kIdescWU = idesc_tf32(kDim, false, true);

// A thread's share of one raw row: piece `part` (4 elements) of each of the four k-blocks (32 dims) of row tid / 8,
// so that the eight lanes of a row read and later store eight consecutive 16-byte pieces of one 128-byte image row.
template <bool F32> struct RowPieces {
  using Word = std::conditional_t<F32, uint4, uint2>;
  Word v[4];
};
template <bool F32> struct ItemRegs {
  RowPieces<F32> k, q, v;
};
__device__ __forceinline__ uint2 lds64u(std::uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
// from a raw [64][128] tile in shared memory (rows past the last token were filled with zeros by the copy)
template <bool F32> __device__ __forceinline__ RowPieces<F32> read_pieces(std::uint32_t tile) {
  RowPieces<F32> regs;
  const std::uint32_t row = threadIdx.x >> 3;
  const std::uint32_t part = threadIdx.x & 7U;
  if constexpr (F32) {
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      regs.v[kb] = lds128u(tile + row * 512U + 128U * kb + 16U * part);
    }
  } else {
    // An 8-byte load is served sixteen lanes (two rows) at a time, and rows lie 256 bytes apart: odd rows take the
    // two k-blocks of a pair in the other order, so that the two rows never read the same banks.
    const std::uint32_t odd = row & 1U;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint2 x = lds64u(tile + row * 256U + 64U * (2 * h + odd) + 8U * part);
      const uint2 y = lds64u(tile + row * 256U + 64U * (2 * h + 1 - odd) + 8U * part);
      regs.v[2 * h] = odd ? y : x;
      regs.v[2 * h + 1] = odd ? x : y;
    }
  }
  return regs;
}
// the four values of a piece as TF32 numbers (BF16 inputs are TF32 numbers as they are)
template <bool F32>
__device__ __forceinline__ void unpack_piece(const typename RowPieces<F32>::Word &w, float (&f)[4]) {
  if constexpr (F32) {
    f[0] = tf32f(__uint_as_float(w.x));
    f[1] = tf32f(__uint_as_float(w.y));
    f[2] = tf32f(__uint_as_float(w.z));
    f[3] = tf32f(__uint_as_float(w.w));
  } else {
    f[0] = __uint_as_float(w.x << 16);
    f[1] = __uint_as_float(w.x & 0xFFFF0000U);
    f[2] = __uint_as_float(w.y << 16);
    f[3] = __uint_as_float(w.y & 0xFFFF0000U);
  }
}

__device__ __forceinline__ void tmem_ld16(std::uint32_t taddr, float (&v)[16]) {
  std::uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = __uint_as_float(r[i]);
  }
}

// ---- small FP32-accurate block products on the warp-level tensor path (the inversion of I + A) ----
__device__ __forceinline__ void mma_tf32(float (&c)[4], const std::uint32_t (&a)[4], std::uint32_t b0,
                                         std::uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo with both parts TF32: hi * hi + hi * lo + lo * hi of two such numbers is their product to FP32 accuracy
__device__ __forceinline__ void split_tf32(float x, std::uint32_t &hi, std::uint32_t &lo) {
  hi = tf32(x);
  lo = tf32(x - __uint_as_float(hi));
}
// acc (a 16 x 8 accumulator tile) += L[r0 .. r0+15][k0 .. k0+8 KSTEPS) R[k0 ..][c0 .. c0+7], L and R row-major FP32
// matrices of pitch kPitchSq in shared memory; one warp.  The three partial products run in accumulators of their
// own, so that consecutive tensor instructions do not wait for each other.
template <int KSTEPS>
__device__ __forceinline__ void tile_product(float (&acc)[4], const float *L, int r0, const float *R, int c0, int k0) {
  const int g = (threadIdx.x & 31) >> 2;
  const int t = threadIdx.x & 3;
  float lo_hi[4] = {};
  float hi_lo[4] = {};
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int k = k0 + 8 * ks;
    const float *l = L + (r0 + g) * kPitchSq + k + t;
    const float *r = R + (k + t) * kPitchSq + c0 + g;
    std::uint32_t a_hi[4];
    std::uint32_t a_lo[4];
    std::uint32_t b_hi[2];
    std::uint32_t b_lo[2];
    split_tf32(l[0], a_hi[0], a_lo[0]);
    split_tf32(l[8 * kPitchSq], a_hi[1], a_lo[1]);
    split_tf32(l[4], a_hi[2], a_lo[2]);
    split_tf32(l[8 * kPitchSq + 4], a_hi[3], a_lo[3]);
    split_tf32(r[0], b_hi[0], b_lo[0]);
    split_tf32(r[4 * kPitchSq], b_hi[1], b_lo[1]);
    mma_tf32(lo_hi, a_lo, b_hi[0], b_hi[1]);
    mma_tf32(hi_lo, a_hi, b_lo[0], b_lo[1]);
    mma_tf32(acc, a_hi, b_hi[0], b_hi[1]);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[e] += lo_hi[e] + hi_lo[e];
  }
}
// the tile, times -1, goes into the [T diag(beta gamma); T diag(beta)] image at `tstack` (rows r0 .., columns c0 ..)
__device__ __forceinline__ void store_tile_scaled(std::uint32_t tstack, int r0, int c0, const float (&acc)[4],
                                                  const float *bg, const float *be) {
  const int g = (threadIdx.x & 31) >> 2;
  const int t = threadIdx.x & 3;
  const int col = c0 + 2 * t;
  const float2 sg = *reinterpret_cast<const float2 *>(bg + col);
  const float2 se = *reinterpret_cast<const float2 *>(be + col);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const std::uint32_t row = static_cast<std::uint32_t>(r0 + g + 8 * h);
    const float x = -acc[2 * h];
    const float y = -acc[2 * h + 1];
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(tstack + image_offset(row, col, kA1Block)),
                 "r"(tf32(x * sg.x)), "r"(tf32(y * sg.y))
                 : "memory");
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(tstack + image_offset(kChunk + row, col, kA1Block)),
                 "r"(tf32(x * se.x)), "r"(tf32(y * se.y))
                 : "memory");
  }
}
// the tile goes to M[r0 ..][c0 ..] times `sign`
__device__ __forceinline__ void store_tile(float *M, int r0, int c0, const float (&acc)[4], float sign) {
  const int g = (threadIdx.x & 31) >> 2;
  const int t = threadIdx.x & 3;
  float *at = M + (r0 + g) * kPitchSq + c0 + 2 * t;
  *reinterpret_cast<float2 *>(at) = make_float2(sign * acc[0], sign * acc[1]);
  *reinterpret_cast<float2 *>(at + 8 * kPitchSq) = make_float2(sign * acc[2], sign * acc[3]);
}

template <bool F32>
__global__ void __launch_bounds__(kPrepThreads, 1)
    gdn_chunk_prepare_kernel(const ChunkParams p, const __grid_constant__ TensorMapBytes k_map,
                             const __grid_constant__ TensorMapBytes q_map, const __grid_constant__ TensorMapBytes v_map) {
  extern __shared__ unsigned char prep_smem_raw[];
  const std::uint32_t base = (smem_address(prep_smem_raw) + 1023U) & ~1023U;
  unsigned char *smem = prep_smem_raw + (base - smem_address(prep_smem_raw));
  float *sA = reinterpret_cast<float *>(smem + kPsA);
  float *sT = reinterpret_cast<float *>(smem + kPsT);
  float *sG = reinterpret_cast<float *>(smem + kPsVec);  // inclusive running log decay
  float *sBeta = sG + kChunk;
  float *sBg = sBeta + kChunk;                            // beta * exp(G)
  float *sCf = sBg + kChunk;                              // exp(G at the end of the token's block of 16 - G)
  const std::uint32_t bar_g = base + kPsBars;
  const std::uint32_t bar_wu = base + kPsBars + 8;
  const std::uint32_t bar_raw = base + kPsBars + 16;
  float *sGateNext = reinterpret_cast<float *>(smem + kPsGateNext);
  volatile std::uint32_t *tmem_slot = reinterpret_cast<volatile std::uint32_t *>(smem + kPsTmemSlot);
  volatile std::uint32_t *abort_flag = reinterpret_cast<volatile std::uint32_t *>(smem + kPsAbort);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const std::uint32_t row = tid >> 3;
  const std::uint32_t part = tid & 7;
  const std::uint32_t items = p.chunks * p.value_heads;

  if (tid == 0) {
    mbarrier_init(bar_g, 1);
    mbarrier_init(bar_wu, 1);
    mbarrier_init(bar_raw, 2); // the rows of an item are asked for in two batches
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(base + kPsTmemSlot),
                 "r"(kPrepTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const std::uint32_t tmem = *tmem_slot;
  // Launched with programmatic stream serialisation: barriers and tensor memory are set up while the kernel in front
  // (the layer's prologue, or whatever the caller queued) finishes; its results are read only after this.
  grid_dependency_wait();
  // Only now may the apply kernel behind this one set itself up on SMs as they become free (it waits for this grid to
  // end before it reads a record): what it reads before that wait, the recurrent state, is final once the kernels in
  // front of this one have ended.
  grid_dependents_may_launch();
  const bool issuer = warp == 4 && elect_one();
  // One lane of the last warp issues every bulk copy to the record (bulk groups belong to the issuing thread) and
  // waits for them to have read their staging areas before those are written again.
  const bool copier = tid == kPrepThreads - 32;

  auto wait = [&](std::uint32_t b, std::uint32_t parity) {
    if (*abort_flag != 0 || mbarrier_try_wait(b, parity)) {
      return;
    }
    const long long started = clock64();
    while (!mbarrier_try_wait(b, parity)) {
      if (*abort_flag != 0) {
        return;
      }
      if (clock64() - started > kPrepWaitLimitCycles) {
        *abort_flag = 1;
        atomicOr(p.status, static_cast<unsigned int>(RIB200_DEVICE_WAIT_TIMED_OUT));
        return;
      }
    }
  };

  // The raw K, Q and V rows of an item come in as three tensor-map copies (rows past the last token arrive as
  // zeros), issued by the copier lane an item ahead; its gates are read by two otherwise idle warps at the same time.
  constexpr std::uint32_t kRawBytes = kChunk * kDim * (F32 ? 4 : 2);
  // Batch 1 (K, Q, and V when it fits the P staging area alone, i.e. BF16 rows) can go out as soon as the copies of
  // the Q rows, of diag(e) K and of P have read their areas; FP32 V rows also cover A and wait for the inversion.
  auto issue_rows = [&](std::uint32_t item, bool first_batch) {
    const std::uint32_t head = item % p.value_heads;
    const int tok0 = static_cast<int>((item / p.value_heads) * kChunk);
    const int key_x = static_cast<int>((head % p.key_heads) * kDim);
    fence_proxy_async(); // the landing areas were last touched by ordinary loads and stores
    if (first_batch) {
      mbarrier_expect_tx(bar_raw, (F32 ? 2 : 3) * kRawBytes);
      tma_load_2d(base + kPsRawK, &k_map, key_x, tok0, bar_raw);
      tma_load_2d(base + kPsRawQ, &q_map, key_x, tok0, bar_raw);
    }
    if (first_batch != F32) {
      if (!first_batch) {
        mbarrier_expect_tx(bar_raw, kRawBytes);
      }
      tma_load_2d(base + kPsRawV, &v_map, static_cast<int>(head * kDim), tok0, bar_raw);
    } else if (!first_batch) {
      mbarrier_arrive(bar_raw);
    }
  };
  auto load_gates = [&](std::uint32_t item) { // warps 8 and 9: one token per thread
    const std::uint32_t t = tid - 256;
    const std::uint32_t tok = min((item / p.value_heads) * kChunk + t, p.tokens - 1);
    const std::size_t at = static_cast<std::size_t>(tok) * p.value_heads + item % p.value_heads;
    sGateNext[t] = p.log_decay[at];
    sGateNext[kChunk + t] = p.beta[at];
  };
  std::uint32_t rows_in_flight = 0;
  if (blockIdx.x < items) {
    if (copier) {
      issue_rows(blockIdx.x, true);
      issue_rows(blockIdx.x, false);
      rows_in_flight = 1;
    }
    if (warp == 8 || warp == 9) {
      load_gates(blockIdx.x);
    }
  }
  __syncthreads();
  ItemRegs<F32> cur;
  std::uint32_t iteration = 0;
  for (std::uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++iteration) {
    const std::uint32_t phase = iteration & 1U;
    PREP_STAMP(0);
    wait(bar_raw, phase);
    PREP_STAMP(13);
    if (copier) {
      rows_in_flight = 0;
    }
    cur.k = read_pieces<F32>(base + kPsRawK);
    cur.q = read_pieces<F32>(base + kPsRawQ);
    cur.v = read_pieces<F32>(base + kPsRawV);
    PREP_STAMP(14);
    unsigned char *rec = p.workspace + static_cast<std::size_t>(item) * kRecBytes; // item = chunk * value_heads + head

    // ---- gates: running sum of the log decays (two tokens per lane, warp scan), beta ----
    const std::uint32_t tok0 = (item / p.value_heads) * kChunk;
    if (warp == 0) {
      float a = tok0 + lane < p.tokens ? sGateNext[lane] : 0.0F;
      float b = tok0 + lane + 32 < p.tokens ? sGateNext[lane + 32] : 0.0F;
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
      const std::uint32_t t = lane + 32 * (warp - 1);
      sBeta[t] = tok0 + t < p.tokens ? sGateNext[kChunk + t] : 0.0F;
    }
    __syncthreads(); // every thread holds its pieces of the raw rows; the gates are in place
    PREP_STAMP(1);
    if (tid < kChunk) {
      sBg[tid] = sBeta[tid] * exp_fast(sG[tid]);
      sCf[tid] = exp_fast(sG[tid | 15] - sG[tid]);
    }

    // ---- operand images ----
    // The W and U staging areas of the item before (the lower half of the [K; Q] image, the MN-major K image and
    // the head of the V image) are still being read by their copies to the record: the images that lie elsewhere
    // are written first, the rest once the copier lane has seen those reads end.
    {
      const float e_row = exp_fast(sG[kChunk - 1] - sG[row]); // exp(G_C - G_row) <= 1
      // Where this thread's piece of k-block kb goes: K-major images are [k-block][row][128 bytes] with the 16-byte
      // piece index XORed with row % 8; MN-major images (see mn_offset) XOR the 32-byte piece index with row % 4.
      const std::uint32_t k_major = row * kRowBytes + ((part ^ (row & 7U)) << 4);
      const std::uint32_t mn_major = row * kRowBytes + ((((part >> 1) ^ (row & 3U)) << 5) | ((part & 1U) << 4));
      const std::uint32_t image_k = base + kPsKQ + k_major;
      const std::uint32_t image_q = image_k + kChunk * kRowBytes;
      float f[4];
      // first: diag(e) K, the upper k-blocks of [K; Q], the upper half of V
#pragma unroll
      for (std::uint32_t kb = 0; kb < 4; ++kb) {
        unpack_piece<F32>(cur.k.v[kb], f);
        sts128(base + kPsKe + kb * kA3AtomBytes + mn_major, tf32f(f[0] * e_row), tf32f(f[1] * e_row), tf32f(f[2] * e_row),
               tf32f(f[3] * e_row));
        if (kb >= 2) {
          sts128(image_k + kb * kA1Block, f[0], f[1], f[2], f[3]);
          unpack_piece<F32>(cur.q.v[kb], f);
          sts128(image_q + kb * kA1Block, f[0], f[1], f[2], f[3]);
          unpack_piece<F32>(cur.v.v[kb], f);
          sts128(base + kPsVb + kb * kA3AtomBytes + mn_major, f[0], f[1], f[2], f[3]);
        }
      }
      if (copier) { // the previous item's W and U copies must have read their staging areas
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
      }
      __syncthreads();
#pragma unroll
      for (std::uint32_t kb = 0; kb < 4; ++kb) {
        unpack_piece<F32>(cur.k.v[kb], f);
        sts128(base + kPsKb + kb * kA3AtomBytes + mn_major, f[0], f[1], f[2], f[3]);
        if (kb < 2) {
          sts128(image_k + kb * kA1Block, f[0], f[1], f[2], f[3]);
          unpack_piece<F32>(cur.q.v[kb], f);
          sts128(image_q + kb * kA1Block, f[0], f[1], f[2], f[3]);
          unpack_piece<F32>(cur.v.v[kb], f);
          sts128(base + kPsVb + kb * kA3AtomBytes + mn_major, f[0], f[1], f[2], f[3]);
        }
      }
    }
    fence_proxy_async();
    tcgen05_fence_before();
    __syncthreads();

    PREP_STAMP(2);
    // ---- G = [K; Q] K^T ----
    if (copier && *abort_flag == 0) {
      // Q is rows 64..127 of every k-block of the [K; Q] image and rows 0..63 of the record's [Q; W] image
#pragma unroll
      for (std::uint32_t kb = 0; kb < 4; ++kb) {
        bulk_copy_s2g(rec + kRecA1 + kb * kA1Block, base + kPsKQ + kb * kA1Block + kChunk * kRowBytes, kChunk * kRowBytes);
      }
      bulk_copy_s2g(rec + kRecA3, base + kPsKe, kA3Bytes);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
    if (warp == 4) {
      tcgen05_fence_after();
      if (issuer && *abort_flag == 0) {
        const std::uint64_t kq_desc = smem_desc(base + kPsKQ);
#pragma unroll
        for (std::uint32_t ks = 0; ks < 16; ++ks) {
          const std::uint64_t step = static_cast<std::uint64_t>(((ks >> 2) * kA1Block + (ks & 3U) * 32U) >> 4);
          umma_tf32(tmem, kq_desc + step, kq_desc + step, ks, kIdescG);
        }
        umma_commit(bar_g);
      }
      __syncwarp();
    }

    // ---- rows of G: A (lower triangle, to shared memory) and P (to its staging image) ----
    {
      wait(bar_g, phase);
    PREP_STAMP(3);
      tcgen05_fence_after();
      const std::uint32_t quarter = warp & 3;       // the 32 tensor-memory lanes this warp may read
      const std::uint32_t cg = warp >> 2;           // its 16 columns
      const std::uint32_t lane_base = (quarter * 32U) << 16;
      const std::uint32_t i = (quarter & 1U) * 32 + lane; // token of the row
      const bool is_p = quarter >= 2;               // rows 64..127 hold Q K^T
      float g[16];
      tmem_ld16(tmem + lane_base + 16 * cg, g);
      PREP_STAMP(15);
      const float g_i = sG[i];
      const float scale_i = is_p ? 1.0F : sBeta[i];
      float out[16];
      if (16 * cg > i) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          out[e] = 0.0F;
        }
      } else if ((i >> 4) == cg) { // diagonal block: one exponential per element
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const std::uint32_t j = 16 * cg + e;
          const bool live = is_p ? j <= i : j < i;
          out[e] = live ? scale_i * exp_fast(g_i - sG[j]) * g[e] : 0.0F;
        }
      } else { // below it: exp(G_i - G_j) = exp(G_i - R) exp(R - G_j), R the running sum at the end of the column block
        const float row_factor = scale_i * exp_fast(g_i - sG[16 * cg + 15]);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          out[e] = row_factor * sCf[16 * cg + e] * g[e];
        }
      }
      PREP_STAMP(11);
      if (!is_p) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          *reinterpret_cast<float4 *>(sA + i * kPitchSq + 16 * cg + 4 * c) =
              make_float4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          sts128(base + kPsPstage + image_offset(i, 16 * cg + 4 * c, kA2Block), tf32f(out[4 * c]), tf32f(out[4 * c + 1]),
                 tf32f(out[4 * c + 2]), tf32f(out[4 * c + 3]));
        }
      }
      PREP_STAMP(12);
      fence_proxy_async();
      tcgen05_fence_before();
    }
    __syncthreads();
    PREP_STAMP(4);
    if (copier && *abort_flag == 0) {
      bulk_copy_s2g(rec + kRecA2, base + kPsPstage, kA2Bytes);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }

    // ---- T = (I + A)^-1: diagonal 16 x 16 blocks by forward substitution, a column per thread ... ----
    if (tid < kChunk) {
      const int b = tid >> 4;
      const int c = tid & 15;
      float tcol[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = i == c ? 1.0F : 0.0F;
        const float *a_row = sA + (16 * b + i) * kPitchSq + 16 * b;
#pragma unroll
        for (int j = 0; j < i; ++j) {
          acc -= a_row[j] * tcol[j];
        }
        tcol[i] = acc;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        sT[(16 * b + i) * kPitchSq + 16 * b + c] = tcol[i];
      }
    } else {
      // ... while the other threads clear the blocks above the diagonal
      for (int e = tid - kChunk; e < 6 * 256; e += kPrepThreads - kChunk) {
        const int blk = e >> 8; // (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
        const int bi = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
        const int bj = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);
        sT[(16 * bi + ((e >> 4) & 15)) * kPitchSq + 16 * bj + (e & 15)] = 0.0F;
      }
    }
    if (copier) {
      // The image of [T diag(beta gamma); T diag(beta)] is written, from here on, over the lower k-blocks of the
      // [K; Q] image: the copies of its Q rows to the record (issued long ago) must have read them.  The copy of P
      // is waited for as well, so that its staging area can take the next item's rows later.
      asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
    }
    __syncthreads();
    if (copier && item + gridDim.x < items && *abort_flag == 0) {
      issue_rows(item + gridDim.x, true);
      rows_in_flight = 1;
    }
    PREP_STAMP(5);
    // Eight columns of a row of T that are final go into the image, scaled per column; idle warps do this for the
    // diagonal blocks and the zeros above them during step 1 below, and for the blocks of step 1 during step 2.
    auto image_unit = [&](std::uint32_t r, std::uint32_t part8) {
      const std::uint32_t j0 = 8 * part8;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float4 t4 = *reinterpret_cast<const float4 *>(sT + r * kPitchSq + j0 + 4 * c);
        const float4 bg = *reinterpret_cast<const float4 *>(sBg + j0 + 4 * c);
        const float4 be = *reinterpret_cast<const float4 *>(sBeta + j0 + 4 * c);
        sts128(base + kPsTstack + image_offset(r, j0 + 4 * c, kA1Block), tf32f(t4.x * bg.x), tf32f(t4.y * bg.y),
               tf32f(t4.z * bg.z), tf32f(t4.w * bg.w));
        sts128(base + kPsTstack + image_offset(kChunk + r, j0 + 4 * c, kA1Block), tf32f(t4.x * be.x),
               tf32f(t4.y * be.y), tf32f(t4.z * be.z), tf32f(t4.w * be.w));
      }
    };
    if (tid >= 128 && tid < 128 + 320) { // units on or above the block diagonal: 128 + 96 + 64 + 32
      const std::uint32_t idx = tid - 128;
      if (idx < 128) {
        image_unit(idx >> 3, idx & 7U);
      } else if (idx < 224) {
        image_unit(16 + (idx - 128) / 6, 2 + (idx - 128) % 6);
      } else if (idx < 288) {
        image_unit(32 + ((idx - 224) >> 2), 4 + ((idx - 224) & 3U));
      } else {
        image_unit(48 + ((idx - 288) >> 1), 6 + ((idx - 288) & 1U));
      }
    }
    // ... then the blocks below the diagonal by doubling: for M = [[M11, 0], [M21, M22]] the lower left block of the
    // inverse is -M22^-1 M21 M11^-1.
    //   step 1 (warps 0..3):  T_10 = -T_11 (A_10 T_00),  T_32 = -T_33 (A_32 T_22)            16 x 16 blocks
    //   step 2 (warps 0..7):  T[32..63][0..31] = -T[32..63][32..63] (A[32..63][0..31] T[0..31][0..31])
    // on warp-level tensor tiles with split operands (FP32 accuracy), a warp per 16 x 8 tile of the result (a column
    // tile of the second product only needs the same column tile of the first).  An intermediate product sits in the
    // place of the block of T that it becomes; triangular factors are only walked over their non-zero blocks.
    if (warp < 4) {
      const int b = 2 * (warp >> 1);
      const int i = b + 1;
      const int c0 = 16 * b + 8 * (warp & 1);
      float y[4] = {};
      tile_product<2>(y, sA, 16 * i, sT, c0, 16 * b);
      store_tile(sT, 16 * i, c0, y, 1.0F);
      __syncwarp();
      float z[4] = {};
      tile_product<2>(z, sT, 16 * i, sT, c0, 16 * i);
      __syncwarp();
      store_tile(sT, 16 * i, c0, z, -1.0F);
    }
    __syncthreads();
    PREP_STAMP(6);
    if ((warp == 8 || warp == 9) && item + gridDim.x < items) {
      load_gates(item + gridDim.x); // while eight warps work below; consumed at the top of the next item
    }
    if (warp == 10 || warp == 11) { // the two blocks of step 1: rows 16..31 x columns 0..15, rows 48..63 x columns 32..47
      const std::uint32_t idx = tid - 320;
      const std::uint32_t half = idx >> 5;
      image_unit(16 + 32 * half + ((idx & 31U) >> 1), 4 * half + (idx & 1U));
    }
    if (warp < 8) {
      const int bi = 2 + (warp >> 2);
      const int bj = (warp >> 1) & 1;
      const int c0 = 16 * bj + 8 * (warp & 1);
      float y[4] = {};
      if (bj == 0) { // T[0..31][0..31] is lower triangular: its second column block starts at row 16
        tile_product<4>(y, sA, 16 * bi, sT, c0, 0);
      } else {
        tile_product<2>(y, sA, 16 * bi, sT, c0, 16);
      }
      store_tile(sT, 16 * bi, c0, y, 1.0F);
      asm volatile("bar.sync 2, 256;\n" ::: "memory"); // row block 3 reads the product of row block 2 as well
      float z[4] = {};
      if (bi == 2) { // row block 2 of T[32..63][32..63] ends at column 47
        tile_product<2>(z, sT, 32, sT, c0, 32);
      } else {
        tile_product<4>(z, sT, 48, sT, c0, 32);
      }
      store_tile_scaled(base + kPsTstack, 16 * bi, c0, z, sBg, sBeta); // nobody reads these blocks of T again
    }
    fence_proxy_async(); // the image is complete: the products below read it through the async proxy
    tcgen05_fence_before();
    __syncthreads();
    // A is idle from here to the end of the item: FP32 V rows, which need its room too, are asked for now.
    if (copier && item + gridDim.x < items && rows_in_flight != 0) {
      issue_rows(item + gridDim.x, false); // completes the pair of arrivals even after a wait ran out
    }

    PREP_STAMP(7);
    PREP_STAMP(8);
    // ---- the two products with T: B operands are K and V as stored (eight tokens = 1 KiB per step) ----
    if (warp == 4) {
      tcgen05_fence_after();
      if (issuer && *abort_flag == 0) {
        const std::uint64_t t_desc = smem_desc(base + kPsTstack);
        const std::uint64_t kb_desc = smem_desc_mn(base + kPsKb, kA3AtomBytes, 512);
        const std::uint64_t vb_desc = smem_desc_mn(base + kPsVb, kA3AtomBytes, 512);
#pragma unroll
        for (std::uint32_t ks = 0; ks < 8; ++ks) {
          const std::uint64_t a_step = static_cast<std::uint64_t>(((ks >> 2) * kA1Block + (ks & 3U) * 32U) >> 4);
          umma_tf32(tmem + 64, t_desc + a_step, kb_desc + static_cast<std::uint64_t>(ks * 1024U >> 4), ks, kIdescWU);
        }
#pragma unroll
        for (std::uint32_t ks = 0; ks < 8; ++ks) {
          const std::uint64_t a_step = static_cast<std::uint64_t>(((ks >> 2) * kA1Block + (ks & 3U) * 32U) >> 4);
          umma_tf32(tmem + 192, t_desc + a_step, vb_desc + static_cast<std::uint64_t>(ks * 1024U >> 4), ks, kIdescWU);
        }
        umma_commit(bar_wu);
      }
      __syncwarp();
    }

    // ---- W (rows 0..63 of the first) and U (rows 64..127 of the second) to their staging images ----
    {
      wait(bar_wu, phase);
    PREP_STAMP(9);
      tcgen05_fence_after();
      const std::uint32_t quarter = warp & 3;
      const std::uint32_t cg = warp >> 2;           // 32 columns: k-block `cg` of W, slice `cg` of U
      const std::uint32_t lane_base = (quarter * 32U) << 16;
      const std::uint32_t i = (quarter & 1U) * 32 + lane;
      float x[32];
      if (quarter < 2) { // W only ever feeds TF32 products: round it here, once
        tmem_ld32(tmem + lane_base + 64 + 32 * cg, x);
#pragma unroll
        for (std::uint32_t c = 0; c < 8; ++c) {
          sts128(base + kPsWstage + cg * (kChunk * kRowBytes) + i * kRowBytes + ((c ^ (i & 7U)) << 4), tf32f(x[4 * c]),
                 tf32f(x[4 * c + 1]), tf32f(x[4 * c + 2]), tf32f(x[4 * c + 3]));
        }
      } else {
        tmem_ld32(tmem + lane_base + 192 + 32 * cg, x);
        const std::uint32_t stage = base + kPsUstage + cg * kUBytes;
#pragma unroll
        for (std::uint32_t c = 0; c < 8; ++c) {
          sts128(stage + (i * kPitchU + 4 * c) * 4, x[4 * c], x[4 * c + 1], x[4 * c + 2], x[4 * c + 3]);
        }
        sts32(stage + (kChunk * kPitchU + i) * 4, __float_as_uint(exp_fast(sG[i])));
      }
      fence_proxy_async();
      tcgen05_fence_before();
    }
    __syncthreads();
    PREP_STAMP(10);
    if (copier && *abort_flag == 0) {
#pragma unroll
      for (std::uint32_t kb = 0; kb < 4; ++kb) { // rows 64..127 of every k-block of the [Q; W] image
        bulk_copy_s2g(rec + kRecA1 + kb * kA1Block + kChunk * kRowBytes, base + kPsWstage + kb * (kChunk * kRowBytes),
                      kChunk * kRowBytes);
      }
      bulk_copy_s2g(rec + kRecU, base + kPsUstage, (kDim / kSlice) * kUBytes);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
    // The staging areas are the next item's operand images: the copier waits for the copies to have read them
    // before the barrier that precedes the next image stores (top of the loop), not here.
  }
  if (copier) {
    asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
    if (rows_in_flight != 0) {
      // only after a wait ran out: rows were asked for and nobody took them; let them land before the CTA goes
      const long long started = clock64();
      while (!mbarrier_try_wait(bar_raw, iteration & 1U) && clock64() - started < kPrepWaitLimitCycles) {
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 4) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kPrepTmemColumns) : "memory");
  }
}

// ---- apply: per (state slice, value head), chunks in order ---------------------------------------------
// 192 threads.  Warps 0-3 own the 128 lanes of tensor memory (thread = row of every product), warp 4 issues the
// tcgen05 products (whole warp in step, one elected lane issuing), lane 0 of warp 5 streams the operand images of
// each chunk into shared memory with bulk copies counted on mbarriers.  Per chunk:
//   X  = [Q; W] S0            M 128 (rows 0..63 Q S0, rows 64..127 W S0), N 32, K 128
//   warps 2-3: Delta = U - X[64..]  ->  B operand (TF32);   warps 0-1: keep gamma_i (Q S0)_i
//   SD = (diag(e) K)^T Delta  M 128, N 32, K 64 (A operand MN-major: diag(e) K in token order)
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

__global__ void __launch_bounds__(kApplyThreads, 1)
    gdn_chunk_apply_kernel(const ChunkParams p, const __grid_constant__ TensorMapBytes out_map) {
  extern __shared__ unsigned char apply_smem_raw[];
  const std::uint32_t base = (smem_address(apply_smem_raw) + 1023U) & ~1023U;
  unsigned char *smem = apply_smem_raw + (base - smem_address(apply_smem_raw));
  const std::uint32_t bars = base + kSmBars;
  auto bar = [&](std::uint32_t index) { return bars + index * 8; };
  volatile std::uint32_t *tmem_slot = reinterpret_cast<volatile std::uint32_t *>(smem + kSmTmemSlot);
  volatile std::uint32_t *abort_flag = reinterpret_cast<volatile std::uint32_t *>(smem + kSmAbort);

  grid_dependents_may_launch(); // the layer's epilogue sets itself up behind this kernel and waits for it to end
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
  // Launched with programmatic stream serialisation behind the prepare kernel: barriers, tensor memory and the state
  // slice (which that kernel does not touch) are set up while its last CTAs finish; the records are read after this.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

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
    // diag(e) K as stored: [token][key dim], the key dim (M of this product) contiguous
    const std::uint64_t a3_desc = smem_desc_mn(base + kSmA23 + kA2Bytes, kA3AtomBytes, 512);
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
          // eight tokens per product = two k atoms = 1 KiB of the image
          umma_tf32(tmem + 64, a3_desc + static_cast<std::uint64_t>(ks * 1024U >> 4), bd_desc + step(ks, kB1Block), ks,
                    kIdescMnA);
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
                                 kPrepSmemBytes),
            "gated-delta prepare shared-memory opt-in");
    cuda_ok(cudaFuncSetAttribute(gdn_chunk_apply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kApplySmemBytes),
            "gated-delta apply shared-memory opt-in");
  });
}

// SMs of the current device: the prepare kernel runs one persistent CTA on each
int sm_count() {
  static int counts[64] = {};
  int device = 0;
  cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
  require(device >= 0 && device < 64, "device ordinal out of range", RIB200_STATUS_INTERNAL);
  if (counts[device] == 0) {
    int count = 0;
    cuda_ok(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device), "SM count");
    counts[device] = count > 0 ? count : 1;
  }
  return counts[device];
}

template <bool F32> void launch(const ChunkParams &params, cudaStream_t stream) {
  configure_once<F32>();
  const std::uint32_t items = params.chunks * params.value_heads;
  const std::uint32_t prepare_ctas = items < static_cast<std::uint32_t>(sm_count()) ? items : sm_count();
  // K, Q, V rows as tensor maps: a box is the 64 tokens x 128 elements of one (chunk, head)
  TensorMapBytes k_map;
  TensorMapBytes q_map;
  TensorMapBytes v_map;
  encode_plain_rows_map(&k_map, params.k, F32, static_cast<std::uint64_t>(params.key_heads) * kDim, params.k_stride,
                        params.tokens, kDim, kChunk);
  encode_plain_rows_map(&q_map, params.q, F32, static_cast<std::uint64_t>(params.key_heads) * kDim, params.q_stride,
                        params.tokens, kDim, kChunk);
  encode_plain_rows_map(&v_map, params.v, F32, static_cast<std::uint64_t>(params.value_heads) * kDim, params.v_stride,
                        params.tokens, kDim, kChunk);
  launch_programmatic(gdn_chunk_prepare_kernel<F32>, dim3(prepare_ctas), dim3(kPrepThreads), kPrepSmemBytes, stream,
                      "gated-delta prepare launch", params, k_map, q_map, v_map);
  TensorMapBytes out_map;
  encode_f32_rows_map(&out_map, params.out, static_cast<std::uint64_t>(params.value_heads) * kDim, params.tokens,
                      kSlice, kChunk);
  launch_programmatic(gdn_chunk_apply_kernel, dim3(kDim / kSlice, params.value_heads), dim3(kApplyThreads),
                      kApplySmemBytes, stream, "gated-delta apply launch", params, out_map);
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
