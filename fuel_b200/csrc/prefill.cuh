// One-kernel form of the tensor-core path (FUELQ_OPT_PREFILL_ONE_KERNEL: no dequantized slab in the workspace; the
// default form, faster from about 100 rows up, is plain_gemm.cuh, which also uses the PTX wrappers, descriptors and
// activation pre-passes of this file).
// Prefill path (large M): Y[M, N] = X[M, K] . W[N, K]^T as a dense bf16 contraction on the
// 5th-generation tensor cores. The reference has no tensor-core quantized path: its CUDA forward
// runs the mat-vec kernel for every M (fuel-cuda-backend/src/quantized.rs:452-473,543-587) and its
// Vulkan path dequantizes the whole matrix to f32 first (fuel-vulkan-backend/src/lib.rs:4221-4283).
// Here weight tiles are dequantized (GgmlType::to_float arithmetic, fuel-quantized/src/k_quants.rs:
// 1595-1622, 2158-2189, 611-627) straight into shared memory as bf16 in the tensor core's K-major
// 128-byte-swizzled layout and multiplied with tcgen05.mma, accumulating f32 in tensor memory.
//
// One CTA computes a 128 (output features) x kTileM (activation rows) tile:
//   warps 0-7  dequantize the weight tile of each 64-wide K stage (two threads per weight row, one per
//              32-element half, for Q4_K; one thread per row for the other formats); thread 0 also
//              issues the stage's activation tile as ONE tensor-map (TMA) copy of the bf16 matrix
//              (converted by a pre-pass) with the same 128-byte swizzle; warps 0-3 then read the
//              accumulator out of tensor memory and store Y;
//   warp  8    allocates tensor memory and, one lane, issues the MMAs and their commits.
// Measured: sixteen dequantizing warps (a quarter row each) are slower than eight; per stage the kernel moves
// 48 KB into shared memory and the MMAs read 48 KB back, which at 128 B/clk is already the stage time of a
// single-SM MMA - the next step is the two-SM form (cta_group::2), which halves the activation reads.
// Stages cycle through full/empty mbarriers; every wait is bounded and on expiry the CTA raises an
// abort flag, skips to the end, frees its tensor memory and returns.
#pragma once
#include <cuda.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dequantize.cuh"
#include "fq_common.cuh"

namespace fq {

constexpr int kPfTileN = 128;   // weight rows per CTA  (UMMA M)
constexpr int kPfTileK = 64;    // K per stage: one 128-byte swizzle atom of bf16
constexpr int kPfStages = 4;
constexpr int kPfDequantWarps = 8;   // two threads per weight row (four were measured slower)
constexpr int kPfThreads = 32 * (kPfDequantWarps + 1);

struct PrefillParams {
  const uint8_t* w;          // GGUF blocks, [N][K / block]
  float* y[8];               // destinations: y[q] is an [M][ldy] matrix (this GPU's, or a peer's mapped here)
  int n_dst;                 // how many of them (1 on a single GPU)
  int ldy;                   // row stride of the destinations (N on a single GPU, the full width when column-sharded)
  int n_off;                 // first column this launch produces within a destination row
  int M, N, K;
  int row_bytes;
  const float* row_unscale;  // f16 operands: factor per activation row that undoes the row's scaling (else null)
};

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// same, operands read as tf32 (f32 words whose low 13 mantissa bits are ignored); K = 8 per instruction
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ uint32_t to_tf32(float x) {  // round to nearest (ties away) at 10 mantissa bits
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 2-D tiled tensor-map copy global -> shared, completion in bytes on an mbarrier. x (innermost, in elements) times the
// element size must be a multiple of 16 bytes; rows outside the tensor arrive as zeros.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_dst),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, 8-row groups
// 1024 bytes apart (stride byte offset), descriptor version 1 (this architecture), layout type 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// the same with A and B as f16 (format code 0)
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// the same with A and B as tf32 (format code 2)
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- per-format dequantization of one weight row's 64-element K stage into 8 x 16-byte bf16 chunks ----
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// two f32 -> the packed 16-bit operand pair: bf16, or f16 (finite values beyond its range saturate to +-65504)
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
template <bool kF16>
__device__ __forceinline__ uint32_t pack_op(float a, float b) {
  return kF16 ? pack_f16(a, b) : pack_bf16(a, b);
}
// exact small-integer -> float without a conversion instruction: 0x43000000 | q << 16 is 128 + q
__device__ __forceinline__ float small_int_f32(uint32_t q_at_bit16) { return __uint_as_float(0x43000000u | q_at_bit16); }

struct Q4KPrefill {
  static constexpr int kType = kQ4K;
  static constexpr bool kSplitLoad = true;
  // the bytes of one 64-wide stage of a row: block header and 32 bytes of nibbles
  struct Raw {
    uint4 hdr, qa, qb;
  };
  // ... and of one 16-element quarter of it (part = 2 * half + quarter: half 0 = low nibbles = elements 0..31,
  // quarter = which 16 bytes of the 32): header and 16 bytes of nibbles
  struct RawQ {
    uint4 hdr, q;
  };
  __device__ __forceinline__ static void load_part(const uint8_t* row, int it, int part, RawQ& r) {
    const int blk = it >> 2, g = it & 3;
    const uint8_t* b = row + blk * Q4KL::kBytes;
    r.hdr = *reinterpret_cast<const uint4*>(b);
    r.q = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 32 * g + 16 * (part & 1));
  }
  // -> two 16-byte chunks: elements 32 * half + 16 * quarter + (0..15) of the stage
  template <bool kF16>
  __device__ __forceinline__ static void convert_part(const RawQ& r, int it, int part, uint4 (&out)[2]) {
    const int g = it & 3, half = part >> 1;
    const uint4 hdr = r.hdr;
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    const uint32_t sh = 16 * (g & 1) + 8 * half;
    uint32_t sc, mn;
    if (g < 2) {
      sc = (hdr.y >> sh) & 0x3fu;
      mn = (hdr.z >> sh) & 0x3fu;
    } else {
      sc = ((hdr.w >> sh) & 0x0fu) | (((hdr.y >> (sh + 6)) & 0x03u) << 4);
      mn = ((hdr.w >> (sh + 4)) & 0x0fu) | (((hdr.z >> (sh + 6)) & 0x03u) << 4);
    }
    const float d1 = d * (float)sc;
    const float c1 = -(dmin * (float)mn) - 128.0f * d1;  // y = d*sc*q - dmin*m, with q taken as (128 + q) - 128
    const uint32_t w[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
    const uint32_t nsh = 4 * half;
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // word j holds bytes 4j..4j+3 -> elements 4j..4j+3 of this quarter
      const uint32_t v = w[j] >> nsh;
      const float l0 = fmaf(d1, small_int_f32((v << 16) & 0x000f0000u), c1), l1 = fmaf(d1, small_int_f32((v << 8) & 0x000f0000u), c1);
      const float l2 = fmaf(d1, small_int_f32(v & 0x000f0000u), c1), l3 = fmaf(d1, small_int_f32((v >> 8) & 0x000f0000u), c1);
      uint32_t* o = reinterpret_cast<uint32_t*>(&out[j >> 1]) + 2 * (j & 1);
      o[0] = pack_op<kF16>(l0, l1), o[1] = pack_op<kF16>(l2, l3);
    }
  }
  // k0 = 64 * it: block it / 4, group it % 4; row points at the weight row's first block
  __device__ __forceinline__ static void load(const uint8_t* row, int it, Raw& r) {
    const int blk = it >> 2, g = it & 3;
    const uint8_t* b = row + blk * Q4KL::kBytes;
    r.hdr = *reinterpret_cast<const uint4*>(b);
    r.qa = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 32 * g);
    r.qb = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 32 * g + 16);
  }
  // one 32-element half of the stage (half 0: low nibbles, elements 0..31; half 1: high nibbles) -> 4 chunks
  template <bool kF16>
  __device__ __forceinline__ static void convert_half(const Raw& r, int it, int half, uint4 (&out)[4]) {
    RawQ q;
    q.hdr = r.hdr;
    uint4 o2[2];
    q.q = r.qa;
    convert_part<kF16>(q, it, 2 * half, o2);
    out[0] = o2[0], out[1] = o2[1];
    q.q = r.qb;
    convert_part<kF16>(q, it, 2 * half + 1, o2);
    out[2] = o2[0], out[3] = o2[1];
  }
  // tf32 form: stage `it` is ONE 32-element sub-block (block it / 8, sub-block it % 8); part = which 16 of them.
  // Values are the exact f32 dequantization rounded to tf32.
  __device__ __forceinline__ static void stage16(const uint8_t* row, int it, int part, uint4 (&out)[4]) {
    const int blk = it >> 3, j = it & 7, g = j >> 1, nib = j & 1;
    const uint8_t* b = row + blk * Q4KL::kBytes;
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);
    const uint4 q = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 32 * g + 16 * part);
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    const uint32_t sh = 16 * (g & 1) + 8 * nib;
    uint32_t sc, mn;
    if (g < 2) {
      sc = (hdr.y >> sh) & 0x3fu;
      mn = (hdr.z >> sh) & 0x3fu;
    } else {
      sc = ((hdr.w >> sh) & 0x0fu) | (((hdr.y >> (sh + 6)) & 0x03u) << 4);
      mn = ((hdr.w >> (sh + 4)) & 0x0fu) | (((hdr.z >> (sh + 6)) & 0x03u) << 4);
    }
    const float d1 = d * (float)sc, m1 = dmin * (float)mn;
    const uint32_t w[4] = {q.x >> (4 * nib), q.y >> (4 * nib), q.z >> (4 * nib), q.w >> (4 * nib)};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      out[c].x = to_tf32(d1 * (float)(w[c] & 0xf) - m1), out[c].y = to_tf32(d1 * (float)((w[c] >> 8) & 0xf) - m1);
      out[c].z = to_tf32(d1 * (float)((w[c] >> 16) & 0xf) - m1), out[c].w = to_tf32(d1 * (float)((w[c] >> 24) & 0xf) - m1);
    }
  }
  __device__ __forceinline__ static void stage(const uint8_t* row, int it, uint4 (&out)[8]) {
    Raw r;
    load(row, it, r);
    convert<false>(r, it, out);
  }
  template <bool kF16>
  __device__ __forceinline__ static void convert(const Raw& r, int it, uint4 (&out)[8]) {
    const int g = it & 3;
    const uint4 hdr = r.hdr, qa = r.qa, qb = r.qb;
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    const uint32_t sh = 16 * (g & 1);
    uint32_t sc2, mn2;
    if (g < 2) {
      sc2 = (hdr.y >> sh) & 0x3f3fu;
      mn2 = (hdr.z >> sh) & 0x3f3fu;
    } else {
      sc2 = ((hdr.w >> sh) & 0x0f0fu) | (((hdr.y >> (sh + 6)) & 0x0303u) << 4);
      mn2 = ((hdr.w >> (sh + 4)) & 0x0f0fu) | (((hdr.z >> (sh + 6)) & 0x0303u) << 4);
    }
    const float d1 = d * (float)(sc2 & 0xff), d2 = d * (float)(sc2 >> 8);
    // y = d*sc*q - dmin*m, with q taken as (128 + q) - 128
    const float c1 = -(dmin * (float)(mn2 & 0xff)) - 128.0f * d1, c2 = -(dmin * (float)(mn2 >> 8)) - 128.0f * d2;
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // word j holds bytes 4j..4j+3: low nibbles -> k = 4j.., high -> k = 32 + 4j..
      const uint32_t v = w[j];
      const float l0 = fmaf(d1, small_int_f32((v << 16) & 0x000f0000u), c1), l1 = fmaf(d1, small_int_f32((v << 8) & 0x000f0000u), c1);
      const float l2 = fmaf(d1, small_int_f32(v & 0x000f0000u), c1), l3 = fmaf(d1, small_int_f32((v >> 8) & 0x000f0000u), c1);
      const float h0 = fmaf(d2, small_int_f32((v << 12) & 0x000f0000u), c2), h1 = fmaf(d2, small_int_f32((v << 4) & 0x000f0000u), c2);
      const float h2 = fmaf(d2, small_int_f32((v >> 4) & 0x000f0000u), c2), h3 = fmaf(d2, small_int_f32((v >> 12) & 0x000f0000u), c2);
      uint32_t* lo = reinterpret_cast<uint32_t*>(&out[j >> 1]) + 2 * (j & 1);       // chunk j/2 (k = 8*(j/2)..)
      uint32_t* hi = reinterpret_cast<uint32_t*>(&out[4 + (j >> 1)]) + 2 * (j & 1);  // chunk 4 + j/2
      lo[0] = pack_op<kF16>(l0, l1), lo[1] = pack_op<kF16>(l2, l3);
      hi[0] = pack_op<kF16>(h0, h1), hi[1] = pack_op<kF16>(h2, h3);
    }
  }
};

// Q8_0: a 64-wide stage is two 34-byte blocks (2-byte aligned): y = q * d
struct Q8_0Prefill {
  static constexpr int kType = kQ8_0;
  static constexpr bool kSplitLoad = false;
  struct Raw {};
  __device__ __forceinline__ static void load(const uint8_t*, int, Raw&) {}
  __device__ __forceinline__ static void convert(const Raw&, int, uint4 (&)[8]) {}
  __device__ __forceinline__ static void convert_half(const Raw&, int, int, uint4 (&)[4]) {}
  // tf32 form: stage `it` is block `it`; part = which 16 of its 32 elements
  __device__ __forceinline__ static void stage16(const uint8_t* row, int it, int part, uint4 (&out)[4]) {
    const uint8_t* b = row + (size_t)it * Q8_0L::kBytes;
    const float d = h2f_bits(ldg_u16(b));
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t v0 = ldg_u16(b + Q8_0L::kOffQs + 16 * part + 4 * c), v1 = ldg_u16(b + Q8_0L::kOffQs + 16 * part + 4 * c + 2);
      out[c].x = to_tf32((float)(int8_t)(v0 & 0xff) * d), out[c].y = to_tf32((float)(int8_t)(v0 >> 8) * d);
      out[c].z = to_tf32((float)(int8_t)(v1 & 0xff) * d), out[c].w = to_tf32((float)(int8_t)(v1 >> 8) * d);
    }
  }
  // half of a 64-wide stage = one 34-byte block: part p is block 2 * it + p -> chunks 4p .. 4p + 3
  __device__ __forceinline__ static int chunk_id(int part, int c) { return 4 * part + c; }
  template <bool kF16>
  __device__ __forceinline__ static void stage_half(const uint8_t* row, int it, int part, uint4 (&out)[4]) {
    const uint8_t* b = row + (size_t)(2 * it + part) * Q8_0L::kBytes;
    const float d = h2f_bits(ldg_u16(b));
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // 4 values per j -> two packed words
      const uint32_t v0 = ldg_u16(b + Q8_0L::kOffQs + 4 * j), v1 = ldg_u16(b + Q8_0L::kOffQs + 4 * j + 2);
      const float f0 = (float)(int8_t)(v0 & 0xff) * d, f1 = (float)(int8_t)(v0 >> 8) * d;
      const float f2 = (float)(int8_t)(v1 & 0xff) * d, f3 = (float)(int8_t)(v1 >> 8) * d;
      uint32_t* o = reinterpret_cast<uint32_t*>(&out[j >> 1]) + 2 * (j & 1);
      o[0] = pack_op<kF16>(f0, f1), o[1] = pack_op<kF16>(f2, f3);
    }
  }
  template <bool kF16>
  __device__ __forceinline__ static void stage(const uint8_t* row, int it, uint4 (&out)[8]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint8_t* b = row + (size_t)(2 * it + h) * Q8_0L::kBytes;
      const float d = h2f_bits(ldg_u16(b));
#pragma unroll
      for (int j = 0; j < 8; ++j) {  // 4 values per j -> two packed words
        const uint32_t v0 = ldg_u16(b + Q8_0L::kOffQs + 4 * j), v1 = ldg_u16(b + Q8_0L::kOffQs + 4 * j + 2);
        const float f0 = (float)(int8_t)(v0 & 0xff) * d, f1 = (float)(int8_t)(v0 >> 8) * d;
        const float f2 = (float)(int8_t)(v1 & 0xff) * d, f3 = (float)(int8_t)(v1 >> 8) * d;
        uint32_t* o = reinterpret_cast<uint32_t*>(&out[4 * h + (j >> 1)]) + 2 * (j & 1);
        o[0] = pack_op<kF16>(f0, f1), o[1] = pack_op<kF16>(f2, f3);
      }
    }
  }
};

// Q6_K: a 64-wide stage is a quarter super-block: half = elements 128*half.., sub selects low (l, l+32)
// or high (l+64, l+96) nibbles of the same 64 ql bytes; y = d * sc * (q - 32)
struct Q6KPrefill {
  static constexpr int kType = kQ6K;
  static constexpr bool kSplitLoad = false;
  struct Raw {};
  __device__ __forceinline__ static void load(const uint8_t*, int, Raw&) {}
  __device__ __forceinline__ static void convert(const Raw&, int, uint4 (&)[8]) {}
  __device__ __forceinline__ static void convert_half(const Raw&, int, int, uint4 (&)[4]) {}
  // tf32 form: stage `it` is 32 consecutive elements: block it / 8, half (it / 4) % 2, quad it % 4 (elements
  // 128*half + 32*quad + l); part = which 16 of them (l = 16*part ..), which share one scale
  __device__ __forceinline__ static void stage16(const uint8_t* row, int it, int part, uint4 (&out)[4]) {
    const int blk = it >> 3, half = (it >> 2) & 1, quad = it & 3;
    const uint8_t* b = row + (size_t)blk * Q6KL::kBytes;
    const float d = h2f_bits(ldg_u16(b + Q6KL::kOffD));
    const uint8_t* ql = b + Q6KL::kOffQl + 64 * half + 32 * (quad & 1) + 16 * part;
    const uint8_t* qh = b + Q6KL::kOffQh + 32 * half + 16 * part;
    const int sci = 8 * half + 2 * quad + part;  // scale index: 8*half + l/16 + 2*quad
    const uint32_t scw = ldg_u16(b + Q6KL::kOffScales + (sci & ~1));
    const float s = d * (float)(int8_t)((scw >> (8 * (sci & 1))) & 0xff);
    const int nsh = 4 * (quad >> 1), hsh = 2 * quad;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t vals[4];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const uint32_t a = ldg_u16(ql + 4 * c + 2 * h2), h = ldg_u16(qh + 4 * c + 2 * h2);
        const int q0 = (int)(((a & 0xff) >> nsh) & 0xf) | (int)((((h & 0xff) >> hsh) & 3) << 4);
        const int q1 = (int)(((a >> 8) >> nsh) & 0xf) | (int)((((h >> 8) >> hsh) & 3) << 4);
        vals[2 * h2] = to_tf32(s * (float)(q0 - 32)), vals[2 * h2 + 1] = to_tf32(s * (float)(q1 - 32));
      }
      out[c] = make_uint4(vals[0], vals[1], vals[2], vals[3]);
    }
  }
  // half of a 64-wide stage: part p takes l = 16p .. 16p + 15, i.e. elements l of the first 32 (chunks 2p, 2p + 1)
  // and the same l of the second 32 (chunks 4 + 2p, 5 + 2p); one scale each
  __device__ __forceinline__ static int chunk_id(int part, int c) { return c < 2 ? 2 * part + c : 4 + 2 * part + (c - 2); }
  template <bool kF16>
  __device__ __forceinline__ static void stage_half(const uint8_t* row, int it, int part, uint4 (&out)[4]) {
    const int blk = it >> 2, half = (it >> 1) & 1, sub = it & 1;
    const uint8_t* b = row + (size_t)blk * Q6KL::kBytes;
    const float d = h2f_bits(ldg_u16(b + Q6KL::kOffD));
    const uint8_t* ql = b + Q6KL::kOffQl + 64 * half + 16 * part;
    const uint8_t* qh = b + Q6KL::kOffQh + 32 * half + 16 * part;
    const uint32_t scw0 = ldg_u16(b + Q6KL::kOffScales + 8 * half + 4 * sub), scw1 = ldg_u16(b + Q6KL::kOffScales + 8 * half + 4 * sub + 2);
    const float sa = d * (float)(int8_t)((scw0 >> (8 * part)) & 0xff), sb = d * (float)(int8_t)((scw1 >> (8 * part)) & 0xff);
    const int nsh = 4 * sub, hsh = 4 * sub;
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // two l values per j
      const uint32_t a = ldg_u16(ql + 2 * j), c = ldg_u16(ql + 32 + 2 * j), h = ldg_u16(qh + 2 * j);
      const int a0 = a & 0xff, a1 = a >> 8, c0 = c & 0xff, c1 = c >> 8, h0 = h & 0xff, h1 = h >> 8;
      const int qa0 = (((a0 >> nsh) & 0xF) | (((h0 >> hsh) & 3) << 4)) - 32, qa1 = (((a1 >> nsh) & 0xF) | (((h1 >> hsh) & 3) << 4)) - 32;
      const int qc0 = (((c0 >> nsh) & 0xF) | (((h0 >> (hsh + 2)) & 3) << 4)) - 32, qc1 = (((c1 >> nsh) & 0xF) | (((h1 >> (hsh + 2)) & 3) << 4)) - 32;
      reinterpret_cast<uint32_t*>(&out[j >> 2])[j & 3] = pack_op<kF16>(sa * (float)qa0, sa * (float)qa1);
      reinterpret_cast<uint32_t*>(&out[2 + (j >> 2)])[j & 3] = pack_op<kF16>(sb * (float)qc0, sb * (float)qc1);
    }
  }
  template <bool kF16>
  __device__ __forceinline__ static void stage(const uint8_t* row, int it, uint4 (&out)[8]) {
    const int blk = it >> 2, half = (it >> 1) & 1, sub = it & 1;
    const uint8_t* b = row + (size_t)blk * Q6KL::kBytes;
    const float d = h2f_bits(ldg_u16(b + Q6KL::kOffD));
    const uint8_t* ql = b + Q6KL::kOffQl + 64 * half;
    const uint8_t* qh = b + Q6KL::kOffQh + 32 * half;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + Q6KL::kOffScales + 8 * half + 4 * sub);
    // scales for elements [0,16) [16,32) of the first 32 and of the second 32
    const float s00 = d * (float)sc[0], s01 = d * (float)sc[1], s10 = d * (float)sc[2], s11 = d * (float)sc[3];
    const int nsh = 4 * sub, hsh = 4 * sub;  // nibble shift in ql, bit-pair shift in qh (pairs 2*sub, 2*sub+1)
#pragma unroll
    for (int j = 0; j < 16; ++j) {  // two l values per j
      const uint32_t a = ldg_u16(ql + 2 * j), c = ldg_u16(ql + 32 + 2 * j), h = ldg_u16(qh + 2 * j);
      const int a0 = a & 0xff, a1 = a >> 8, c0 = c & 0xff, c1 = c >> 8, h0 = h & 0xff, h1 = h >> 8;
      const int qa0 = (((a0 >> nsh) & 0xF) | (((h0 >> hsh) & 3) << 4)) - 32, qa1 = (((a1 >> nsh) & 0xF) | (((h1 >> hsh) & 3) << 4)) - 32;
      const int qc0 = (((c0 >> nsh) & 0xF) | (((h0 >> (hsh + 2)) & 3) << 4)) - 32, qc1 = (((c1 >> nsh) & 0xF) | (((h1 >> (hsh + 2)) & 3) << 4)) - 32;
      const float sa = j < 8 ? s00 : s01, sb = j < 8 ? s10 : s11;
      // first 32 elements of the stage: l = 2j, 2j+1 ; second 32: the same l from the other ql half
      reinterpret_cast<uint32_t*>(&out[j >> 2])[j & 3] = pack_op<kF16>(sa * (float)qa0, sa * (float)qa1);
      reinterpret_cast<uint32_t*>(&out[4 + (j >> 2)])[j & 3] = pack_op<kF16>(sb * (float)qc0, sb * (float)qc1);
    }
  }
};

struct PrefillSmem {
  uint64_t full[kPfStages];   // weight tile of the stage written (the dequantizing threads)
  uint64_t xfull[kPfStages];  // activation tile of the stage landed (tensor-map copy, counted in bytes)
  uint64_t empty[kPfStages];
  uint64_t accum;
  uint32_t tmem_base;
  int abort_flag;
};

// kTf32: operands in tf32 instead of bf16 - stages are 32 wide (one 128-byte row of f32), activations are the f32
// matrix rounded to tf32 by the pre-pass, half the MMA rate, about eight times smaller rounding error.
// kMulti: the epilogue stores every tile into several destinations (column-sharded across GPUs).
// kF16 (not with kTf32): 16-bit operands are f16 instead of bf16 - three more mantissa bits at the same MMA rate. The
// weights' range fits (finite values saturate at +-65504); the activation rows arrive scaled by a power of two
// into f16's range and p.row_unscale[m] undoes it in the epilogue.
template <class Fmt, int kTileM, bool kTf32 = false, bool kMulti = false, bool kF16 = false>
__global__ void __launch_bounds__(kPfThreads, 1) prefill_gemm_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap xmap) {
  extern __shared__ __align__(1024) uint8_t pf_smem[];
  // [stage][ weights 128 x 128 B | activations kTileM x 128 B ], each 1024-byte aligned; control block after
  constexpr int kWBytes = kPfTileN * 128, kXBytes = kTileM * 128, kStageBytes = kWBytes + kXBytes;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_smem) + 1023) & ~(uintptr_t)1023);
  PrefillSmem* sm = reinterpret_cast<PrefillSmem*>(base + kPfStages * kStageBytes);
  const uint32_t base_u32 = smem_u32(base);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kPfTileN, m0 = blockIdx.y * kTileM;
  constexpr int kStageK = kTf32 ? 32 : kPfTileK;  // elements per 128-byte row
  const int n_iter = p.K / kStageK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(&sm->full[s], 32 * kPfDequantWarps);  // the dequantizing threads
      mbar_init(&sm->xfull[s], 1);                    // the thread that issues the activation copy (plus its bytes)
      mbar_init(&sm->empty[s], 1);   // one commit from the MMA thread
    }
    mbar_init(&sm->accum, 1);
    sm->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kPfDequantWarps) tmem_alloc(&sm->tmem_base, kTileM);  // kTileM f32 accumulator columns x 128 lanes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *reinterpret_cast<volatile uint32_t*>(&sm->tmem_base);
  volatile int* abort_flag = &sm->abort_flag;

  if (warp < kPfDequantWarps) {
    // ---------------- weight producers: thread t owns half (t >> 7) of weight row n0 + (t & 127)
    const int t = threadIdx.x, r = t & 127, part = t >> 7;
    const bool live = n0 + r < p.N;
    const uint8_t* row = p.w + (size_t)(live ? n0 + r : 0) * p.row_bytes;
    int s = 0;
    uint32_t ph = 0;
    int x_issued = 0;
    // the bytes of the next three stages, requested that far ahead: a stage takes less time than one trip to L2
    using RawT = typename Fmt::Raw;
    auto load_raw = [&](int it, RawT& dst_raw) { Fmt::load(row, it, dst_raw); };
    RawT r0, r1, r2;
    if (!kTf32 && Fmt::kSplitLoad && live) {
      if (n_iter > 0) load_raw(0, r0);
      if (n_iter > 1) load_raw(1, r1);
      if (n_iter > 2) load_raw(2, r2);
    }
    for (int it = 0; it < n_iter && !*abort_flag; ++it) {
      if (it >= kPfStages && !mbar_wait_bounded(&sm->empty[s], ph ^ 1u)) {
        record_dev_error(kErrEmptyWait);
        *abort_flag = 1;
        break;
      }
      if (t == 0) {  // the stage is free: its activation tile, rows m0.. x columns 64*it.., as one copy
        mbar_arrive_expect_tx(&sm->xfull[s], (uint32_t)kXBytes);
        tma_load_2d(base_u32 + s * kStageBytes + kWBytes, &xmap, it * kStageK, m0, &sm->xfull[s]);
        x_issued = it + 1;
      }
      uint8_t* dst = base + s * kStageBytes + r * 128;
      if constexpr (kTf32) {
        static_assert(!kTf32 || kPfDequantWarps == 8, "the tf32 form splits a row's 32 elements between two threads");
        uint4 out[4];
        if (live) {
          Fmt::stage16(row, it, part, out);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + (((4 * part + c) ^ (r & 7)) << 4)) = out[c];
      } else if constexpr (Fmt::kSplitLoad) {
        constexpr int kChunks = 4;  // 16-byte chunks this thread writes
        uint4 out[4];
        if (live) {
          const RawT cur = r0;
          r0 = r1;
          r1 = r2;
          if (it + 3 < n_iter) load_raw(it + 3, r2);
          Fmt::template convert_half<kF16>(cur, it, part, out);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < kChunks; ++c) *reinterpret_cast<uint4*>(dst + (((kChunks * part + c) ^ (r & 7)) << 4)) = out[c];
      } else {  // the other formats: each of the row's two threads dequantizes half of the stage
        uint4 out[4];
        if (live) {
          Fmt::template stage_half<kF16>(row, it, part, out);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + ((Fmt::chunk_id(part, c) ^ (r & 7)) << 4)) = out[c];
      }
      fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's reads
      mbar_arrive(&sm->full[s]);
      if (++s == kPfStages) s = 0, ph ^= 1u;
    }
    if (t == 0 && *abort_flag) {  // leaving early: let the copies already issued land first
      for (int it = (x_issued > kPfStages ? x_issued - kPfStages : 0); it < x_issued; ++it)
        if (!mbar_wait_bounded(&sm->xfull[it % kPfStages], (it / kPfStages) & 1)) record_dev_error(kErrDrainWait);
    }
  } else if (lane == 0) {
    // ---------------- MMA issue: one thread
    constexpr uint32_t idesc = kTf32 ? umma_idesc_tf32(kPfTileN, kTileM) : kF16 ? umma_idesc_f16(kPfTileN, kTileM) : umma_idesc_bf16(kPfTileN, kTileM);
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      if (*abort_flag || !mbar_wait_bounded(&sm->full[s], ph) || !mbar_wait_bounded(&sm->xfull[s], ph)) {
        if (!*abort_flag) record_dev_error(kErrFullWait);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t a_addr = base_u32 + s * kStageBytes, b_addr = a_addr + kWBytes;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // 32 bytes along K per instruction: 16 bf16 or 8 tf32
        if constexpr (kTf32)
          umma_tf32(tmem_d, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc, (it | kk) != 0);
        else
          umma_bf16(tmem_d, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc, (it | kk) != 0);
      }
      umma_commit(&sm->empty[s]);  // frees the stage once these MMAs have read it
      if (++s == kPfStages) s = 0, ph ^= 1u;
    }
    if (ok) umma_commit(&sm->accum);  // accumulator complete
  }

  // ---------------- epilogue: warps 0-3 read their 32 TMEM lanes (weight rows) and store Y
  if (warp < 4) {
    bool ready = !*abort_flag;
    if (ready && !mbar_wait_bounded(&sm->accum, 0)) {
      record_dev_error(kErrMmaWait);
      *abort_flag = 1;
      ready = false;
    }
    ready = __all_sync(0xffffffffu, ready);
    if (ready) {
      tc_fence_after();
      const int n = n0 + warp * 32 + lane;
      // The accumulator arrives one weight row (output column) per lane; Y is row-major in the other direction. Each warp
      // turns 32 x 32 pieces around in shared memory (the stage buffers are free by now) so that it stores 16 bytes per
      // lane along a row of Y - four times fewer, four times larger stores, which matters most for the peers' copies.
      float* tbuf = reinterpret_cast<float*>(base) + warp * (32 * 36);  // [32 m][36]: rows 16-byte aligned, shifted banks
      // (measured: for a single local destination the direct 4-byte stores, already 128 bytes per warp, are faster)
      bool vec_ok = kMulti && p.n_dst > 1 && (p.ldy & 3) == 0 && (p.n_off & 3) == 0 && n0 + warp * 32 + 32 <= p.N;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < p.n_dst) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(p.y[q]) & 15) == 0;
      const int sub_m = lane >> 3, n4 = (lane & 7) * 4;
#pragma unroll 1
      for (int c = 0; c < kTileM / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), v);
        if constexpr (kF16) {  // undo the scaling of activation row m0 + 32c + j (a power of two: exact)
          const int ml = m0 + c * 32 + lane;
          const float mine = ml < p.M ? p.row_unscale[ml] : 1.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * __shfl_sync(0xffffffffu, mine, j));
        }
        if (kMulti && vec_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) tbuf[j * 36 + lane] = __uint_as_float(v[j]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int mm = sub_m + 4 * i, m = m0 + c * 32 + mm;
            if (m < p.M) {
              const float4 val = *reinterpret_cast<const float4*>(tbuf + mm * 36 + n4);
              // column-sharded across GPUs: the piece goes straight into every GPU's copy of Y (plain stores over
              // NVLink for the peers'), so the all-gather of the shards happens inside the epilogue
              const size_t off = (size_t)m * p.ldy + p.n_off + n0 + warp * 32 + n4;
#pragma unroll
              for (int q = 0; q < 8; ++q)  // constant indices: a runtime index would copy the pointer table to local memory
                if (q < p.n_dst) *reinterpret_cast<float4*>(p.y[q] + off) = val;
            }
          }
          __syncwarp();
        } else if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = m0 + c * 32 + j;
            if (m < p.M) {
              const size_t off = (size_t)m * p.ldy + p.n_off + n;
              p.y[0][off] = __uint_as_float(v[j]);
              if (kMulti && p.n_dst > 1) {
#pragma unroll
                for (int q = 1; q < 8; ++q)
                  if (q < p.n_dst) p.y[q][off] = __uint_as_float(v[j]);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kPfDequantWarps) tmem_dealloc(tmem_d, kTileM);
}

// f32 -> f32 rounded to tf32 (activation pre-pass of the tf32 form)
__global__ void __launch_bounds__(256) f32_to_tf32_kernel(const float* x, int64_t n4, float* y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    uint4 o;
    o.x = to_tf32(v.x), o.y = to_tf32(v.y), o.z = to_tf32(v.z), o.w = to_tf32(v.w);
    reinterpret_cast<uint4*>(y)[i] = o;
  }
}

// f32 -> f16 activation pre-pass, one thread block per row: the row is scaled by the power of two that brings its
// largest magnitude into [2^13, 2^14) (exact; keeps large rows finite and small rows out of the subnormals), and
// unscale[row] holds the inverse for the epilogue. Rows of zeros or with non-finite values are left unscaled.
__global__ void __launch_bounds__(256) f32_to_f16_rows_kernel(const float* __restrict__ x, int K, __half* __restrict__ y,
                                                              float* __restrict__ unscale) {
  __shared__ float red[8];
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * K);
  const int n4 = K >> 2;
  float amax = 0.f;
  for (int i = threadIdx.x; i < n4; i += 256) {
    const float4 v = src[i];
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  float scale = 1.0f, inv = 1.0f;
  if (amax > 0.f && amax <= 3.0e38f) {
    int e;
    frexpf(amax, &e);            // amax = f * 2^e, f in [0.5, 1)
    int sh = 14 - e;             // amax * 2^sh in [2^13, 2^14)
    sh = sh > 100 ? 100 : (sh < -100 ? -100 : sh);
    scale = ldexpf(1.0f, sh);
    inv = ldexpf(1.0f, -sh);
  }
  if (threadIdx.x == 0) unscale[blockIdx.x] = inv;
  uint2* dst = reinterpret_cast<uint2*>(y + (size_t)blockIdx.x * K);
  for (int i = threadIdx.x; i < n4; i += 256) {
    const float4 v = src[i];
    uint2 o;
    o.x = pack_f16(v.x * scale, v.y * scale);
    o.y = pack_f16(v.z * scale, v.w * scale);
    dst[i] = o;
  }
}

// f32 -> bf16 activation pre-pass
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ x, int64_t n4, __nv_bfloat16* __restrict__ y) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = reinterpret_cast<const float4*>(x)[i];
  uint2 o;
  o.x = pack_bf16(v.x, v.y);
  o.y = pack_bf16(v.z, v.w);
  reinterpret_cast<uint2*>(y)[i] = o;
}

}  // namespace fq
