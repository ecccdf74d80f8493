// Decode path (small M): fused dequant mat-vec  y[m, n] = sum_k W[n, k] * x[m, k]
// over GGUF blocks, bandwidth-bound. Replaces the reference's MMVQ calls
// (fuel-cuda-backend/src/quantized.rs:138-231) and computes what the CPU path's
// vec_dot computes (fuel-quantized/src/k_quants.rs:1388-1468, 1946-2003, 674-692,
// 252-269): integer dot products of packed weights with 8-bit activation blocks,
// scaled per block in f32.
//
// Structure (one CTA = 1 producer warp + kConsumerWarps):
//   * the weight matrix is a flat byte stream; each CTA owns a contiguous range of
//     rows and streams it through a ring of shared-memory stages with 1-D bulk TMA
//     copies (16-byte aligned source, the row's sub-16 skew is kept in the stage);
//   * consumer warps take (row, k-segment) items of a stage; each lane unpacks
//     16/12/32 bytes of weights from shared memory and runs dp4a against the
//     plane-split activation blocks (read through L1);
//   * per-item warp-shuffle reduction; rows cut into several k-segments are summed
//     in a fixed order from a small shared buffer, so results never depend on timing.
// Every wait is bounded: on expiry the kernel records a code and returns.
#pragma once
#include "fq_common.cuh"

namespace fq {

constexpr int kDecodeConsumerWarps = 8;
constexpr int kDecodeThreads = 32 * (kDecodeConsumerWarps + 1);
constexpr int kDecodeMaxStages = 8;
constexpr int kDecodeMaxItems = 64;   // rows_per_stage * nseg
constexpr int kDecodeMaxM = 16;

struct DecodeParams {
  const uint8_t* w;
  ActPlanes act;
  float* y;
  int64_t n;
  int64_t total_bytes;
  int k;
  int m;
  int row_bytes;
  int units_per_row;
  int rows_per_stage;
  int nseg;
  int num_stages;
  int stage_stride;  // bytes between stage buffers (multiple of 128)
};

// ------------------------------------------------------------------ per-format inner loops
// unit(): one lane's share of one row: accumulate into acc[0..MT) for activation rows m0..m0+mc.

struct Q4KDecode {
  static constexpr int kUnitsPerBlock = 8;  // 16 bytes of nibbles each
  static constexpr int kBlockElems = 256;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const int blk = u >> 3, cc = u & 7, g = cc >> 1, h = cc & 1;
    const uint8_t* b = rowp + blk * Q4KL::kBytes;
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);
    const uint4 qv = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 16 * cc);
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    // 6-bit scales / mins of sub-blocks 2g and 2g+1 (get_scale_min_k4, fuel-quantized/src/utils.rs:50-60)
    uint32_t scw, mnw;
    if (g < 2) {
      scw = hdr.y & 0x3f3f3f3fu;
      mnw = hdr.z & 0x3f3f3f3fu;
    } else {
      scw = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
      mnw = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    }
    const int sh = (g & 1) * 16;
    const int sc_lo = (scw >> sh) & 0xff, sc_hi = (scw >> (sh + 8)) & 0xff;
    const int mn_lo = (mnw >> sh) & 0xff, mn_hi = (mnw >> (sh + 8)) & 0xff;
    const int l0 = qv.x & 0x0f0f0f0f, l1 = qv.y & 0x0f0f0f0f, l2 = qv.z & 0x0f0f0f0f, l3 = qv.w & 0x0f0f0f0f;
    const int h0 = (qv.x >> 4) & 0x0f0f0f0f, h1 = (qv.y >> 4) & 0x0f0f0f0f, h2 = (qv.z >> 4) & 0x0f0f0f0f,
              h3 = (qv.w >> 4) & 0x0f0f0f0f;
    const int nblk = k >> 8;
    const int eoff = blk * 256 + 64 * g + 16 * h;  // low nibbles: elements eoff..eoff+15, high: +32
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int8_t* q8 = a.qs + (size_t)m * k + eoff;
        const int4 alo = *reinterpret_cast<const int4*>(q8);
        const int4 ahi = *reinterpret_cast<const int4*>(q8 + 32);
        int dl = dp4a_ss(l0, alo.x, 0);
        dl = dp4a_ss(l1, alo.y, dl);
        dl = dp4a_ss(l2, alo.z, dl);
        dl = dp4a_ss(l3, alo.w, dl);
        int dh = dp4a_ss(h0, ahi.x, 0);
        dh = dp4a_ss(h1, ahi.y, dh);
        dh = dp4a_ss(h2, ahi.z, dh);
        dh = dp4a_ss(h3, ahi.w, dh);
        const int16_t* bs = a.bsums + (size_t)m * (k >> 4) + blk * 16 + 4 * g + h;
        const int bl = bs[0], bh = bs[2];
        const float yd = a.d[(size_t)m * nblk + blk];
        acc[i] += (d * yd) * (float)(sc_lo * dl + sc_hi * dh) - (dmin * yd) * (float)(mn_lo * bl + mn_hi * bh);
      }
    }
  }
};

struct Q6KDecode {
  static constexpr int kUnitsPerBlock = 16;  // four consecutive l of one 128-half: 16 elements
  static constexpr int kBlockElems = 256;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const int blk = u >> 4, uu = u & 15, half = uu >> 3, l0 = (uu & 7) * 4;
    const uint8_t* b = rowp + blk * Q6KL::kBytes;
    const uint32_t ql_a = lds_u32_2b(b + Q6KL::kOffQl + 64 * half + l0);
    const uint32_t ql_b = lds_u32_2b(b + Q6KL::kOffQl + 64 * half + 32 + l0);
    const uint32_t qh = lds_u32_2b(b + Q6KL::kOffQh + 32 * half + l0);
    const float d = h2f_bits(lds_u16(b + Q6KL::kOffD));
    const int8_t* scp = reinterpret_cast<const int8_t*>(b + Q6KL::kOffScales + 8 * half + (l0 >> 4));
    const int s0 = scp[0], s1 = scp[2], s2 = scp[4], s3 = scp[6];
    // 6-bit values 0..63, minus 32, as packed signed bytes: ((q | 0x80) - 0x20) ^ 0x80 per byte
    auto center = [](uint32_t q) -> int { return (int)(((q | 0x80808080u) - 0x20202020u) ^ 0x80808080u); };
    const int q1 = center((ql_a & 0x0f0f0f0fu) | ((qh & 0x03030303u) << 4));
    const int q2 = center((ql_b & 0x0f0f0f0fu) | (((qh >> 2) & 0x03030303u) << 4));
    const int q3 = center(((ql_a >> 4) & 0x0f0f0f0fu) | (((qh >> 4) & 0x03030303u) << 4));
    const int q4 = center(((ql_b >> 4) & 0x0f0f0f0fu) | (((qh >> 6) & 0x03030303u) << 4));
    const int nblk = k >> 8;
    const int eoff = blk * 256 + 128 * half + l0;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int* q8 = reinterpret_cast<const int*>(a.qs + (size_t)m * k + eoff);
        int s = s0 * dp4a_ss(q1, q8[0], 0);
        s += s1 * dp4a_ss(q2, q8[8], 0);
        s += s2 * dp4a_ss(q3, q8[16], 0);
        s += s3 * dp4a_ss(q4, q8[24], 0);
        acc[i] += (d * a.d[(size_t)m * nblk + blk]) * (float)s;
      }
    }
  }
};

struct Q8_0Decode {
  static constexpr int kUnitsPerBlock = 1;  // one 34-byte block
  static constexpr int kBlockElems = 32;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const uint8_t* b = rowp + u * Q8_0L::kBytes;
    const float d = h2f_bits(lds_u16(b));
    int w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = (int)lds_u32_2b(b + Q8_0L::kOffQs + 4 * j);
    const int nblk = k >> 5;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + u * 32);
        const int4 a0 = q8[0], a1 = q8[1];
        int s = dp4a_ss(w[0], a0.x, 0);
        s = dp4a_ss(w[1], a0.y, s);
        s = dp4a_ss(w[2], a0.z, s);
        s = dp4a_ss(w[3], a0.w, s);
        s = dp4a_ss(w[4], a1.x, s);
        s = dp4a_ss(w[5], a1.y, s);
        s = dp4a_ss(w[6], a1.z, s);
        s = dp4a_ss(w[7], a1.w, s);
        acc[i] += (d * a.d[(size_t)m * nblk + u]) * (float)s;
      }
    }
  }
};

struct Q4_0Decode {
  static constexpr int kUnitsPerBlock = 1;  // one 18-byte block: nibble j -> element j (low) / j+16 (high), minus 8
  static constexpr int kBlockElems = 32;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const uint8_t* b = rowp + u * Q4_0L::kBytes;
    const float d = h2f_bits(lds_u16(b));
    int lo[4], hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t v = lds_u32_2b(b + Q4_0L::kOffQs + 4 * j);
      // nibble - 8 per byte, as signed bytes: values 0..15 -> -8..7
      lo[j] = (int)((((v & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
      hi[j] = (int)(((((v >> 4) & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u);
    }
    const int nblk = k >> 5;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + u * 32);
        const int4 a0 = q8[0], a1 = q8[1];
        int s = dp4a_ss(lo[0], a0.x, 0);
        s = dp4a_ss(lo[1], a0.y, s);
        s = dp4a_ss(lo[2], a0.z, s);
        s = dp4a_ss(lo[3], a0.w, s);
        s = dp4a_ss(hi[0], a1.x, s);
        s = dp4a_ss(hi[1], a1.y, s);
        s = dp4a_ss(hi[2], a1.z, s);
        s = dp4a_ss(hi[3], a1.w, s);
        acc[i] += (d * a.d[(size_t)m * nblk + u]) * (float)s;
      }
    }
  }
};

// The other 32-element formats (k_quants.rs:285-313 Q4_1, :401-422 Q5_0, :501-533 Q5_1): nibble j is element j (low)
// / j + 16 (high); Q5 adds bit j of the little-endian word qh as the fifth bit of element j; Q4_1 / Q5_1 are
// unsigned with a per-block minimum m, whose share of the dot product is m * s with the activation block's
// s = d * sum(q) (Q8_1, kept as an f32 plane in the slot Q8_K uses for its block sums).
template <class L, bool kFive, bool kMin>
struct Legacy32Decode {
  static constexpr int kUnitsPerBlock = 1;
  static constexpr int kBlockElems = 32;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const uint8_t* b = rowp + u * L::kBytes;
    // blocks of 20 and 24 bytes keep every field 4-byte aligned (rows and stage skews are multiples of 4): whole-word loads
    constexpr bool kWord = L::kBytes % 4 == 0;
    auto word = [&](int off) -> uint32_t {
      if constexpr (kWord) return *reinterpret_cast<const uint32_t*>(b + off);
      else return lds_u32_2b(b + off);
    };
    float d, mval = 0.f;
    if constexpr (kMin) {
      const uint32_t dm = word(0);
      d = h2f_bits(dm & 0xffffu), mval = h2f_bits(dm >> 16);
    } else {
      d = h2f_bits(lds_u16(b));
    }
    uint32_t qh = 0;
    if constexpr (kFive) qh = word(L::kBytes - 20);  // the four bytes before the nibbles
    int lo[4], hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t v = word(L::kBytes - 16 + 4 * j);
      uint32_t l = v & 0x0f0f0f0fu, h = (v >> 4) & 0x0f0f0f0fu;
      if constexpr (kFive) {
        // bits 4j..4j+3 of qh -> bit 4 of bytes 0..3 (elements 4j..4j+3); bits 16+4j.. for the high nibbles
        const uint32_t bl = (qh >> (4 * j)) & 0xfu, bh = (qh >> (16 + 4 * j)) & 0xfu;
        l |= ((bl & 1u) << 4) | ((bl & 2u) << 11) | ((bl & 4u) << 18) | ((bl & 8u) << 25);
        h |= ((bh & 1u) << 4) | ((bh & 2u) << 11) | ((bh & 4u) << 18) | ((bh & 8u) << 25);
      }
      if constexpr (kFive && !kMin) {  // Q5_0: value - 16 per byte, as signed bytes (0..31 -> -16..15)
        l = ((l | 0x80808080u) - 0x10101010u) ^ 0x80808080u;
        h = ((h | 0x80808080u) - 0x10101010u) ^ 0x80808080u;
      }
      lo[j] = (int)l, hi[j] = (int)h;
    }
    const int nblk = k >> 5;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + u * 32);
        const int4 a0 = q8[0], a1 = q8[1];
        int s = dp4a_ss(lo[0], a0.x, 0);
        s = dp4a_ss(lo[1], a0.y, s);
        s = dp4a_ss(lo[2], a0.z, s);
        s = dp4a_ss(lo[3], a0.w, s);
        s = dp4a_ss(hi[0], a1.x, s);
        s = dp4a_ss(hi[1], a1.y, s);
        s = dp4a_ss(hi[2], a1.z, s);
        s = dp4a_ss(hi[3], a1.w, s);
        float t = ((float)s * d) * a.d[(size_t)m * nblk + u];
        if constexpr (kMin) t += mval * reinterpret_cast<const float*>(a.bsums)[(size_t)m * nblk + u];
        acc[i] += t;
      }
    }
  }
};
using Q4_1Decode = Legacy32Decode<Q4_1L, false, true>;
using Q5_0Decode = Legacy32Decode<Q5_0L, true, false>;
using Q5_1Decode = Legacy32Decode<Q5_1L, true, true>;

// Q2_K and Q3_K (k_quants.rs:783-833, 1013-1133). Element e of a block sits in qs[32 * (e / 128) + e % 32] at bits
// 2 * ((e % 128) / 32); every 16 elements share scale e / 16. A unit is 16 bytes of qs = half a 128-element chunk:
// four 16-element runs (bit pairs j = 0..3) with scale indices 8c + 2j + h, against activation bytes 128c + 32j + 16h.
struct Q2KDecode {
  static constexpr int kUnitsPerBlock = 4;
  static constexpr int kBlockElems = 256;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const int blk = u >> 2, c = (u >> 1) & 1, h = u & 1;
    const uint8_t* b = rowp + blk * Q2KL::kBytes;   // 84-byte blocks: 4-byte aligned
    const uint32_t dd = *reinterpret_cast<const uint32_t*>(b + Q2KL::kOffD);
    const float d = h2f_bits(dd & 0xffffu), dmin = h2f_bits(dd >> 16);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = *reinterpret_cast<const uint32_t*>(b + Q2KL::kOffQs + 32 * c + 16 * h + 4 * i);
    int sc[4], mn[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t s = b[8 * c + 2 * j + h];
      sc[j] = (int)(s & 0xFu), mn[j] = (int)(s >> 4);
    }
    const int nblk = k >> 8;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int8_t* q8 = a.qs + (size_t)m * k + (size_t)blk * 256 + 128 * c + 16 * h;
        const int16_t* bs = a.bsums + (size_t)m * (k >> 4) + blk * 16 + 8 * c + h;
        int isum = 0, msum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int4 av = *reinterpret_cast<const int4*>(q8 + 32 * j);
          int s = dp4a_ss((int)((w[0] >> (2 * j)) & 0x03030303u), av.x, 0);
          s = dp4a_ss((int)((w[1] >> (2 * j)) & 0x03030303u), av.y, s);
          s = dp4a_ss((int)((w[2] >> (2 * j)) & 0x03030303u), av.z, s);
          s = dp4a_ss((int)((w[3] >> (2 * j)) & 0x03030303u), av.w, s);
          isum += sc[j] * s;
          msum += mn[j] * (int)bs[2 * j];
        }
        const float yd = a.d[(size_t)m * nblk + blk];
        acc[i] += (yd * d) * (float)isum - (yd * dmin) * (float)msum;
      }
    }
  }
};

struct Q3KDecode {
  static constexpr int kUnitsPerBlock = 4;
  static constexpr int kBlockElems = 256;
  template <int MT>
  __device__ __forceinline__ static void unit(const uint8_t* rowp, int u, const ActPlanes& a, int k, int m0, int mc,
                                              float (&acc)[MT]) {
    const int blk = u >> 2, c = (u >> 1) & 1, h = u & 1;
    const uint8_t* b = rowp + blk * Q3KL::kBytes;   // 110-byte blocks: 2-byte aligned
    const float d = h2f_bits(lds_u16(b + Q3KL::kOffD));
    uint32_t w[4], hm[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = lds_u32_2b(b + Q3KL::kOffQs + 32 * c + 16 * h + 4 * i);
      hm[i] = lds_u32_2b(b + Q3KL::kOffHmask + 16 * h + 4 * i);
    }
    // 6-bit scales (k_quants.rs:1095-1103): index is < 8: low nibble of byte is, else high nibble of byte is - 8;
    // two more bits from byte 8 + is % 4 at 2 * (is / 4)
    int sc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int is = 8 * c + 2 * j + h;
      const uint32_t lo = is < 8 ? (b[Q3KL::kOffScales + is] & 0xFu) : (uint32_t)(b[Q3KL::kOffScales + is - 8] >> 4);
      const uint32_t hi = (b[Q3KL::kOffScales + 8 + (is & 3)] >> (2 * (is >> 2))) & 3u;
      sc[j] = (int)(lo | (hi << 4)) - 32;
    }
    const int nblk = k >> 8;
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i < mc) {
        const int m = m0 + i;
        const int8_t* q8 = a.qs + (size_t)m * k + (size_t)blk * 256 + 128 * c + 16 * h;
        const int16_t* bs = a.bsums + (size_t)m * (k >> 4) + blk * 16 + 8 * c + h;
        int isum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // value = low two bits - (high bit set ? 0 : 4) = (low | high << 2) - 4: unsigned bytes 0..7 against the
          // activations, minus four times the run's activation sum
          const int bit = 4 * c + j;
          const int4 av = *reinterpret_cast<const int4*>(q8 + 32 * j);
          int s = dp4a_ss((int)(((w[0] >> (2 * j)) & 0x03030303u) | (((hm[0] >> bit) & 0x01010101u) << 2)), av.x, 0);
          s = dp4a_ss((int)(((w[1] >> (2 * j)) & 0x03030303u) | (((hm[1] >> bit) & 0x01010101u) << 2)), av.y, s);
          s = dp4a_ss((int)(((w[2] >> (2 * j)) & 0x03030303u) | (((hm[2] >> bit) & 0x01010101u) << 2)), av.z, s);
          s = dp4a_ss((int)(((w[3] >> (2 * j)) & 0x03030303u) | (((hm[3] >> bit) & 0x01010101u) << 2)), av.w, s);
          isum += sc[j] * (s - 4 * (int)bs[2 * j]);
        }
        acc[i] += (d * a.d[(size_t)m * nblk + blk]) * (float)isum;
      }
    }
  }
};

// ------------------------------------------------------------------ the kernel
struct DecodeSmemHeader {
  uint64_t full[kDecodeMaxStages];
  uint64_t empty[kDecodeMaxStages];
  uint64_t part_ready[2];
  int abort_flag;
  int pad[3];
  float partial[2][kDecodeMaxItems][kDecodeMaxM];
};

template <class Fmt, int MT>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_matvec_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  DecodeSmemHeader* hd = reinterpret_cast<DecodeSmemHeader*>(smem_raw);
  uint8_t* stages = smem_raw + align_up(sizeof(DecodeSmemHeader), 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.num_stages, R = p.rows_per_stage;

  // this CTA's contiguous row range
  const int64_t r_begin = p.n * (int64_t)blockIdx.x / gridDim.x;
  const int64_t r_end = p.n * (int64_t)(blockIdx.x + 1) / gridDim.x;
  const int n_iter = (int)((r_end - r_begin + R - 1) / R);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hd->full[s], 1);
      mbar_init(&hd->empty[s], kDecodeConsumerWarps);
    }
    mbar_init(&hd->part_ready[0], kDecodeConsumerWarps);
    mbar_init(&hd->part_ready[1], kDecodeConsumerWarps);
    hd->abort_flag = 0;
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kDecodeConsumerWarps) {
    // ---------------- producer: weights never depend on the previous kernel, so no pdl_wait here
    if (lane == 0) {
      const int64_t tma_limit = p.total_bytes & ~(int64_t)15;
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % S;
        if (it >= S) {
          ok = mbar_wait_bounded(&hd->empty[s], ((it / S) - 1) & 1);
          if (!ok) {
            record_dev_error(kErrEmptyWait);
            break;
          }
        }
        const int64_t row0 = r_begin + (int64_t)it * R;
        const int64_t row1 = (row0 + R < r_end) ? row0 + R : r_end;
        const int64_t b0 = row0 * p.row_bytes, b1 = row1 * p.row_bytes;
        const int64_t a0 = b0 & ~(int64_t)15;
        int64_t a1 = (b1 + 15) & ~(int64_t)15;
        if (a1 > tma_limit) a1 = tma_limit;
        uint8_t* dst = stages + (size_t)s * p.stage_stride;
        if (b1 > a1) {  // matrix ends off a 16-byte boundary: last few bytes by hand
          const int64_t from = a1 > a0 ? a1 : a0;
          for (int64_t j = from; j < b1; ++j) dst[j - a0] = p.w[j];
        }
        if (a1 > a0) {
          mbar_arrive_expect_tx(&hd->full[s], (uint32_t)(a1 - a0));
          bulk_g2s(dst, p.w + a0, (uint32_t)(a1 - a0), &hd->full[s]);
        } else {
          mbar_arrive(&hd->full[s]);
        }
        issued = it + 1;
      }
      if (!ok) {
        // consumers stopped releasing stages: let our own copies land before leaving
        for (int it = (issued > S ? issued - S : 0); it < issued; ++it)
          if (!mbar_wait_bounded(&hd->full[it % S], (it / S) & 1)) record_dev_error(kErrDrainWait);
      }
    }
    pdl_wait();
    return;
  }

  // ---------------- consumers
  pdl_wait();  // activation blocks are written by the preceding kernel
  const int nseg = p.nseg;
  for (int it = 0; it < n_iter; ++it) {
    const int s = it % S;
    if (!mbar_wait_bounded(&hd->full[s], (it / S) & 1)) {
      record_dev_error(kErrFullWait);
      return;
    }
    const int64_t row0 = r_begin + (int64_t)it * R;
    const int rows_here = (int)((row0 + R < r_end ? row0 + R : r_end) - row0);
    const int skew = (int)((row0 * p.row_bytes) & 15);
    const uint8_t* sbase = stages + (size_t)s * p.stage_stride + skew;
    const int n_items = rows_here * nseg;
    const int buf = it & 1;
    for (int item = warp; item < n_items; item += kDecodeConsumerWarps) {
      const int r = item / nseg, seg = item - r * nseg;
      const int u0 = (int)((int64_t)p.units_per_row * seg / nseg);
      const int u1 = (int)((int64_t)p.units_per_row * (seg + 1) / nseg);
      const uint8_t* rowp = sbase + (size_t)r * p.row_bytes;
      for (int m0 = 0; m0 < p.m; m0 += MT) {
        const int mc = (p.m - m0 < MT) ? p.m - m0 : MT;
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[i] = 0.f;
        for (int u = u0 + lane; u < u1; u += 32) Fmt::template unit<MT>(rowp, u, p.act, p.k, m0, mc, acc);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
        }
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if (i < mc) {
              if (nseg == 1)
                p.y[(size_t)(m0 + i) * p.n + row0 + r] = acc[i];
              else
                hd->partial[buf][item][m0 + i] = acc[i];
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hd->empty[s]);
    if (nseg > 1) {
      // all consumer warps meet here (bounded), then sum the k-segments in fixed order
      if (lane == 0) mbar_arrive(&hd->part_ready[buf]);
      __syncwarp();  // reconverge first: lanes spinning below must not starve lane 0's arrive
      if (!mbar_wait_bounded(&hd->part_ready[buf], (it >> 1) & 1)) {
        record_dev_error(kErrFullWait);
        return;
      }
      for (int t = threadIdx.x; t < rows_here * p.m; t += 32 * kDecodeConsumerWarps) {
        const int r = t / p.m, m = t - r * p.m;
        float sum = hd->partial[buf][r * nseg][m];
        for (int sg = 1; sg < nseg; ++sg) sum += hd->partial[buf][r * nseg + sg][m];
        p.y[(size_t)m * p.n + row0 + r] = sum;
      }
    }
  }
}

}  // namespace fq
