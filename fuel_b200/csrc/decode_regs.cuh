// Decode mat-vec, register-resident activations (M = 1 or 2).
//
// Same job and same streaming structure as decode.cuh (a producer warp feeds a ring of
// shared-memory stages with 1-D bulk TMA copies of whole weight rows; bounded waits), but the
// inner loop is rebuilt around the instruction budget of an HBM-bound kernel: at ~23 bytes per
// clock per SM there are fewer than 90 issue slots for every 512 bytes of weights, so
//   * each lane owns fixed positions along k for the whole kernel and keeps the matching
//     8-bit activations, block sums and scales in registers (loaded once, after the
//     predecessor kernel is known to have finished) — no activation loads in the loop;
//   * a lane's unit is 64 bytes of nibbles (Q4_K: half a super-block, four sub-blocks), so one
//     header load and one 4-wide 6-bit scale decode are paid per 64 bytes; the mins term is
//     two dp2a instructions on packed int16 block sums;
//   * high nibbles are not shifted down: dp4a(unsigned bytes & 0xf0, act) gives 16x the
//     dot product, which is shifted once;
//   * every byte offset is a lane constant; per row only the row base changes.
// A row is handled by `ks` warps (k-slices) so that a lane never owns more than NU units;
// the slices of a row are summed in a fixed order from shared memory.
#pragma once
#include "decode.cuh"
#include "fq_common.cuh"
#include "peer.cuh"
#include "quantize_act.cuh"

namespace fq {

struct DecodeRegsParams {
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
  int ks;  // warps per row: 1, 2, 4 or 8
  int num_stages;
  int stage_stride;
  int depth;                      // copies a CTA keeps in flight (< num_stages)
  int pre_stages;                 // stages issued before the consumers hold their activations (0 = all)
  int rows_q, rows_rem;           // n / grid, n % grid: CTA c owns rows_q (+1 if c < rows_rem) rows
  int u_begin[9];                 // unit range of k-slice s: [u_begin[s], u_begin[s+1])
  const float* x_f32;             // not null: f32 activations [m][k]; every CTA quantizes them itself (Q8_K) into
  int act_smem_off;               //   plain planes at this byte offset of its shared memory, instead of reading `act`
  float* host_y;                  // not null (M = 1): the last CTA to finish copies y[0..n) here (device-mapped host memory)
  unsigned* host_done;            //   device word, zero at kernel start, counting finished CTAs
  // Tree form (kTree kernels): the row's k range is cut into n_leaves leaves (1, 2, 4 or 8) of leaf_u0[l+1] - leaf_u0[l]
  // units each; leaf l sits on lanes [l * leaf_lw, (l + 1) * leaf_lw) of the row's warps.
  int n_leaves, leaf_lw;
  int leaf_u0[9];
};

// Extra arguments of the tensor-parallel form (kPeer): the output rows go, as stamped pairs of exchange
// point ctx.push_seq, to dst[q] on every rank q (already offset to this rank's slice).
struct DecodeRegsPeer {
  PeerCtx ctx;
  uint2* dst[kPeerMaxWorld];
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// ---- Q4_K: unit = 64 bytes of nibbles = half a super-block (groups 2h, 2h+1: sub-blocks 4h..4h+3,
// elements 128h..128h+127). One header load and one 4-wide scale decode per 64 bytes.
struct Q4KRegs {
  static constexpr int kUnitsPerBlock = 2;
  struct Unit {
    uint32_t off_hdr, off_qs;  // byte offsets from the row base
    bool upper;                // h == 1: scales 4..7 use the split 4+2 bit packing
  };
  struct Act {
    int q[32];       // 128 activations, in element order
    int bs01, bs23;  // sums of the four 32-element sub-blocks as packed int16 pairs
    float yd;
  };
  __device__ __forceinline__ static void make_unit(int u, bool valid, Unit& un) {
    const int blk = valid ? (u >> 1) : 0, h = valid ? (u & 1) : 0;
    un.off_hdr = blk * Q4KL::kBytes;
    un.off_qs = blk * Q4KL::kBytes + Q4KL::kOffQs + 64 * h;
    un.upper = h != 0;
  }
  __device__ __forceinline__ static void load_act(int u, bool valid, const ActPlanes& a, int k, int m, Act& ac) {
    if (!valid) {
#pragma unroll
      for (int i = 0; i < 32; ++i) ac.q[i] = 0;
      ac.bs01 = ac.bs23 = 0;
      ac.yd = 0.f;
      return;
    }
    const int blk = u >> 1, h = u & 1;
    const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + blk * 256 + 128 * h);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int4 v = q8[i];
      ac.q[4 * i] = v.x, ac.q[4 * i + 1] = v.y, ac.q[4 * i + 2] = v.z, ac.q[4 * i + 3] = v.w;
    }
    const int4 bs = *reinterpret_cast<const int4*>(a.bsums + (size_t)m * (k >> 4) + blk * 16 + 8 * h);
    set_sums(bs.x, bs.y, bs.z, bs.w, ac);
    ac.yd = a.d[(size_t)m * (k >> 8) + blk];
  }
  // eight 16-element sums -> four 32-element sums (each |s| <= 4096, fits int16)
  __device__ __forceinline__ static void set_sums(int x, int y, int z, int w, Act& ac) {
    const int s0 = (int)(short)(x & 0xffff) + (x >> 16), s1 = (int)(short)(y & 0xffff) + (y >> 16);
    const int s2 = (int)(short)(z & 0xffff) + (z >> 16), s3 = (int)(short)(w & 0xffff) + (w >> 16);
    ac.bs01 = (s0 & 0xffff) | (s1 << 16);
    ac.bs23 = (s2 & 0xffff) | (s3 << 16);
  }
  static constexpr bool kHasRaw = true;  // Q8_K activations: a stamped form exists
  __device__ __forceinline__ static int probe(const Act& ac) { return ac.q[0] ^ ac.q[31] ^ ac.bs23 ^ __float_as_int(ac.yd); }
  // The shared-memory loads of a unit and the arithmetic on them are separate steps, so that a warp can have the
  // loads of two weight rows in flight before it starts on the first (kSplit).
  static constexpr bool kSplit = true;
  struct Raw {
    uint4 hdr;
    uint32_t w[16];
  };
  __device__ __forceinline__ static void load_raw(uint32_t rowbase, const Unit& un, Raw& raw) {
    raw.hdr = lds128(rowbase + un.off_hdr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = lds128(rowbase + un.off_qs + 16 * i);
      raw.w[4 * i] = v.x, raw.w[4 * i + 1] = v.y, raw.w[4 * i + 2] = v.z, raw.w[4 * i + 3] = v.w;
    }
  }
  template <int M>
  __device__ __forceinline__ static void compute(uint32_t rowbase, const Unit& un, const Act (&ac)[M], float (&acc)[M]) {
    Raw raw;
    load_raw(rowbase, un, raw);
    math<M>(raw, un, ac, acc);
  }
  template <int M>
  __device__ __forceinline__ static void math(const Raw& raw, const Unit& un, const Act (&ac)[M], float (&acc)[M]) {
    const uint4 hdr = raw.hdr;
    const uint32_t (&w)[16] = raw.w;
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    // four 6-bit scales and mins at once, one per byte (get_scale_min_k4, fuel-quantized/src/utils.rs:50-60)
    const uint32_t sc_lo4 = hdr.y & 0x3f3f3f3fu, mn_lo4 = hdr.z & 0x3f3f3f3fu;
    const uint32_t sc_hi4 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    const uint32_t mn_hi4 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    const uint32_t sc4 = un.upper ? sc_hi4 : sc_lo4, mn4 = un.upper ? mn_hi4 : mn_lo4;
    const int sc0 = sc4 & 0xff, sc1 = (sc4 >> 8) & 0xff, sc2 = (sc4 >> 16) & 0xff, sc3 = sc4 >> 24;
#pragma unroll
    for (int i = 0; i < M; ++i) {
      int d0a = 0, d0b = 0, d1a = 0, d1b = 0, d2a = 0, d2b = 0, d3a = 0, d3b = 0;  // independent chains
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        d0a = dp4a_ss((int)(w[j] & 0x0f0f0f0fu), ac[i].q[j], d0a);
        d0b = dp4a_ss((int)(w[j + 1] & 0x0f0f0f0fu), ac[i].q[j + 1], d0b);
        d1a = dp4a_us(w[j] & 0xf0f0f0f0u, ac[i].q[8 + j], d1a);  // 16 x the high-nibble dot product
        d1b = dp4a_us(w[j + 1] & 0xf0f0f0f0u, ac[i].q[9 + j], d1b);
        d2a = dp4a_ss((int)(w[8 + j] & 0x0f0f0f0fu), ac[i].q[16 + j], d2a);
        d2b = dp4a_ss((int)(w[9 + j] & 0x0f0f0f0fu), ac[i].q[17 + j], d2b);
        d3a = dp4a_us(w[8 + j] & 0xf0f0f0f0u, ac[i].q[24 + j], d3a);
        d3b = dp4a_us(w[9 + j] & 0xf0f0f0f0u, ac[i].q[25 + j], d3b);
      }
      // the two high-nibble dots are multiples of 16, and stay so after the integer scale
      const int si = sc0 * (d0a + d0b) + sc2 * (d2a + d2b) + ((sc1 * (d1a + d1b) + sc3 * (d3a + d3b)) >> 4);
      const int mi = __dp2a_hi(ac[i].bs23, (int)mn4, __dp2a_lo(ac[i].bs01, (int)mn4, 0));
      acc[i] += (d * ac[i].yd) * (float)si - (dmin * ac[i].yd) * (float)mi;
    }
  }
};

// ---- Q5_K: Q4_K's unit (half a super-block, four sub-blocks) with the fifth bits merged in from qh: sub-block 4h+i
// of half h takes bit 4h+i of every qh byte (fuel-quantized/src/k_quants.rs:1664-1680). The 5-bit values are built
// once per unit as unsigned bytes, so the high nibbles are shifted down here (a 5-bit value times 16 overflows a byte).
struct Q5KRegs : Q4KRegs {
  static constexpr bool kSplit = false;
  struct Unit {
    uint32_t off_hdr, off_qh, off_qs;
    bool upper;
  };
  __device__ __forceinline__ static void make_unit(int u, bool valid, Unit& un) {
    const int blk = valid ? (u >> 1) : 0, h = valid ? (u & 1) : 0;
    un.off_hdr = blk * Q5KL::kBytes;
    un.off_qh = blk * Q5KL::kBytes + Q5KL::kOffQh;
    un.off_qs = blk * Q5KL::kBytes + Q5KL::kOffQs + 64 * h;
    un.upper = h != 0;
  }
  template <int M>
  __device__ __forceinline__ static void compute(uint32_t rowbase, const Unit& un, const Act (&ac)[M], float (&acc)[M]) {
    const uint4 hdr = lds128(rowbase + un.off_hdr);
    uint32_t w[16], hq[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = lds128(rowbase + un.off_qs + 16 * i);
      w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = lds128(rowbase + un.off_qh + 16 * i);
      hq[4 * i] = v.x, hq[4 * i + 1] = v.y, hq[4 * i + 2] = v.z, hq[4 * i + 3] = v.w;
    }
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    const uint32_t sc_lo4 = hdr.y & 0x3f3f3f3fu, mn_lo4 = hdr.z & 0x3f3f3f3fu;
    const uint32_t sc_hi4 = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
    const uint32_t mn_hi4 = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    const uint32_t sc4 = un.upper ? sc_hi4 : sc_lo4, mn4 = un.upper ? mn_hi4 : mn_lo4;
    const int sc0 = sc4 & 0xff, sc1 = (sc4 >> 8) & 0xff, sc2 = (sc4 >> 16) & 0xff, sc3 = sc4 >> 24;
    const uint32_t sh = un.upper ? 4u : 0u;
    uint32_t v[32];  // 5-bit values in element order: sub-blocks 0..3 of the half, eight words each
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t hb = hq[j] >> sh;
      v[j] = (w[j] & 0x0f0f0f0fu) | ((hb & 0x01010101u) << 4);
      v[8 + j] = ((w[j] >> 4) & 0x0f0f0f0fu) | (((hb >> 1) & 0x01010101u) << 4);
      v[16 + j] = (w[8 + j] & 0x0f0f0f0fu) | (((hb >> 2) & 0x01010101u) << 4);
      v[24 + j] = ((w[8 + j] >> 4) & 0x0f0f0f0fu) | (((hb >> 3) & 0x01010101u) << 4);
    }
#pragma unroll
    for (int i = 0; i < M; ++i) {
      int dsum[4];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        int a = 0, b = 0;  // two independent chains per sub-block
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          a = dp4a_us(v[8 * s + j], ac[i].q[8 * s + j], a);
          b = dp4a_us(v[8 * s + j + 1], ac[i].q[8 * s + j + 1], b);
        }
        dsum[s] = a + b;
      }
      const int si = sc0 * dsum[0] + sc1 * dsum[1] + sc2 * dsum[2] + sc3 * dsum[3];
      const int mi = __dp2a_hi(ac[i].bs23, (int)mn4, __dp2a_lo(ac[i].bs01, (int)mn4, 0));
      acc[i] += (d * ac[i].yd) * (float)si - (dmin * ac[i].yd) * (float)mi;
    }
  }
};

// ---- helpers for formats whose blocks are only 2-byte aligned in the stage --------------------
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// NW consecutive 32-bit words starting at a 2-byte-aligned shared address: NW + 1 aligned loads
// and one funnel shift each (a no-op shift when the address happens to be 4-byte aligned)
template <int NW>
__device__ __forceinline__ void lds_words_2b(uint32_t addr, uint32_t (&w)[NW]) {
  const uint32_t base = addr & ~3u, sh = (addr & 2u) * 8u;
  uint32_t prev = lds32(base);
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    const uint32_t nxt = lds32(base + 4 * (i + 1));
    w[i] = __funnelshift_r(prev, nxt, sh);
    prev = nxt;
  }
}

// ---- Q6_K: unit = half a super-block (128 elements: 64 B ql, 32 B qh, 8 scales). The 6-bit values are
// used unsigned (0..63) in dp4a; the "-32" of every element is folded into one correction per half,
// 32 * sum_g scale_g * (sum of the 16 activations of group g), from the activation block sums.
struct Q6KRegs {
  static constexpr int kUnitsPerBlock = 2;
  static constexpr bool kSplit = false;
  struct Unit {
    uint32_t off_blk;  // byte offset of the super-block from the row base
    uint32_t half;
  };
  struct Act {
    int q[32];
    int bs[4];  // eight 16-element sums as packed int16 pairs
    float yd;
  };
  __device__ __forceinline__ static void make_unit(int u, bool valid, Unit& un) {
    un.off_blk = (valid ? (u >> 1) : 0) * Q6KL::kBytes;
    un.half = valid ? (u & 1) : 0;
  }
  __device__ __forceinline__ static void load_act(int u, bool valid, const ActPlanes& a, int k, int m, Act& ac) {
    if (!valid) {
#pragma unroll
      for (int i = 0; i < 32; ++i) ac.q[i] = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) ac.bs[i] = 0;
      ac.yd = 0.f;
      return;
    }
    const int blk = u >> 1, h = u & 1;
    const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + blk * 256 + 128 * h);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int4 v = q8[i];
      ac.q[4 * i] = v.x, ac.q[4 * i + 1] = v.y, ac.q[4 * i + 2] = v.z, ac.q[4 * i + 3] = v.w;
    }
    const int4 bs = *reinterpret_cast<const int4*>(a.bsums + (size_t)m * (k >> 4) + blk * 16 + 8 * h);
    ac.bs[0] = bs.x, ac.bs[1] = bs.y, ac.bs[2] = bs.z, ac.bs[3] = bs.w;
    ac.yd = a.d[(size_t)m * (k >> 8) + blk];
  }
  static constexpr bool kHasRaw = true;
  __device__ __forceinline__ static int probe(const Act& ac) { return ac.q[0] ^ ac.q[31] ^ ac.bs[3] ^ __float_as_int(ac.yd); }
  template <int M>
  __device__ __forceinline__ static void compute(uint32_t rowbase, const Unit& un, const Act (&ac)[M], float (&acc)[M]) {
    const uint32_t b = rowbase + un.off_blk;
    uint32_t ql[16], qh[8], sc[2];
    lds_words_2b<16>(b + Q6KL::kOffQl + 64 * un.half, ql);
    lds_words_2b<8>(b + Q6KL::kOffQh + 32 * un.half, qh);
    lds_words_2b<2>(b + Q6KL::kOffScales + 8 * un.half, sc);
    uint16_t dh;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(dh) : "r"(b + Q6KL::kOffD));
    const float d = h2f_bits(dh);
    // unsigned 6-bit values, four per word; word j covers l = 4j..4j+3
    uint32_t qv[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t h = qh[j];
      qv[j] = (ql[j] & 0x0f0f0f0fu) | ((h << 4) & 0x30303030u);             // elements l
      qv[8 + j] = (ql[8 + j] & 0x0f0f0f0fu) | ((h << 2) & 0x30303030u);     // l + 32
      qv[16 + j] = ((ql[j] >> 4) & 0x0f0f0f0fu) | (h & 0x30303030u);        // l + 64
      qv[24 + j] = ((ql[8 + j] >> 4) & 0x0f0f0f0fu) | ((h >> 2) & 0x30303030u);  // l + 96
    }
    int s8[8];  // signed scales of the eight 16-element groups
#pragma unroll
    for (int g = 0; g < 8; ++g) s8[g] = (int)(int8_t)((sc[g >> 2] >> (8 * (g & 3))) & 0xff);
#pragma unroll
    for (int i = 0; i < M; ++i) {
      int si = 0;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        int dg = dp4a_us(qv[4 * g], ac[i].q[4 * g], 0);
        dg = dp4a_us(qv[4 * g + 1], ac[i].q[4 * g + 1], dg);
        dg = dp4a_us(qv[4 * g + 2], ac[i].q[4 * g + 2], dg);
        dg = dp4a_us(qv[4 * g + 3], ac[i].q[4 * g + 3], dg);
        si += s8[g] * dg;
      }
      // correction: sum_g scale_g * bsum_g, two groups per dp2a
      int corr = __dp2a_lo(ac[i].bs[0], (int)sc[0], 0);
      corr = __dp2a_hi(ac[i].bs[1], (int)sc[0], corr);
      corr = __dp2a_lo(ac[i].bs[2], (int)sc[1], corr);
      corr = __dp2a_hi(ac[i].bs[3], (int)sc[1], corr);
      acc[i] += (d * ac[i].yd) * (float)(si - 32 * corr);
    }
  }
};

// ---- Q8_0: unit = four 34-byte blocks (128 elements)
struct Q8_0Regs {
  static constexpr bool kSplit = false;
  static constexpr int kUnitsPerBlock = 0;  // units are counted per 128 elements, see the launcher
  struct Unit {
    uint32_t off;  // byte offset of the first of the four blocks
  };
  struct Act {
    int q[32];
    float yd[4];
  };
  __device__ __forceinline__ static void make_unit(int u, bool valid, Unit& un) { un.off = (valid ? u : 0) * 4 * Q8_0L::kBytes; }
  __device__ __forceinline__ static void load_act(int u, bool valid, const ActPlanes& a, int k, int m, Act& ac) {
    if (!valid) {
#pragma unroll
      for (int i = 0; i < 32; ++i) ac.q[i] = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) ac.yd[i] = 0.f;
      return;
    }
    const int4* q8 = reinterpret_cast<const int4*>(a.qs + (size_t)m * k + u * 128);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int4 v = q8[i];
      ac.q[4 * i] = v.x, ac.q[4 * i + 1] = v.y, ac.q[4 * i + 2] = v.z, ac.q[4 * i + 3] = v.w;
    }
    const float4 dv = *reinterpret_cast<const float4*>(a.d + (size_t)m * (k >> 5) + u * 4);
    ac.yd[0] = dv.x, ac.yd[1] = dv.y, ac.yd[2] = dv.z, ac.yd[3] = dv.w;
  }
  static constexpr bool kHasRaw = false;  // its activations are Q8_0 blocks; no stamped form
  __device__ __forceinline__ static int probe(const Act& ac) { return ac.q[0] ^ ac.q[31] ^ __float_as_int(ac.yd[3]); }
  template <int M>
  __device__ __forceinline__ static void compute(uint32_t rowbase, const Unit& un, const Act (&ac)[M], float (&acc)[M]) {
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      const uint32_t b = rowbase + un.off + blk * Q8_0L::kBytes;
      uint16_t dh;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(dh) : "r"(b));
      const float d = h2f_bits(dh);
      uint32_t w[8];
      lds_words_2b<8>(b + Q8_0L::kOffQs, w);
#pragma unroll
      for (int i = 0; i < M; ++i) {
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          s0 = dp4a_ss((int)w[j], ac[i].q[8 * blk + j], s0);
          s1 = dp4a_ss((int)w[j + 1], ac[i].q[8 * blk + j + 1], s1);
        }
        acc[i] += (d * ac[i].yd[blk]) * (float)(s0 + s1);
      }
    }
  }
};

struct DecodeRegsSmemHeader {
  uint64_t full[kDecodeMaxStages];
  uint64_t empty[kDecodeMaxStages];
  uint64_t part_ready[2];
  uint64_t acts_ready;
  uint64_t rows_stored, host_go;  // write-back to a host buffer: consumer warps done / thread 0 has counted this CTA
  int host_last;
  float partial[2][32][8][2];  // [buffer][row in stage][k-slice][m]
};

// kTree: the dot product of a row is summed as a balanced binary tree over (up to) eight fixed ranges of k ("leaves"),
// each leaf summed in an order that depends on nothing but the leaf: leaf l occupies leaf_lw consecutive lanes, the
// lanes of a leaf are added pairwise from the lowest lane bit up, then leaves pairwise, in registers and (for rows
// spread over several warps) in shared memory. A matrix cut along k into 2, 4 or 8 aligned groups of leaves (one per
// GPU) therefore gives partial results whose pairwise sum, in the same tree, is BIT-IDENTICAL to the one-GPU result:
// each GPU computes a complete subtree. This is what lets the row-parallel layers of a tensor-parallel model produce
// the same tokens at every GPU count.
template <class Fmt, int M, int NU, bool kPeer, bool kTree = false>
__device__ __forceinline__ void decode_regs_body(const DecodeRegsParams& p, const DecodeRegsPeer* g) {
  static_assert(!kPeer || M == 1, "the tensor-parallel form is a single-row mat-vec");
  static_assert(!kTree || (M == 1 && NU == 1), "the tree form is a single-row mat-vec with one unit per lane");
  extern __shared__ __align__(128) uint8_t smem_raw[];
  DecodeRegsSmemHeader* hd = reinterpret_cast<DecodeRegsSmemHeader*>(smem_raw);
  uint8_t* stages = smem_raw + align_up(sizeof(DecodeRegsSmemHeader), 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.num_stages, R = p.rows_per_stage;
  // this CTA's contiguous rows; all index arithmetic is 32-bit with host-computed quotients, since a
  // CTA lives for only a few dozen rows and 64-bit divisions would dominate its prologue
  const int cta = blockIdx.x;
  const int r_begin = cta * p.rows_q + (cta < p.rows_rem ? cta : p.rows_rem);
  const int r_count = p.rows_q + (cta < p.rows_rem ? 1 : 0);
  const int n_iter = (int)(((unsigned)r_count + (unsigned)R - 1u) / (unsigned)R);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hd->full[s], 1);
      mbar_init(&hd->empty[s], kDecodeConsumerWarps);
    }
    mbar_init(&hd->part_ready[0], kDecodeConsumerWarps);
    mbar_init(&hd->part_ready[1], kDecodeConsumerWarps);
    mbar_init(&hd->acts_ready, kDecodeConsumerWarps);
    mbar_init(&hd->rows_stored, kDecodeConsumerWarps);
    mbar_init(&hd->host_go, 1);
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kDecodeConsumerWarps) {
    // ---------------- producer (weights do not depend on the previous kernel: no pdl_wait before loading)
    if (lane == 0) {
      const int64_t tma_limit = p.total_bytes & ~(int64_t)15;
      int issued = 0;
      bool ok = true;
      int s = 0, js = 0;          // ring slot of stage `it`, and of stage `it - depth`
      uint32_t ph = 0, jph = 0;   // their phase parities
      for (int it = 0; it < n_iter; ++it) {
        if (it >= S && !mbar_poll_bounded(&hd->empty[s], ph ^ 1u)) {
          record_dev_error(kErrEmptyWait);
          ok = false;
          break;
        }
        // Activation loads queue behind whatever bulk traffic this SM has outstanding; hold the
        // rest of the stream back until the consumers have theirs.
        if (p.pre_stages && it == p.pre_stages && !mbar_poll_bounded(&hd->acts_ready, 0)) {
          record_dev_error(kErrFullWait);
          ok = false;
          break;
        }
        // Keep at most `depth` copies of this CTA in flight, so stages complete in order and the
        // consumers can start on the first while the rest stream in.
        if (it >= p.depth) {
          if (!mbar_poll_bounded(&hd->full[js], jph)) {
            record_dev_error(kErrFullWait);
            ok = false;
            break;
          }
          if (++js == S) js = 0, jph ^= 1u;
        }
        const int row0 = r_begin + it * R;
        const int rows_here = (r_count - it * R < R) ? r_count - it * R : R;
        const int64_t b0 = (int64_t)row0 * p.row_bytes, b1 = b0 + (int64_t)rows_here * p.row_bytes;
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
        if (++s == S) s = 0, ph ^= 1u;
      }
      if (!ok) {  // consumers stopped releasing stages: let our own copies land before leaving
        for (int it = (issued > S ? issued - S : 0); it < issued; ++it)
          if (!mbar_poll_bounded(&hd->full[it % S], (it / S) & 1)) record_dev_error(kErrDrainWait);
      }
    }
    pdl_wait();
    return;
  }

  // ---------------- consumers
  const int ks = p.ks;
  const int slice = warp & (ks - 1), rgroup = warp / ks, n_rgroups = kDecodeConsumerWarps / ks;  // ks is a power of two
  const int u_begin = p.u_begin[slice], u_end = p.u_begin[slice + 1];

  typename Fmt::Unit un[NU];
  typename Fmt::Act ac[NU][M];
  uint32_t push_stamp = 0;
  pdl_wait();  // activation planes are written by the preceding kernel
  ActPlanes planes = p.act;
  if (Fmt::kHasRaw && p.x_f32) {
    // fused activation quantization: the consumer warps take the 256-element blocks of the M rows in turn
    // (the same routine as the stand-alone kernel, so the same bytes), while the producer streams weights
    planes = act_planes(smem_raw + p.act_smem_off, kQ4K, M, p.k);
    const int nblk = M * (p.k >> 8);
    for (int b = warp; b < nblk; b += 2 * kDecodeConsumerWarps) {  // two blocks per round: both loads in flight at once
      const int b2 = b + kDecodeConsumerWarps;
      const bool two = b2 < nblk;
      const float4* s0 = reinterpret_cast<const float4*>(p.x_f32 + (size_t)b * 256);
      const float4* s1 = reinterpret_cast<const float4*>(p.x_f32 + (size_t)(two ? b2 : b) * 256);
      const float4 a0 = s0[lane], a1 = s0[32 + lane], c0 = s1[lane], c1 = s1[32 + lane];
      const float e0[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float e1[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      q8k_block_from_regs(e0, lane, b, (int8_t*)planes.qs, (float*)planes.d, (int16_t*)planes.bsums);
      if (two) q8k_block_from_regs(e1, lane, b2, (int8_t*)planes.qs, (float*)planes.d, (int16_t*)planes.bsums);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecodeConsumerWarps) : "memory");
  }
  if constexpr (kPeer) {
    push_stamp = peer_stamp(g->ctx, g->ctx.push_seq);
  }
#pragma unroll
  for (int j = 0; j < NU; ++j) {
    int u = u_begin + lane + 32 * j;
    bool valid = u < u_end;
    if constexpr (kTree) {
      const int slot = slice * 32 + lane, leaf = slot / p.leaf_lw, pos = slot - leaf * p.leaf_lw;
      valid = leaf < p.n_leaves && pos < p.leaf_u0[leaf < 8 ? leaf + 1 : 8] - p.leaf_u0[leaf < 8 ? leaf : 8];
      u = valid ? p.leaf_u0[leaf] + pos : 0;
    }
    Fmt::make_unit(u, valid, un[j]);
#pragma unroll
    for (int i = 0; i < M; ++i) Fmt::load_act(u, valid, planes, p.k, i, ac[j][i]);
  }

  {
    // wait for the loads to land (a use of the last-loaded registers), then tell the producer
    int probe = 0;
#pragma unroll
    for (int j = 0; j < NU; ++j)
#pragma unroll
      for (int i = 0; i < M; ++i) probe ^= Fmt::probe(ac[j][i]);
    asm volatile("" ::"r"(probe));
    __syncwarp();
    if (lane == 0) mbar_arrive(&hd->acts_ready);
  }
  const uint32_t stages_u32 = smem_u32(stages);
  int s = 0;
  uint32_t ph = 0;
  for (int it = 0; it < n_iter; ++it) {
    if (!mbar_wait_bounded(&hd->full[s], ph)) {
      record_dev_error(kErrFullWait);
      return;
    }
    const int row0 = r_begin + it * R;
    const int rows_here = (r_count - it * R < R) ? r_count - it * R : R;
    const uint32_t skew = (uint32_t)(((int64_t)row0 * p.row_bytes) & 15);
    const uint32_t sbase = stages_u32 + (uint32_t)s * p.stage_stride + skew;
    const int buf = it & 1;
    // lane 0 hands a finished row on: to y, to every rank's buffer, or to the k-slice partials
    auto emit = [&](int r, const float (&acc)[M]) {
#pragma unroll
      for (int i = 0; i < M; ++i) {
        if (ks == 1) {
          if constexpr (kPeer) {
            for (int q = 0; q < g->ctx.world; ++q) st_pair(g->dst[q] + row0 + r, __float_as_uint(acc[i]), push_stamp);
          } else {
            p.y[(size_t)i * p.n + row0 + r] = acc[i];
          }
        } else
          hd->partial[buf][r][slice][i] = acc[i];
      }
    };
    int r = rgroup;
    if constexpr (Fmt::kSplit && NU == 1 && M == 1) {
      // two rows at a time: both rows' shared-memory loads are issued before the arithmetic of the first, and the two
      // shuffle reductions interleave (each row's own arithmetic and order are unchanged)
      for (; r + n_rgroups < rows_here; r += 2 * n_rgroups) {
        typename Fmt::Raw ra, rb;
        Fmt::load_raw(sbase + (uint32_t)r * p.row_bytes, un[0], ra);
        Fmt::load_raw(sbase + (uint32_t)(r + n_rgroups) * p.row_bytes, un[0], rb);
        float acc0[M] = {0.f}, acc1[M] = {0.f};
        Fmt::template math<M>(ra, un[0], ac[0], acc0);
        Fmt::template math<M>(rb, un[0], ac[0], acc1);
#pragma unroll
        for (int lv = 0; lv < 5; ++lv) {
          const int off = kTree ? (1 << lv) : (16 >> lv);  // tree form: lowest lane bit first
          acc0[0] += __shfl_xor_sync(0xffffffffu, acc0[0], off);
          acc1[0] += __shfl_xor_sync(0xffffffffu, acc1[0], off);
        }
        if (lane == 0) {
          emit(r, acc0);
          emit(r + n_rgroups, acc1);
        }
      }
    }
    for (; r < rows_here; r += n_rgroups) {
      const uint32_t rowbase = sbase + (uint32_t)r * p.row_bytes;
      float acc[M];
#pragma unroll
      for (int i = 0; i < M; ++i) acc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < NU; ++j) Fmt::template compute<M>(rowbase, un[j], ac[j], acc);
#pragma unroll
      for (int i = 0; i < M; ++i) {
#pragma unroll
        for (int lv = 0; lv < 5; ++lv) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], kTree ? (1 << lv) : (16 >> lv));
      }
      if (lane == 0) emit(r, acc);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&hd->empty[s]);
    if (ks > 1) {
      // all consumer warps meet here (bounded), then the k-slices of each row are summed in fixed order
      if (lane == 0) mbar_arrive(&hd->part_ready[buf]);
      __syncwarp();  // reconverge first: lanes spinning below must not starve lane 0's arrive
      if (!mbar_wait_bounded(&hd->part_ready[buf], (it >> 1) & 1)) {
        record_dev_error(kErrFullWait);
        return;
      }
      for (int t = threadIdx.x; t < rows_here * M; t += 32 * kDecodeConsumerWarps) {
        const int r = t / M, i = t - r * M;
        float sum;
        if constexpr (kTree) {  // pairwise, continuing the tree of the lanes
          float v[8];
#pragma unroll
          for (int sg = 0; sg < 8; ++sg) v[sg] = sg < ks ? hd->partial[buf][r][sg][i] : 0.f;
#pragma unroll
          for (int w = 1; w < 8; w <<= 1)
#pragma unroll
            for (int sg = 0; sg < 8; sg += 2 * w)
              if (sg + w < ks) v[sg] += v[sg + w];
          sum = v[0];
        } else {
          sum = hd->partial[buf][r][0][i];
          for (int sg = 1; sg < ks; ++sg) sum += hd->partial[buf][r][sg][i];
        }
        if constexpr (kPeer) {
          for (int q = 0; q < g->ctx.world; ++q) st_pair(g->dst[q] + row0 + r, __float_as_uint(sum), push_stamp);
        } else {
          p.y[(size_t)i * p.n + row0 + r] = sum;
        }
      }
    }
    if (++s == S) s = 0, ph ^= 1u;
  }
  if constexpr (!kPeer && !kTree && M == 1) {
    if (p.host_y) {
      // Result wanted in host memory: every CTA counts itself once its rows are stored (fence, then a device-wide
      // counter); the CTA that counts last sees all of y and copies it out, 16 bytes per thread. Waits are bounded.
      __threadfence();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->rows_stored);
      if (warp == 0) {
        const bool met = mbar_wait_bounded(&hd->rows_stored, 0);
        if (lane == 0) {
          hd->host_last = met && atomicAdd(p.host_done, 1u) == gridDim.x - 1u;
          if (!met) record_dev_error(kErrFullWait);
          __threadfence();
          mbar_arrive(&hd->host_go);
        }
      }
      __syncwarp();
      if (!mbar_wait_bounded(&hd->host_go, 0)) {
        record_dev_error(kErrFullWait);
        return;
      }
      if (hd->host_last) {
        __threadfence();
        const int t = threadIdx.x, nt = 32 * kDecodeConsumerWarps;
        const int n = (int)p.n, n4 = (((reinterpret_cast<uintptr_t>(p.host_y) | reinterpret_cast<uintptr_t>(p.y)) & 15) == 0) ? (n >> 2) : 0;
        for (int i = t; i < n4; i += nt)
          reinterpret_cast<float4*>(p.host_y)[i] = __ldcg(reinterpret_cast<const float4*>(p.y) + i);
        for (int i = (n4 << 2) + t; i < n; i += nt) p.host_y[i] = __ldcg(p.y + i);
      }
    }
  }
}

template <class Fmt, int M, int NU>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_regs_kernel(const DecodeRegsParams p) {
  decode_regs_body<Fmt, M, NU, false>(p, nullptr);
}

// Tensor-parallel form: same arithmetic and order, output scattered to every rank.
template <class Fmt, int NU>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_regs_peer_kernel(const DecodeRegsParams p,
                                                                             const DecodeRegsPeer g) {
  decode_regs_body<Fmt, 1, NU, true>(p, &g);
}

// Tree-ordered forms (see kTree above): plain output, and output scattered to every rank.
template <class Fmt>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_regs_tree_kernel(const DecodeRegsParams p) {
  decode_regs_body<Fmt, 1, 1, false, true>(p, nullptr);
}
template <class Fmt>
__global__ void __launch_bounds__(kDecodeThreads, 2) decode_regs_tree_peer_kernel(const DecodeRegsParams p,
                                                                                  const DecodeRegsPeer g) {
  decode_regs_body<Fmt, 1, 1, true, true>(p, &g);
}

}  // namespace fq
