// Small-batch quantized matmul on the integer tensor cores: a handful of activation rows (a dense batch of
// 2..16 rows, or the rows routed to one expert) against Q4_K, Q5_K, Q6_K or Q8_0 weights, the weights streamed
// from HBM exactly once per 16 activation rows.
//
// Arithmetic: the reference's vec_dot per (weight row, activation row) — exact integer dot products of the
// packed weights with the 8-bit activation blocks per sub-block, combined per block in f32
// (fuel-quantized/src/k_quants.rs:1388-1468 Q4_K, 1946-2003 Q6_K, 674-692 Q8_0). Only the f32 summation order
// over blocks differs from the CPU path.
//
// Mapping onto mma.sync (s32 accumulate): the WEIGHTS are the 16-row A operand and the activations the 8-column
// B operand, so one instruction covers 16 weight rows x 8 activation rows x one sub-block:
//   Q4_K  m16n8k32, A = unsigned nibbles (low nibbles masked; high nibbles left in place, i.e. x16, and the
//         scaled sum shifted down once per block), one instruction per 32-element sub-block, then
//         S += scale * c per accumulator; mins through the activations' 32-element sums (dp2a);
//   Q6_K  m16n8k16, A = unsigned 6-bit values, one instruction per 16-element group (its scale unit), the
//         "-32" of every element folded into one correction per block, sum_g scale_g * bsum_g, itself two
//         k16 instructions on the scale bytes and the block sums split into 6 low bits and the rest;
//   Q8_0  m16n8k32 (s8 x s8), one instruction per 32-element block, scaled in f32.
// A fragments come from the staged weight rows by ldmatrix (Q4_K) or 32-bit loads (Q6_K / Q8_0 blocks are only
// 2-byte aligned), B fragments from the staged activation rows by ldmatrix.
//
// Thread block = 1 producer warp + 16 consumer warps, one block per SM. The producer streams 16-row tiles (one
// bulk copy per weight row into padded shared-memory rows, so that the eight rows a fragment load touches fall
// in different banks) through a ring of stages, one tile per stage. The consumer warps form 1, 2 or 4 groups;
// group g takes tiles g, g + groups, ... so several tiles are in work at once, and the warps of a group take
// consecutive ranges of the 256-element blocks along k; their partial sums meet in shared memory and are added
// in a fixed order, so results never depend on timing. When the activation rows of one pass (16 rows x k bytes)
// do not fit beside the ring, k is swept in chunks and each sweep adds into y in order. Every wait is bounded:
// a warp whose wait expires raises a flag in shared memory and keeps arriving at the block's barriers; the flag
// is read through the barrier itself (an OR reduction), so a group's warps always agree on it and leave together.
#pragma once
#include "decode_regs.cuh"
#include "fq_common.cuh"

namespace fq {

constexpr int kMbConsumerWarps = 16;
constexpr int kMbThreads = 32 * (kMbConsumerWarps + 1);
constexpr int kMbMaxStages = 8;

struct MmaBatchParams {
  const uint8_t* w;      // [n_groups][n][k] blocks
  ActPlanes act;         // plain activation planes of all rows
  const int* offsets;    // [n_groups + 1] row ranges, or null: one group holding rows [0, fixed_rows)
  const int* out_rows;   // row -> output row, or null for the identity
  float* y;              // [rows][n]
  int64_t group_bytes;   // n * row_bytes
  int64_t total_bytes;   // n_groups * group_bytes
  int fixed_rows;
  int n, k, row_bytes;
  int n_wgroups;         // consumer warp groups (1, 2 or 4): group g takes stages g, g + n_wgroups, ... and its warps split k
  int num_stages, stage_stride;
  int wstride;           // bytes between staged copies (rows_per_copy rows' bytes + skew room + bank padding)
  int rows_per_copy;     // 1, 2 or 4 consecutive rows per bulk copy (more than 1 only when whole rows are staged)
  int act_off, part_off; // shared-memory offsets of the activation area and of the partial-sum area
  int kc_blocks;         // 256-element blocks of k per sweep
};


struct MmaBatchHeader {
  uint64_t full[kMbMaxStages];
  uint64_t empty[kMbMaxStages];
  uint64_t acts;      // the first sweep's activation rows have landed (bulk copies issued by the producer)
  volatile int dead;  // a bounded wait expired somewhere in this block
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
// c = A(16x32 u8, weights) * B(32x8 s8, activations); fresh accumulators
// (the MMA wrappers are pure functions of their operands: not volatile, so the compiler may schedule them among the
// surrounding arithmetic; the shared-memory loads stay volatile and keep their order against the barriers)
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8s8_k32(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// accumulating form, s8 x s8
__device__ __forceinline__ void mma_s8s8_k16_acc(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t lds_u32_2b_addr(uint32_t a) {
  const uint32_t base = a & ~3u;
  uint32_t lo, hi;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lo) : "r"(base));
  asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(hi) : "r"(base));
  return __funnelshift_r(lo, hi, (a & 2u) * 8u);
}
__device__ __forceinline__ uint32_t lds_u16_addr(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}

// Shared-memory layout of one pass's activation rows (one k-chunk of KC blocks), per format:
//   qs    [rows][KC*256 + 16]                 int8, padded rows (ldmatrix: eight rows, eight different bank groups)
//   aux   Q4_K: [rows][KC*8 + 8] int16 32-element sums;  Q6_K: two byte planes [rows][KC*16 + 16], the 16-element
//         sums split as 64 * hi + lo (lo 0..63);  Q8_0: none
//   d     f32 [KC * scales-per-256][16]       activation-row index fastest
struct MbActLayout {
  int astride, aux_stride, aux_plane;  // bytes
  int off_aux, off_d, bytes;
};
template <class F>
__host__ __device__ inline MbActLayout mb_act_layout(int kc_blocks, int rows) {
  MbActLayout L;
  L.astride = kc_blocks * 256 + 16;
  size_t off = align_up((size_t)rows * L.astride, 128);
  L.off_aux = (int)off;
  L.aux_stride = F::kAuxBytesPer256 ? kc_blocks * F::kAuxBytesPer256 + 16 : 0;
  L.aux_plane = (int)align_up((size_t)rows * L.aux_stride, 128);
  off += (size_t)L.aux_plane * F::kAuxPlanes;
  L.off_d = (int)off;
  off += align_up((size_t)kc_blocks * F::kScalesPer256 * 16 * 4, 128);
  L.bytes = (int)off;
  return L;
}

struct MbCtx {
  uint32_t tile_s;   // shared address of the tile's first weight row (chunk start)
  uint32_t act_s;    // shared address of the activation area
  int wstride;       // bytes between staged copies
  int rpc_shift;     // log2(rows per copy)
  int row_bytes;     // bytes between the rows of one copy
  int lane, gid, tig;
  MbActLayout L;
  // byte offset of tile row i from tile_s (before the copy's skew)
  __device__ __forceinline__ uint32_t row_off(int i) const {
    return (uint32_t)(i >> rpc_shift) * (uint32_t)wstride + (uint32_t)(i & ((1 << rpc_shift) - 1)) * (uint32_t)row_bytes;
  }
};

// ------------------------------------------------------------------------------------------------ Q4_K
struct MbQ4K {
  static constexpr int kType = kQ4K;
  static constexpr int kBytes256 = 144;
  static constexpr int kAuxBytesPer256 = 16, kAuxPlanes = 1, kScalesPer256 = 1;
  static constexpr bool kRowsAligned = true;  // every row and chunk starts on a 16-byte boundary
  // cooperative staging of the aux planes and scales for rows [a0, a0 + ac) (zeros past ac), blocks [cb0, cb0 + cbn)
  __device__ static void stage_aux(const ActPlanes& act, int k, int a0, int ac, int rows, int cb0, int cbn, uint8_t* area,
                                   const MbActLayout& L, int t, int nt) {
    const int nblk = k >> 8;
    const int s32 = cbn * 8;
    for (int i = t; i < rows * s32; i += nt) {
      const int r = i / s32, c = i - r * s32;
      int v = 0;
      if (r < ac) {
        const int16_t* bs = act.bsums + (size_t)(a0 + r) * (k >> 4) + cb0 * 16 + 2 * c;
        v = (int)bs[0] + (int)bs[1];
      }
      *reinterpret_cast<int16_t*>(area + L.off_aux + (size_t)r * L.aux_stride + 2 * c) = (int16_t)v;
    }
    float* d = reinterpret_cast<float*>(area + L.off_d);
    for (int i = t; i < rows * cbn; i += nt) {
      const int r = i / cbn, c = i - r * cbn;
      d[c * 16 + r] = r < ac ? act.d[(size_t)(a0 + r) * nblk + cb0 + c] : 0.f;
    }
  }
  template <int MT>
  __device__ __forceinline__ static void block_step(const MbCtx& cx, int b, uint32_t, uint32_t, float (&facc)[MT][4]) {
    const uint32_t blk = (uint32_t)b * 144u;
    const uint4 h0 = lds128(cx.tile_s + cx.row_off(cx.gid) + blk);
    const uint4 h1 = lds128(cx.tile_s + cx.row_off(cx.gid + 8) + blk);
    // eight 6-bit scales / mins per row as bytes of two words (get_scale_min_k4, fuel-quantized/src/utils.rs:50-60)
    const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | (((h0.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | (((h0.z >> 6) & 0x03030303u) << 4)};
    const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | (((h1.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | (((h1.z >> 6) & 0x03030303u) << 4)};
    // ldmatrix addresses: weights, rows (lane & 7) + 8 * bit 3, byte column 16 * bit 4 of the 32 bytes of a nibble group;
    // activations, rows (lane & 7), the four 16-byte pieces of the group's 64 elements
    const uint32_t wq = cx.tile_s + cx.row_off((cx.lane & 7) + 8 * ((cx.lane >> 3) & 1)) + blk + 16u + 16u * (cx.lane >> 4);
    const uint32_t aq = cx.act_s + (uint32_t)(cx.lane & 7) * cx.L.astride + (uint32_t)b * 256u + 16u * (cx.lane >> 3);
    int Slo[MT][4], Shi[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) Slo[mt][i] = 0, Shi[mt][i] = 0;
    // Four groups of 64 elements (low nibbles = sub-block 2g, high nibbles = 2g + 1). The fragment loads of group g + 1 are
    // issued before the arithmetic of group g, and a group's MMAs all issue before the first use of their results, so a
    // warp pays the load and tensor-pipe latencies once per group instead of once per instruction.
    uint32_t r[2][4], q[2][MT][4];
    ldmatrix_x4(r[0], wq);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(q[0][mt], aq + (uint32_t)(8 * mt) * cx.L.astride);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int cur = g & 1, nxt = cur ^ 1;
      if (g < 3) {
        ldmatrix_x4(r[nxt], wq + 32u * (g + 1));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(q[nxt][mt], aq + (uint32_t)(8 * mt) * cx.L.astride + 64u * (g + 1));
      }
      uint32_t alo[4], ahi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) alo[i] = r[cur][i] & 0x0f0f0f0fu, ahi[i] = r[cur][i] & 0xf0f0f0f0u;
      int cl[MT][4], ch[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_u8s8_k32(cl[mt], alo, q[cur][mt][0], q[cur][mt][1]);
        mma_u8s8_k32(ch[mt], ahi, q[cur][mt][2], q[cur][mt][3]);  // 16 x the high-nibble dots
      }
      const int sh = 16 * (g & 1);
      const int s0l = (int)((sc0[g >> 1] >> sh) & 0xff), s0h = (int)((sc0[g >> 1] >> (sh + 8)) & 0xff);
      const int s1l = (int)((sc1[g >> 1] >> sh) & 0xff), s1h = (int)((sc1[g >> 1] >> (sh + 8)) & 0xff);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        Slo[mt][0] += cl[mt][0] * s0l, Slo[mt][1] += cl[mt][1] * s0l, Slo[mt][2] += cl[mt][2] * s1l, Slo[mt][3] += cl[mt][3] * s1l;
        Shi[mt][0] += ch[mt][0] * s0h, Shi[mt][1] += ch[mt][1] * s0h, Shi[mt][2] += ch[mt][2] * s1h, Shi[mt][3] += ch[mt][3] * s1h;
      }
    }
    const float d0 = h2f_bits(h0.x & 0xffffu), dm0 = h2f_bits(h0.x >> 16);
    const float d1 = h2f_bits(h1.x & 0xffffu), dm1 = h2f_bits(h1.x >> 16);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m0 = 8 * mt + 2 * cx.tig;
      // sum_j min_j * bsum_j: two sub-blocks per dp2a (16-bit sums x 8-bit mins)
      const uint4 ba = lds128(cx.act_s + cx.L.off_aux + (uint32_t)m0 * cx.L.aux_stride + (uint32_t)b * 16u);
      const uint4 bb = lds128(cx.act_s + cx.L.off_aux + (uint32_t)(m0 + 1) * cx.L.aux_stride + (uint32_t)b * 16u);
      auto mins = [](const uint4& bs, const uint32_t (&mn)[2]) {
        return __dp2a_hi((int)bs.w, (int)mn[1], __dp2a_lo((int)bs.z, (int)mn[1], __dp2a_hi((int)bs.y, (int)mn[0], __dp2a_lo((int)bs.x, (int)mn[0], 0))));
      };
      const int T0 = mins(ba, mn0), T1 = mins(bb, mn0), T2 = mins(ba, mn1), T3 = mins(bb, mn1);
      const uint2 ydw = lds64(cx.act_s + cx.L.off_d + (uint32_t)(b * 16 + m0) * 4u);
      const float ya = __uint_as_float(ydw.x), yb = __uint_as_float(ydw.y);
      // the high-nibble sums are multiples of 16 and stay so after the integer scale
      facc[mt][0] += (d0 * ya) * (float)(Slo[mt][0] + (Shi[mt][0] >> 4)) - (dm0 * ya) * (float)T0;
      facc[mt][1] += (d0 * yb) * (float)(Slo[mt][1] + (Shi[mt][1] >> 4)) - (dm0 * yb) * (float)T1;
      facc[mt][2] += (d1 * ya) * (float)(Slo[mt][2] + (Shi[mt][2] >> 4)) - (dm1 * ya) * (float)T2;
      facc[mt][3] += (d1 * yb) * (float)(Slo[mt][3] + (Shi[mt][3] >> 4)) - (dm1 * yb) * (float)T3;
    }
  }
};

// ------------------------------------------------------------------------------------------------ Q5_K
// Q4_K's block with a fifth bit per element (fuel-quantized/src/k_quants.rs:1626-1760): the same 16-byte header (d, dmin,
// packed 6-bit scales and mins), then 32 bytes of qh, then the 128 bytes of nibbles. Byte t of qh carries, in bits 2g and
// 2g + 1, the fifth bits of the low- and high-nibble elements of byte t of nibble group g - so one ldmatrix of the qh
// bytes per block lands in exactly the fragment positions of every group's nibble bytes. The 5-bit values are built as
// unsigned bytes (a value times 16 no longer fits one), one MMA per 32-element sub-block as for Q4_K.
struct MbQ5K : MbQ4K {
  static constexpr int kType = kQ5K;
  static constexpr int kBytes256 = 176;
  template <int MT>
  __device__ __forceinline__ static void block_step(const MbCtx& cx, int b, uint32_t, uint32_t, float (&facc)[MT][4]) {
    const uint32_t blk = (uint32_t)b * 176u;
    const uint4 h0 = lds128(cx.tile_s + cx.row_off(cx.gid) + blk);
    const uint4 h1 = lds128(cx.tile_s + cx.row_off(cx.gid + 8) + blk);
    const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | (((h0.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | (((h0.z >> 6) & 0x03030303u) << 4)};
    const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | (((h1.y >> 6) & 0x03030303u) << 4)};
    const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | (((h1.z >> 6) & 0x03030303u) << 4)};
    // ldmatrix addresses as for Q4_K: rows (lane & 7) + 8 * bit 3, byte column 16 * bit 4 of a 32-byte run - the qh bytes
    // at offset 16 of the block, the nibble groups from offset 48
    const uint32_t wrow = cx.tile_s + cx.row_off((cx.lane & 7) + 8 * ((cx.lane >> 3) & 1)) + blk + 16u * (cx.lane >> 4);
    const uint32_t wq = wrow + 48u;
    const uint32_t aq = cx.act_s + (uint32_t)(cx.lane & 7) * cx.L.astride + (uint32_t)b * 256u + 16u * (cx.lane >> 3);
    int Slo[MT][4], Shi[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) Slo[mt][i] = 0, Shi[mt][i] = 0;
    uint32_t hq[4], r[2][4], q[2][MT][4];
    ldmatrix_x4(hq, wrow + 16u);
    ldmatrix_x4(r[0], wq);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(q[0][mt], aq + (uint32_t)(8 * mt) * cx.L.astride);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int cur = g & 1, nxt = cur ^ 1;
      if (g < 3) {
        ldmatrix_x4(r[nxt], wq + 32u * (g + 1));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(q[nxt][mt], aq + (uint32_t)(8 * mt) * cx.L.astride + 64u * (g + 1));
      }
      uint32_t alo[4], ahi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        alo[i] = (r[cur][i] & 0x0f0f0f0fu) | (((hq[i] >> (2 * g)) & 0x01010101u) << 4);
        ahi[i] = ((r[cur][i] >> 4) & 0x0f0f0f0fu) | (((hq[i] >> (2 * g + 1)) & 0x01010101u) << 4);
      }
      int cl[MT][4], ch[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_u8s8_k32(cl[mt], alo, q[cur][mt][0], q[cur][mt][1]);
        mma_u8s8_k32(ch[mt], ahi, q[cur][mt][2], q[cur][mt][3]);
      }
      const int sh = 16 * (g & 1);
      const int s0l = (int)((sc0[g >> 1] >> sh) & 0xff), s0h = (int)((sc0[g >> 1] >> (sh + 8)) & 0xff);
      const int s1l = (int)((sc1[g >> 1] >> sh) & 0xff), s1h = (int)((sc1[g >> 1] >> (sh + 8)) & 0xff);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        Slo[mt][0] += cl[mt][0] * s0l, Slo[mt][1] += cl[mt][1] * s0l, Slo[mt][2] += cl[mt][2] * s1l, Slo[mt][3] += cl[mt][3] * s1l;
        Shi[mt][0] += ch[mt][0] * s0h, Shi[mt][1] += ch[mt][1] * s0h, Shi[mt][2] += ch[mt][2] * s1h, Shi[mt][3] += ch[mt][3] * s1h;
      }
    }
    const float d0 = h2f_bits(h0.x & 0xffffu), dm0 = h2f_bits(h0.x >> 16);
    const float d1 = h2f_bits(h1.x & 0xffffu), dm1 = h2f_bits(h1.x >> 16);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m0 = 8 * mt + 2 * cx.tig;
      const uint4 ba = lds128(cx.act_s + cx.L.off_aux + (uint32_t)m0 * cx.L.aux_stride + (uint32_t)b * 16u);
      const uint4 bb = lds128(cx.act_s + cx.L.off_aux + (uint32_t)(m0 + 1) * cx.L.aux_stride + (uint32_t)b * 16u);
      auto mins = [](const uint4& bs, const uint32_t (&mn)[2]) {
        return __dp2a_hi((int)bs.w, (int)mn[1], __dp2a_lo((int)bs.z, (int)mn[1], __dp2a_hi((int)bs.y, (int)mn[0], __dp2a_lo((int)bs.x, (int)mn[0], 0))));
      };
      const int T0 = mins(ba, mn0), T1 = mins(bb, mn0), T2 = mins(ba, mn1), T3 = mins(bb, mn1);
      const uint2 ydw = lds64(cx.act_s + cx.L.off_d + (uint32_t)(b * 16 + m0) * 4u);
      const float ya = __uint_as_float(ydw.x), yb = __uint_as_float(ydw.y);
      facc[mt][0] += (d0 * ya) * (float)(Slo[mt][0] + Shi[mt][0]) - (dm0 * ya) * (float)T0;
      facc[mt][1] += (d0 * yb) * (float)(Slo[mt][1] + Shi[mt][1]) - (dm0 * yb) * (float)T1;
      facc[mt][2] += (d1 * ya) * (float)(Slo[mt][2] + Shi[mt][2]) - (dm1 * ya) * (float)T2;
      facc[mt][3] += (d1 * yb) * (float)(Slo[mt][3] + Shi[mt][3]) - (dm1 * yb) * (float)T3;
    }
  }
};

// ------------------------------------------------------------------------------------------------ Q8_0
struct MbQ8_0 {
  static constexpr int kType = kQ8_0;
  static constexpr int kBytes256 = 272;  // eight 34-byte blocks
  static constexpr int kAuxBytesPer256 = 0, kAuxPlanes = 0, kScalesPer256 = 8;
  static constexpr bool kRowsAligned = true;  // 272 = 17 * 16
  __device__ static void stage_aux(const ActPlanes& act, int k, int a0, int ac, int rows, int cb0, int cbn, uint8_t* area,
                                   const MbActLayout& L, int t, int nt) {
    const int nb32 = k >> 5;
    float* d = reinterpret_cast<float*>(area + L.off_d);
    const int per = cbn * 8;
    for (int i = t; i < rows * per; i += nt) {
      const int r = i / per, c = i - r * per;
      d[c * 16 + r] = r < ac ? act.d[(size_t)(a0 + r) * nb32 + cb0 * 8 + c] : 0.f;
    }
  }
  template <int MT>
  __device__ __forceinline__ static void block_step(const MbCtx& cx, int b, uint32_t, uint32_t, float (&facc)[MT][4]) {
    const uint32_t r0 = cx.tile_s + cx.row_off(cx.gid) + (uint32_t)b * 272u;
    const uint32_t r1 = cx.tile_s + cx.row_off(cx.gid + 8) + (uint32_t)b * 272u;
    // B fragments: MT == 2: rows (lane & 7) + 8 * bit 4, byte column 16 * bit 3; MT == 1: lanes 0-15 address rows and columns
    const uint32_t aq = cx.act_s + (uint32_t)((cx.lane & 7) + (MT == 2 ? 8 * (cx.lane >> 4) : 0)) * cx.L.astride + (uint32_t)b * 256u +
                        16u * ((cx.lane >> 3) & 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // one 34-byte block: f16 scale, 32 int8
      const uint32_t o = 34u * j;
      const float dw0 = h2f_bits(lds_u16_addr(r0 + o)), dw1 = h2f_bits(lds_u16_addr(r1 + o));
      uint32_t a[4];
      a[0] = lds_u32_2b_addr(r0 + o + 2u + 4u * cx.tig);
      a[1] = lds_u32_2b_addr(r1 + o + 2u + 4u * cx.tig);
      a[2] = lds_u32_2b_addr(r0 + o + 18u + 4u * cx.tig);
      a[3] = lds_u32_2b_addr(r1 + o + 18u + 4u * cx.tig);
      uint32_t q[4];
      if (MT == 2) {
        ldmatrix_x4(q, aq + 32u * j);
      } else {
        uint32_t q2[2];
        ldmatrix_x2(q2, aq + 32u * j);
        q[0] = q2[0], q[1] = q2[1], q[2] = 0, q[3] = 0;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        int c[4];
        mma_s8s8_k32(c, a, q[2 * mt], q[2 * mt + 1]);
        const uint2 ydw = lds64(cx.act_s + cx.L.off_d + (uint32_t)((b * 8 + j) * 16 + 8 * mt + 2 * cx.tig) * 4u);
        const float ya = __uint_as_float(ydw.x), yb = __uint_as_float(ydw.y);
        facc[mt][0] += (dw0 * ya) * (float)c[0];
        facc[mt][1] += (dw0 * yb) * (float)c[1];
        facc[mt][2] += (dw1 * ya) * (float)c[2];
        facc[mt][3] += (dw1 * yb) * (float)c[3];
      }
    }
  }
};

// ------------------------------------------------------------------------------------------------ Q4_0, Q5_0
// 32-element blocks without a minimum (fuel-quantized/src/k_quants.rs:177-269, 463-559): f16 scale, for Q5_0 32 fifth bits,
// 16 bytes of nibbles - byte t holds element t (low nibble) and element 16 + t (high nibble). The values minus their
// offset (8, or 16 with the fifth bit) are signed bytes, so one s8 x s8 instruction per block against the Q8_0 activation
// block gives the reference's integer sum directly; activation scales as for Q8_0.
template <int kBlk, bool kFive>
struct MbLegacy0 : MbQ8_0 {
  static constexpr int kType = kFive ? kQ5_0 : kQ4_0;
  static constexpr int kBytes256 = 8 * kBlk;  // 144 or 176: rows and chunks start on 16-byte boundaries
  __device__ __forceinline__ static uint32_t spread4(uint32_t bits) {  // bit i of a nibble -> bit 4 of byte i
    return (((bits & 0xFu) * 0x00204081u) & 0x01010101u) << 4;
  }
  template <int MT>
  __device__ __forceinline__ static void block_step(const MbCtx& cx, int b, uint32_t, uint32_t, float (&facc)[MT][4]) {
    const uint32_t r0 = cx.tile_s + cx.row_off(cx.gid) + (uint32_t)b * (uint32_t)kBytes256;
    const uint32_t r1 = cx.tile_s + cx.row_off(cx.gid + 8) + (uint32_t)b * (uint32_t)kBytes256;
    const uint32_t aq = cx.act_s + (uint32_t)((cx.lane & 7) + (MT == 2 ? 8 * (cx.lane >> 4) : 0)) * cx.L.astride + (uint32_t)b * 256u +
                        16u * ((cx.lane >> 3) & 1);
    constexpr uint32_t kOffQs = (uint32_t)kBlk - 16u;
    constexpr uint32_t kBias = kFive ? 0x10101010u : 0x08080808u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t o = (uint32_t)kBlk * j;
      const float dw0 = h2f_bits(lds_u16_addr(r0 + o)), dw1 = h2f_bits(lds_u16_addr(r1 + o));
      const uint32_t w0 = lds_u32_2b_addr(r0 + o + kOffQs + 4u * cx.tig), w1 = lds_u32_2b_addr(r1 + o + kOffQs + 4u * cx.tig);
      uint32_t lo0 = w0 & 0x0f0f0f0fu, hi0 = (w0 >> 4) & 0x0f0f0f0fu, lo1 = w1 & 0x0f0f0f0fu, hi1 = (w1 >> 4) & 0x0f0f0f0fu;
      if (kFive) {  // bit t of qh belongs to element t, bit 16 + t to element 16 + t
        const uint32_t h0 = lds_u32_2b_addr(r0 + o + 2u), h1 = lds_u32_2b_addr(r1 + o + 2u);
        lo0 |= spread4(h0 >> (4 * cx.tig)), hi0 |= spread4(h0 >> (16 + 4 * cx.tig));
        lo1 |= spread4(h1 >> (4 * cx.tig)), hi1 |= spread4(h1 >> (16 + 4 * cx.tig));
      }
      uint32_t a[4];
      a[0] = __vsub4(lo0, kBias), a[1] = __vsub4(lo1, kBias), a[2] = __vsub4(hi0, kBias), a[3] = __vsub4(hi1, kBias);
      uint32_t q[4];
      if (MT == 2) {
        ldmatrix_x4(q, aq + 32u * j);
      } else {
        uint32_t q2[2];
        ldmatrix_x2(q2, aq + 32u * j);
        q[0] = q2[0], q[1] = q2[1], q[2] = 0, q[3] = 0;
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        int c[4];
        mma_s8s8_k32(c, a, q[2 * mt], q[2 * mt + 1]);
        const uint2 ydw = lds64(cx.act_s + cx.L.off_d + (uint32_t)((b * 8 + j) * 16 + 8 * mt + 2 * cx.tig) * 4u);
        const float ya = __uint_as_float(ydw.x), yb = __uint_as_float(ydw.y);
        facc[mt][0] += (dw0 * ya) * (float)c[0];
        facc[mt][1] += (dw0 * yb) * (float)c[1];
        facc[mt][2] += (dw1 * ya) * (float)c[2];
        facc[mt][3] += (dw1 * yb) * (float)c[3];
      }
    }
  }
};
using MbQ4_0 = MbLegacy0<18, false>;
using MbQ5_0 = MbLegacy0<22, true>;

// ------------------------------------------------------------------------------------------------ Q6_K
struct MbQ6K {
  static constexpr int kType = kQ6K;
  static constexpr int kBytes256 = 210;
  static constexpr int kAuxBytesPer256 = 16, kAuxPlanes = 2, kScalesPer256 = 1;
  static constexpr bool kRowsAligned = false;  // 210-byte blocks: rows start at any even byte
  __device__ static void stage_aux(const ActPlanes& act, int k, int a0, int ac, int rows, int cb0, int cbn, uint8_t* area,
                                   const MbActLayout& L, int t, int nt) {
    const int nblk = k >> 8;
    const int s16 = cbn * 16;
    for (int i = t; i < rows * s16; i += nt) {  // 16-element sums (|s| <= 2048) as 64 * hi + lo, lo in 0..63
      const int r = i / s16, c = i - r * s16;
      int v = 0;
      if (r < ac) v = act.bsums[(size_t)(a0 + r) * (k >> 4) + cb0 * 16 + c];
      const int lo = v & 63, hi = (v - lo) >> 6;
      area[L.off_aux + (size_t)r * L.aux_stride + c] = (uint8_t)lo;
      area[L.off_aux + L.aux_plane + (size_t)r * L.aux_stride + c] = (uint8_t)(int8_t)hi;
    }
    float* d = reinterpret_cast<float*>(area + L.off_d);
    for (int i = t; i < rows * cbn; i += nt) {
      const int r = i / cbn, c = i - r * cbn;
      d[c * 16 + r] = r < ac ? act.d[(size_t)(a0 + r) * nblk + cb0 + c] : 0.f;
    }
  }
  // skew0 / skew1: byte offsets (0..14, even) of rows gid and gid + 8 inside their staged slots
  template <int MT>
  __device__ __forceinline__ static void block_step(const MbCtx& cx, int b, uint32_t skew0, uint32_t skew1, float (&facc)[MT][4]) {
    const uint32_t r0 = cx.tile_s + cx.row_off(cx.gid) + skew0 + (uint32_t)b * 210u;
    const uint32_t r1 = cx.tile_s + cx.row_off(cx.gid + 8) + skew1 + (uint32_t)b * 210u;
    // scales: 16 signed bytes per row; this lane's word holds groups 4 tig .. 4 tig + 3 (the A fragment of the correction)
    const uint32_t scw0 = lds_u32_2b_addr(r0 + 192u + 4u * cx.tig), scw1 = lds_u32_2b_addr(r1 + 192u + 4u * cx.tig);
    uint32_t sc0[4], sc1[4];  // all 16, for the per-group scaling
#pragma unroll
    for (int i = 0; i < 4; ++i) sc0[i] = lds_u32_2b_addr(r0 + 192u + 4u * i), sc1[i] = lds_u32_2b_addr(r1 + 192u + 4u * i);
    const float d0 = h2f_bits(lds_u16_addr(r0 + 208u)), d1 = h2f_bits(lds_u16_addr(r1 + 208u));
    int S[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) S[mt][i] = 0;
    // B fragments of a 128-element half: four 16-element groups per ldmatrix.x4, rows (lane & 7), 16-byte piece lane >> 3
    const uint32_t aq = cx.act_s + (uint32_t)(cx.lane & 7) * cx.L.astride + (uint32_t)b * 256u + 16u * (cx.lane >> 3);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t bq[MT][8];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t q[4];
        ldmatrix_x4(q, aq + (uint32_t)(8 * mt) * cx.L.astride + 128u * h);
        bq[mt][0] = q[0], bq[mt][1] = q[1], bq[mt][2] = q[2], bq[mt][3] = q[3];
        ldmatrix_x4(q, aq + (uint32_t)(8 * mt) * cx.L.astride + 128u * h + 64u);
        bq[mt][4] = q[0], bq[mt][5] = q[1], bq[mt][6] = q[2], bq[mt][7] = q[3];
      }
#pragma unroll
      for (int s = 0; s < 2; ++s) {  // l = 16 s + 4 tig .. + 3
        const uint32_t lo = 64u * h + 16u * s + 4u * cx.tig, ho = 128u + 32u * h + 16u * s + 4u * cx.tig;
        const uint32_t qla0 = lds_u32_2b_addr(r0 + lo), qlb0 = lds_u32_2b_addr(r0 + lo + 32u), qh0 = lds_u32_2b_addr(r0 + ho);
        const uint32_t qla1 = lds_u32_2b_addr(r1 + lo), qlb1 = lds_u32_2b_addr(r1 + lo + 32u), qh1 = lds_u32_2b_addr(r1 + ho);
        uint32_t v0[4], v1[4];  // quadrant q: elements 128 h + 32 q + l (fuel-quantized/src/k_quants.rs:2170-2185)
        v0[0] = (qla0 & 0x0f0f0f0fu) | ((qh0 << 4) & 0x30303030u);
        v0[1] = (qlb0 & 0x0f0f0f0fu) | ((qh0 << 2) & 0x30303030u);
        v0[2] = ((qla0 >> 4) & 0x0f0f0f0fu) | (qh0 & 0x30303030u);
        v0[3] = ((qlb0 >> 4) & 0x0f0f0f0fu) | ((qh0 >> 2) & 0x30303030u);
        v1[0] = (qla1 & 0x0f0f0f0fu) | ((qh1 << 4) & 0x30303030u);
        v1[1] = (qlb1 & 0x0f0f0f0fu) | ((qh1 << 2) & 0x30303030u);
        v1[2] = ((qla1 >> 4) & 0x0f0f0f0fu) | (qh1 & 0x30303030u);
        v1[3] = ((qlb1 >> 4) & 0x0f0f0f0fu) | ((qh1 >> 2) & 0x30303030u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int G = 8 * h + 2 * q + s;  // scale group of these 16 elements
          const int s0 = (int)(int8_t)((sc0[G >> 2] >> (8 * (G & 3))) & 0xff), s1 = (int)(int8_t)((sc1[G >> 2] >> (8 * (G & 3))) & 0xff);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            int c[4];
            mma_u8s8_k16(c, v0[q], v1[q], bq[mt][2 * q + s]);
            S[mt][0] += c[0] * s0, S[mt][1] += c[1] * s0, S[mt][2] += c[2] * s1, S[mt][3] += c[3] * s1;
          }
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      // correction sum_g scale_g * bsum_g = 64 * (scales . hi) + (scales . lo), k = 16 groups
      const uint32_t aux = cx.act_s + cx.L.off_aux + (uint32_t)(8 * mt + cx.gid) * cx.L.aux_stride + (uint32_t)b * 16u + 4u * cx.tig;
      uint32_t blo, bhi;
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(blo) : "r"(aux));
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(bhi) : "r"(aux + (uint32_t)cx.L.aux_plane));
      int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
      mma_s8s8_k16_acc(cl, scw0, scw1, blo);
      mma_s8s8_k16_acc(ch, scw0, scw1, bhi);
      const uint2 ydw = lds64(cx.act_s + cx.L.off_d + (uint32_t)(b * 16 + 8 * mt + 2 * cx.tig) * 4u);
      const float ya = __uint_as_float(ydw.x), yb = __uint_as_float(ydw.y);
      facc[mt][0] += (d0 * ya) * (float)(S[mt][0] - 32 * (64 * ch[0] + cl[0]));
      facc[mt][1] += (d0 * yb) * (float)(S[mt][1] - 32 * (64 * ch[1] + cl[1]));
      facc[mt][2] += (d1 * ya) * (float)(S[mt][2] - 32 * (64 * ch[2] + cl[2]));
      facc[mt][3] += (d1 * yb) * (float)(S[mt][3] - 32 * (64 * ch[3] + cl[3]));
    }
  }
};

// ------------------------------------------------------------------------------------------------ kernel
// barrier among `count` threads that also ORs a predicate over them
__device__ __forceinline__ bool bar_or(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %3, 0;\n\t"
      "barrier.cta.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

template <class F, int MT>
__global__ void __launch_bounds__(kMbThreads, 1) mma_batch_kernel(const MmaBatchParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  MmaBatchHeader* hd = reinterpret_cast<MmaBatchHeader*>(smem_raw);
  uint8_t* stages = smem_raw + align_up(sizeof(MmaBatchHeader), 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kActRows = 8 * MT;
  const int S = p.num_stages, NG = p.n_wgroups, GW = kMbConsumerWarps / NG;
  const int nblk = p.k >> 8, KC = p.kc_blocks, n_kc = (nblk + KC - 1) / KC;
  const int grp = blockIdx.y;
  // this block's share of the weight rows, in whole 16-row tiles
  const int n_tiles = (p.n + 15) >> 4;
  const int t_begin = (int)((int64_t)n_tiles * blockIdx.x / gridDim.x), t_end = (int)((int64_t)n_tiles * (blockIdx.x + 1) / gridDim.x);
  const int r_begin = t_begin * 16, r_end = (t_end * 16 < p.n) ? t_end * 16 : p.n;
  const int n_iter = t_end - t_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hd->full[s], 1);
      mbar_init(&hd->empty[s], GW);
    }
    mbar_init(&hd->acts, 1);
    hd->dead = 0;
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();
  // Row ranges and activations come from the preceding kernels; the weights do not, so with one group of fixed size
  // (a dense batch) the producer starts streaming before the predecessor has finished.
  const bool early = warp == kMbConsumerWarps && !p.offsets;  // the producer of a dense batch
  if (!early) pdl_wait();
  const int m_begin = p.offsets ? p.offsets[grp] : 0;
  const int m_count = p.offsets ? p.offsets[grp + 1] - m_begin : p.fixed_rows;
  if (m_count <= 0 || n_iter <= 0) return;  // nothing is streamed for a group without rows
  const int n_pass = (m_count + kActRows - 1) / kActRows;
  const int total_iter = n_pass * n_kc * n_iter;
  const int64_t base = (int64_t)grp * p.group_bytes;

  if (warp == kMbConsumerWarps) {
    // ---------------- producer: one bulk copy per group of rows_per_copy consecutive weight rows, a lane per copy.
    // Issuing a bulk copy costs ~60-90 ns whatever its size, so one copy per 1-2 KB row caps the stream well below HBM
    // speed; when whole rows are staged (no k chunks) consecutive rows are contiguous in memory and travel together,
    // at the price of a rows_per_copy-way bank conflict on the weight fragment loads, which are few.
    const int64_t tma_limit = p.total_bytes & ~(int64_t)15;
    const int RPC = p.rows_per_copy;
    bool ok = true;
    int it = 0, kc = 0, issued = 0;
    for (int g = 0; g < total_iter; ++g) {
      const int s = g % S;
      if (g >= S) {
        if (lane == 0) ok = mbar_poll_bounded(&hd->empty[s], ((g / S) - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) record_dev_error(kErrEmptyWait);
          break;
        }
      }
      const int row0 = r_begin + it * 16;
      const int rows_here = ((row0 + 16 < r_end) ? row0 + 16 : r_end) - row0;
      const int cb0 = kc * KC, cbn = (nblk - cb0 < KC) ? nblk - cb0 : KC;  // this sweep's blocks of every row
      // byte range of a copy (rows lane * RPC ..), widened to 16-byte boundaries (the consumer re-derives the skew)
      uint32_t my_bytes = 0;
      int64_t a0 = 0;
      uint8_t* dst = nullptr;
      if (lane * RPC < rows_here) {
        const int nr = rows_here - lane * RPC < RPC ? rows_here - lane * RPC : RPC;
        const int64_t b0 = base + (int64_t)(row0 + lane * RPC) * p.row_bytes + (int64_t)cb0 * F::kBytes256;
        const int64_t b1 = b0 + (int64_t)(nr - 1) * p.row_bytes + (int64_t)cbn * F::kBytes256;
        a0 = b0 & ~(int64_t)15;
        int64_t a1 = (b1 + 15) & ~(int64_t)15;
        if (a1 > tma_limit) a1 = tma_limit;
        dst = stages + (size_t)s * p.stage_stride + (size_t)lane * p.wstride;
        if (b1 > a1) {  // the buffer ends off a 16-byte boundary: its last bytes by hand
          const int64_t from = a1 > a0 ? a1 : a0;
          for (int64_t j = from; j < b1; ++j) dst[j - a0] = p.w[j];
        }
        my_bytes = a1 > a0 ? (uint32_t)(a1 - a0) : 0u;
      }
      uint32_t tot = my_bytes;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, off);
      if (lane == 0) {
        if (tot)
          mbar_arrive_expect_tx(&hd->full[s], tot);
        else
          mbar_arrive(&hd->full[s]);
      }
      __syncwarp();
      if (my_bytes) bulk_g2s(dst, p.w + a0, my_bytes, &hd->full[s]);
      if (g == 0) {
        // The first sweep's activation rows, one bulk copy per row, right behind the first weight tile: requested any
        // later they would queue behind every weight copy in flight (the rows of later sweeps are staged by the consumers).
        if (early) pdl_wait();
        const int ac0 = m_count < kActRows ? m_count : kActRows;
        const int cbn0 = nblk < KC ? nblk : KC;
        const MbActLayout L0 = mb_act_layout<F>(KC, kActRows);
        if (lane == 0) mbar_arrive_expect_tx(&hd->acts, (uint32_t)ac0 * (uint32_t)cbn0 * 256u);
        __syncwarp();
        if (lane < ac0)
          bulk_g2s(smem_raw + p.act_off + (size_t)lane * L0.astride, p.act.qs + (size_t)(m_begin + lane) * p.k, (uint32_t)cbn0 * 256u,
                   &hd->acts);
      }
      issued = g + 1;
      if (++it == n_iter) {
        it = 0;
        if (++kc == n_kc) kc = 0;
      }
    }
    if (!ok && lane == 0) {
      for (int g = (issued > S ? issued - S : 0); g < issued; ++g)
        if (!mbar_poll_bounded(&hd->full[g % S], (g / S) & 1)) record_dev_error(kErrDrainWait);
    }
    return;
  }

  // ---------------- consumers
  uint8_t* act_area = smem_raw + p.act_off;
  constexpr int nt_const = 32 * kMbConsumerWarps;
  const int t = threadIdx.x, nt = nt_const;
  const int gi = warp / GW, kpart = warp - gi * GW;   // warp group and this warp's share of k
  const int gt = t - gi * 32 * GW, gnt = 32 * GW;      // thread index within the group
  float* part = reinterpret_cast<float*>(smem_raw + p.part_off) + (size_t)gi * GW * (MT * 128);  // [k-part][MT * 128]
  MbCtx cx;
  cx.lane = lane, cx.gid = lane >> 2, cx.tig = lane & 3;
  cx.wstride = p.wstride;
  cx.rpc_shift = p.rows_per_copy == 4 ? 2 : p.rows_per_copy == 2 ? 1 : 0;
  cx.row_bytes = p.row_bytes;
  cx.L = mb_act_layout<F>(KC, kActRows);
  cx.act_s = smem_u32(act_area);
  bool dead = false;  // uniform within a warp group

  int g_base = 0;  // stage counter at the start of the sweep
  for (int pass = 0; pass < n_pass; ++pass) {
    const int a0 = m_begin + pass * kActRows;
    const int ac = (m_count - pass * kActRows < kActRows) ? m_count - pass * kActRows : kActRows;
    for (int kc = 0; kc < n_kc; ++kc, g_base += n_iter) {
      const int cb0 = kc * KC, cbn = (nblk - cb0 < KC) ? nblk - cb0 : KC;  // this sweep's blocks
      const int b_begin = cbn * kpart / GW, b_end = cbn * (kpart + 1) / GW;
      // every consumer thread passes both barriers of every sweep, dead or not
      if (pass > 0 || kc > 0) asm volatile("bar.sync 1, %0;" ::"n"(32 * kMbConsumerWarps) : "memory");  // previous rows are done with
      if (!dead) {
        // stage the activation rows (this sweep's columns): quants into padded rows, zero rows past ac;
        // 512 / kActRows threads per row
        constexpr int kTpr = nt_const / kActRows;
        const int r = t / kTpr, c0 = t - r * kTpr;
        const int q16 = cbn * 16;  // 16-byte pieces per row
        const bool by_producer = pass == 0 && kc == 0;  // rows < ac arrive by bulk copy (see the producer)
        if (!by_producer || r >= ac) {
          const uint4* src = reinterpret_cast<const uint4*>(p.act.qs + (size_t)(a0 + (r < ac ? r : 0)) * p.k + (size_t)cb0 * 256);
          uint4* dstq = reinterpret_cast<uint4*>(act_area + (size_t)r * cx.L.astride);
          for (int c = c0; c < q16; c += kTpr) dstq[c] = r < ac ? src[c] : make_uint4(0, 0, 0, 0);
        }
        F::stage_aux(p.act, p.k, a0, ac, kActRows, cb0, cbn, act_area, cx.L, t, nt);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kMbConsumerWarps) : "memory");
      if (pass == 0 && kc == 0 && !dead && !mbar_wait_bounded(&hd->acts, 0)) {
        record_dev_error(kErrFullWait);
        hd->dead = 1;  // every group sees it at its next barrier
      }

      for (int it = gi; it < n_iter && !dead; it += NG) {
        const int g = g_base + it, s = g % S;
        bool bad = false;
        if (!mbar_wait_bounded(&hd->full[s], (g / S) & 1)) {
          record_dev_error(kErrFullWait);
          hd->dead = 1;
          bad = true;
        }
        const int row0 = r_begin + it * 16;
        const int rows_here = ((row0 + 16 < r_end) ? row0 + 16 : r_end) - row0;
        float facc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) facc[mt][i] = 0.f;
        if (!bad) {
          cx.tile_s = smem_u32(stages) + (uint32_t)s * p.stage_stride;
          uint32_t skew0 = 0, skew1 = 0;
          if (!F::kRowsAligned) {
            // the skew of a staged copy is that of its first row
            const int first = cx.gid & ~(p.rows_per_copy - 1);
            const int64_t c0 = base + (int64_t)(row0 + first) * p.row_bytes + (int64_t)cb0 * F::kBytes256;
            skew0 = (uint32_t)(c0 & 15);
            skew1 = (uint32_t)((c0 + 8 * (int64_t)p.row_bytes) & 15);
          }
          for (int b = b_begin; b < b_end; ++b) F::template block_step<MT>(cx, b, skew0, skew1, facc);
        }
        // partial sums of the group's warps meet in shared memory and are added in k order
        float* my = part + (size_t)kpart * (MT * 128);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) my[(mt * 4 + i) * 32 + lane] = facc[mt][i];
        dead = bar_or(2 + gi, gnt, bad || hd->dead != 0);
        if (!dead) {
          // slot = (mt * 4 + i) * 32 + lane of the accumulator fragment layout
          for (int slot = gt; slot < MT * 128; slot += gnt) {
            float sum = part[slot];
            for (int kp = 1; kp < GW; ++kp) sum += part[(size_t)kp * (MT * 128) + slot];
            const int ln = slot & 31, fi = slot >> 5, mt = fi >> 2, i = fi & 3;
            const int m = 8 * mt + 2 * (ln & 3) + (i & 1), col = (ln >> 2) + 8 * (i >> 1);
            if (m < ac && col < rows_here) {
              const int srow = a0 + m;
              const int orow = p.out_rows ? p.out_rows[srow] : srow;
              float* dst = p.y + (size_t)orow * p.n + row0 + col;
              *dst = kc == 0 ? sum : *dst + sum;  // later sweeps add, in order, by the same thread
            }
          }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(2 + gi), "r"(gnt) : "memory");  // partials consumed
        __syncwarp();
        if (lane == 0) mbar_arrive(&hd->empty[s]);
      }
    }
  }
}

}  // namespace fq
