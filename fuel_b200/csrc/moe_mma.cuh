// Grouped Q4_K mat-vec for a handful of activation rows per weight matrix (an expert's routed rows, or a
// small dense batch), on the integer tensor-core instruction mma.sync m16n8k32 (s8 x s8 -> s32).
//
// Same arithmetic as the dp4a decode kernels: per 32-element sub-block an exact integer dot of the 4-bit
// weights with the 8-bit activations, combined per 256-block as
//   y += (d * yd) * sum_j sc_j * isum_j  -  (dmin * yd) * sum_j mn_j * bsum_j
// (the reference's BlockQ4K::vec_dot, fuel-quantized/src/k_quants.rs:1388-1468, with the two integer sums
// kept exact in 32 bits). An MMA tile is 16 activation rows x 8 weight rows x one sub-block; the plain
// dp4a form spends ~3 instructions per 128 multiply-adds, this one ~1 per 180, which is what makes the
// 16-rows-per-expert case bandwidth-bound instead of issue-bound.
//
// Layout in shared memory (per thread block, two per SM):
//   * activation rows of the current pass (16), row stride k + 16 bytes so that the eight rows a warp's
//     fragment loads touch fall in different banks; their 32-element sums and block scales beside them;
//   * a ring of weight stages, each R rows copied by one bulk copy per row into rows of stride
//     row_bytes + 16 for the same reason.
// Work split inside a stage: R / 8 tiles of 8 weight rows, each tile shared by 64 / R warps that take
// consecutive ranges of the 256-blocks along k; their partial sums meet in shared memory and are added in
// a fixed order. When a row of activations does not fit (large k), k is cut into chunks of kc_blocks blocks and
// the same rows are swept once per chunk, each sweep adding into y. Every wait is bounded.
#pragma once
#include "decode_regs.cuh"
#include "fq_common.cuh"
#include "mma_batch.cuh"
#include "moe.cuh"

namespace fq {

struct MmaParams {
  const uint8_t* w;      // [n_groups][n][k] Q4_K blocks
  ActPlanes act;         // plain activation planes of all rows
  const int* offsets;    // [n_groups + 1] row ranges, or null: one group holding rows [0, fixed_rows)
  const int* out_rows;   // row -> output row, or null for the identity
  float* y;              // [rows][n]
  int64_t group_bytes;   // n * row_bytes
  int fixed_rows;
  int n, k, row_bytes;
  int rows_per_stage;    // R: 8, 16 or 32
  int num_stages, stage_stride;
  int act_off, part_off; // shared-memory offsets of the activation area and of the partial-sum area
  int kc_blocks;         // 256-blocks of k handled per sweep (all of k when it fits in shared memory; else the
                         // sweeps' results are added into y in order, by the thread that wrote the first one)
};

constexpr int kMmaActRows = 16;

struct MmaSmemHeader {
  uint64_t full[kDecodeMaxStages];
  uint64_t empty[kDecodeMaxStages];
  int dead;  // a consumer warp's bounded wait expired: every warp skips the remaining work but keeps meeting the barriers
};

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__host__ __device__ inline size_t mma_act_bytes(int kc_blocks) {
  // one k-chunk of the activation rows: quants (padded rows), 32-element sums (int16), block scales (f32)
  return align_up((size_t)kMmaActRows * (kc_blocks * 256 + 16), 128) + align_up((size_t)kMmaActRows * (kc_blocks * 16 + 16), 128) +
         align_up((size_t)kMmaActRows * kc_blocks * 4, 128);
}

__global__ void __launch_bounds__(kDecodeThreads, 2) mma_q4k_kernel(const MmaParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  MmaSmemHeader* hd = reinterpret_cast<MmaSmemHeader*>(smem_raw);
  uint8_t* stages = smem_raw + align_up(sizeof(MmaSmemHeader), 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.num_stages, R = p.rows_per_stage;
  const int nblk = p.k >> 8, KC = p.kc_blocks, n_kc = (nblk + KC - 1) / KC;
  const int wstride = KC * Q4KL::kBytes + 16, astride = KC * 256 + 16;  // rows of one k-chunk, padded
  const int grp = blockIdx.y;
  const int r_begin = (int)((int64_t)p.n * blockIdx.x / gridDim.x);
  const int r_end = (int)((int64_t)p.n * (blockIdx.x + 1) / gridDim.x);
  const int n_iter = (r_end - r_begin + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hd->full[s], 1);
      mbar_init(&hd->empty[s], kDecodeConsumerWarps);
    }
    hd->dead = 0;
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();  // row ranges and activations come from the preceding kernels
  const int m_begin = p.offsets ? p.offsets[grp] : 0;
  const int m_count = p.offsets ? p.offsets[grp + 1] - m_begin : p.fixed_rows;
  if (m_count <= 0 || n_iter <= 0) return;  // nothing is streamed for a group without rows
  const int n_pass = (m_count + kMmaActRows - 1) / kMmaActRows;
  const int total_iter = n_pass * n_kc * n_iter;
  const int64_t base = (int64_t)grp * p.group_bytes;

  if (warp == kDecodeConsumerWarps) {
    // ---------------- producer: one bulk copy per weight row, a lane per row
    bool ok = true;
    int it = 0, kc = 0, issued = 0;
    for (int g = 0; g < total_iter; ++g) {
      const int s = g % S;
      if (g >= S) {
        if (lane == 0) ok = mbar_wait_bounded(&hd->empty[s], ((g / S) - 1) & 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          if (lane == 0) record_dev_error(kErrEmptyWait);
          break;
        }
      }
      const int row0 = r_begin + it * R;
      const int rows_here = ((row0 + R < r_end) ? row0 + R : r_end) - row0;
      const int cb0 = kc * KC, cbn = (nblk - cb0 < KC) ? nblk - cb0 : KC;  // this sweep's blocks of every row
      const uint32_t cbytes = (uint32_t)cbn * Q4KL::kBytes;
      if (lane == 0) mbar_arrive_expect_tx(&hd->full[s], (uint32_t)rows_here * cbytes);
      __syncwarp();
      if (lane < rows_here)
        bulk_g2s(stages + (size_t)s * p.stage_stride + (size_t)lane * wstride,
                 p.w + base + (int64_t)(row0 + lane) * p.row_bytes + (int64_t)cb0 * Q4KL::kBytes, cbytes, &hd->full[s]);
      issued = g + 1;
      if (++it == n_iter) {
        it = 0;
        if (++kc == n_kc) kc = 0;
      }
    }
    if (!ok && lane == 0) {
      for (int g = (issued > S ? issued - S : 0); g < issued; ++g)
        if (!mbar_wait_bounded(&hd->full[g % S], (g / S) & 1)) record_dev_error(kErrDrainWait);
    }
    return;
  }

  // ---------------- consumers
  uint8_t* act_qs = smem_raw + p.act_off;
  int16_t* act_bs = reinterpret_cast<int16_t*>(act_qs + align_up((size_t)kMmaActRows * astride, 128));
  const int bstride = KC * 16 + 16;  // bytes per row of 32-sums (padded: rows fall in different banks)
  float* act_d = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(act_bs) + align_up((size_t)kMmaActRows * bstride, 128));
  float* part = reinterpret_cast<float*>(smem_raw + p.part_off);  // [tile][k-part][128]
  const int t = threadIdx.x, nt = 32 * kDecodeConsumerWarps;
  const int tiles = R >> 3;                      // 8-row tiles per stage
  const int ksplit = kDecodeConsumerWarps / tiles;  // warps sharing a tile
  const int tile = warp / ksplit, kpart = warp - tile * ksplit;
  const int gid = lane >> 2, tig = lane & 3;

  int g = 0;
  bool dead = false;
  for (int pass = 0; pass < n_pass; ++pass) {
    const int a0 = m_begin + pass * kMmaActRows;
    const int ac = (m_count - pass * kMmaActRows < kMmaActRows) ? m_count - pass * kMmaActRows : kMmaActRows;
   for (int kc = 0; kc < n_kc; ++kc) {
    const int cb0 = kc * KC, cbn = (nblk - cb0 < KC) ? nblk - cb0 : KC;  // this sweep's blocks
    const int b_begin = cbn * kpart / ksplit, b_end = cbn * (kpart + 1) / ksplit;
    if (pass > 0 || kc > 0) asm volatile("bar.sync 8, %0;" ::"n"(32 * kDecodeConsumerWarps) : "memory");  // previous rows are done with
    {
      // stage the activation rows (this sweep's columns): quants into padded rows, 16-sums folded to 32-sums, scales;
      // rows past ac are zero
      const int q16 = cbn * 16;  // 16-byte pieces per row
      for (int i = t; i < kMmaActRows * q16; i += nt) {
        const int r = i / q16, c = i - r * q16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < ac) v = reinterpret_cast<const uint4*>(p.act.qs + (size_t)(a0 + r) * p.k + (size_t)cb0 * 256)[c];
        reinterpret_cast<uint4*>(act_qs + (size_t)r * astride)[c] = v;
      }
      const int s32 = cbn * 8;
      for (int i = t; i < kMmaActRows * s32; i += nt) {
        const int r = i / s32, c = i - r * s32;
        int v = 0;
        if (r < ac) {
          const int16_t* bs = p.act.bsums + (size_t)(a0 + r) * (p.k >> 4) + cb0 * 16 + 2 * c;
          v = (int)bs[0] + (int)bs[1];
        }
        *reinterpret_cast<int16_t*>(reinterpret_cast<uint8_t*>(act_bs) + (size_t)r * bstride + 2 * c) = (int16_t)v;
      }
      for (int i = t; i < kMmaActRows * cbn; i += nt) {
        const int r = i / cbn, c = i - r * cbn;
        act_d[r * KC + c] = r < ac ? p.act.d[(size_t)(a0 + r) * nblk + cb0 + c] : 0.f;
      }
    }
    asm volatile("bar.sync 8, %0;" ::"n"(32 * kDecodeConsumerWarps) : "memory");

    for (int it = 0; it < n_iter; ++it, ++g) {
      const int s = g % S;
      // A wait that runs out must not strand the other warps at the named barriers below (their thread counts are
      // fixed): the warp marks the CTA dead and carries on through every barrier, skipping loads, math and stores.
      if (!dead && !mbar_wait_bounded(&hd->full[s], (g / S) & 1)) {
        record_dev_error(kErrFullWait);
        *reinterpret_cast<volatile int*>(&hd->dead) = 1;
      }
      dead = dead || *reinterpret_cast<volatile int*>(&hd->dead) != 0;
      const int row0 = r_begin + it * R;
      const int rows_here = ((row0 + R < r_end) ? row0 + R : r_end) - row0;
      float facc[4] = {0.f, 0.f, 0.f, 0.f};  // (row gid, col 2tig) (gid, 2tig+1) (gid+8, 2tig) (gid+8, 2tig+1)
      if (!dead && tile * 8 < rows_here) {
        // 32-bit shared addresses, so every load below is one ld.shared with an immediate offset
        const uint32_t tile_s = smem_u32(stages) + (uint32_t)s * p.stage_stride + (uint32_t)(tile * 8) * wstride;
        const uint32_t wb_s = tile_s + (uint32_t)gid * wstride + Q4KL::kOffQs + 4 * tig;  // B fragments: weight row gid
        const uint32_t wc_s = tile_s + (uint32_t)(2 * tig) * wstride;                      // accumulator columns: rows 2tig, 2tig+1
        // A fragments by ldmatrix: lane l addresses row (l & 7) + 8 * ((l >> 3) & 1), byte column 16 * (l >> 4)
        const uint32_t aq_s = smem_u32(act_qs) + (uint32_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * astride + 16 * (lane >> 4);
        const uint32_t bs_s = smem_u32(act_bs) + (uint32_t)gid * bstride;
        const uint32_t d_s = smem_u32(act_d) + (uint32_t)gid * KC * 4;
        for (int b = b_begin; b < b_end; ++b) {
          const uint4 h0 = lds128(wc_s + b * Q4KL::kBytes);
          const uint4 h1 = lds128(wc_s + wstride + b * Q4KL::kBytes);
          // eight 6-bit scales / mins per row as bytes of two words (get_scale_min_k4, fuel-quantized/src/utils.rs:50-60)
          const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | (((h0.y >> 6) & 0x03030303u) << 4)};
          const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | (((h0.z >> 6) & 0x03030303u) << 4)};
          const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | (((h1.y >> 6) & 0x03030303u) << 4)};
          const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | (((h1.z >> 6) & 0x03030303u) << 4)};
          const uint4 bl = lds128(bs_s + b * 16);                 // eight 32-sums of activation row gid
          const uint4 bh = lds128(bs_s + 8 * bstride + b * 16);   // ... of row gid + 8
          int S4[4] = {0, 0, 0, 0};
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) {  // 64 elements: low nibbles = sub-block 2gq, high nibbles = 2gq + 1
            const uint32_t q0 = lds32(wb_s + b * Q4KL::kBytes + 32 * gq);
            const uint32_t q1 = lds32(wb_s + b * Q4KL::kBytes + 32 * gq + 16);
#pragma unroll
            for (int sb = 0; sb < 2; ++sb) {
              const int j = 2 * gq + sb;
              const uint32_t b0 = (q0 >> (4 * sb)) & 0x0f0f0f0fu, b1 = (q1 >> (4 * sb)) & 0x0f0f0f0fu;
              uint32_t a[4];
              ldmatrix_x4(a, aq_s + b * 256 + 32 * j);
              int c[4] = {0, 0, 0, 0};
              mma_s8_16832(c, a, b0, b1);
              const int sh = 8 * (j & 3);
              const int s0 = (int)((sc0[j >> 2] >> sh) & 0xff), s1 = (int)((sc1[j >> 2] >> sh) & 0xff);
              S4[0] += c[0] * s0, S4[1] += c[1] * s1, S4[2] += c[2] * s0, S4[3] += c[3] * s1;
            }
          }
          // sum_j min_j * bsum_j: two sub-blocks per dp2a (16-bit sums x 8-bit mins)
          int T4[4];
          T4[0] = __dp2a_hi((int)bl.w, (int)mn0[1], __dp2a_lo((int)bl.z, (int)mn0[1], __dp2a_hi((int)bl.y, (int)mn0[0], __dp2a_lo((int)bl.x, (int)mn0[0], 0))));
          T4[1] = __dp2a_hi((int)bl.w, (int)mn1[1], __dp2a_lo((int)bl.z, (int)mn1[1], __dp2a_hi((int)bl.y, (int)mn1[0], __dp2a_lo((int)bl.x, (int)mn1[0], 0))));
          T4[2] = __dp2a_hi((int)bh.w, (int)mn0[1], __dp2a_lo((int)bh.z, (int)mn0[1], __dp2a_hi((int)bh.y, (int)mn0[0], __dp2a_lo((int)bh.x, (int)mn0[0], 0))));
          T4[3] = __dp2a_hi((int)bh.w, (int)mn1[1], __dp2a_lo((int)bh.z, (int)mn1[1], __dp2a_hi((int)bh.y, (int)mn1[0], __dp2a_lo((int)bh.x, (int)mn1[0], 0))));
          const float d0 = h2f_bits(h0.x & 0xffffu), dm0 = h2f_bits(h0.x >> 16);
          const float d1 = h2f_bits(h1.x & 0xffffu), dm1 = h2f_bits(h1.x >> 16);
          const float yl = __uint_as_float(lds32(d_s + 4 * b)), yh = __uint_as_float(lds32(d_s + 8 * KC * 4 + 4 * b));
          facc[0] += (d0 * yl) * (float)S4[0] - (dm0 * yl) * (float)T4[0];
          facc[1] += (d1 * yl) * (float)S4[1] - (dm1 * yl) * (float)T4[1];
          facc[2] += (d0 * yh) * (float)S4[2] - (dm0 * yh) * (float)T4[2];
          facc[3] += (d1 * yh) * (float)S4[3] - (dm1 * yh) * (float)T4[3];
        }
      }
      // partial sums of the warps sharing this tile meet in shared memory; k-part 0 adds them in order
      float* my = part + ((size_t)tile * ksplit + kpart) * 128;
      if (ksplit > 1) {
        if (kpart != 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) my[4 * lane + i] = facc[i];
        }
        // tile barrier (ids 1..4), ksplit warps
        asm volatile("bar.sync %0, %1;" ::"r"(1 + tile), "r"(32 * ksplit) : "memory");
        if (kpart == 0) {
          for (int kp = 1; kp < ksplit; ++kp) {
#pragma unroll
            for (int i = 0; i < 4; ++i) facc[i] += my[(size_t)kp * 128 + 4 * lane + i];
          }
        }
      }
      if (!dead && kpart == 0 && tile * 8 < rows_here) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = gid + 8 * (i >> 1), col = tile * 8 + 2 * tig + (i & 1);
          if (m < ac && col < rows_here) {
            const int srow = a0 + m;
            const int orow = p.out_rows ? p.out_rows[srow] : srow;
            float* dst = p.y + (size_t)orow * p.n + row0 + col;
            *dst = kc == 0 ? facc[i] : *dst + facc[i];  // later sweeps add, in order, by the same thread
          }
        }
      }
      if (ksplit > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + tile), "r"(32 * ksplit) : "memory");  // partials consumed
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->empty[s]);
    }
   }
  }
}

}  // namespace fq
