// Tensor-core GEMM on weights that are already in the operand type: Y[M, N] = X[M, K] . W[N, K]^T with W a slab of rows
// dequantized by the stand-alone kernels (dequantize.cuh: GgmlType::to_float arithmetic, fuel-quantized/src/k_quants.rs)
// into f16, bf16 or tf32-rounded f32, and X the activations converted by the pre-pass of prefill.cuh. The reference has
// no such path (its CUDA forward runs the mat-vec kernel for every M, fuel-cuda-backend/src/quantized.rs:452-473; its
// Vulkan path dequantizes the whole matrix to f32 and calls a float matmul, fuel-vulkan-backend/src/lib.rs:4221-4283).
//
// A persistent kernel, one thread block per SM, three roles:
//   warp 0, one lane   both operand tiles of every 128-byte-wide K stage by tensor-map (TMA) copies with the 128-byte
//                      swizzle, into a ring of shared-memory stages that runs on across output tiles;
//   warp 1, one lane   tcgen05.mma on each landed stage, accumulating a 128 (weight rows) x kTileM (activation rows) tile
//                      in tensor memory; two accumulators, so the next tile's products start while
//   warps 2-5          read the finished accumulator out of tensor memory and store Y (the f16 form undoes the
//                      activation rows' power-of-two scaling here).
// Work items are the 128 x kTileM output tiles in an order that keeps the thread blocks of one round on the same few weight
// rows (M fastest). When the tiles do not fill a last round of thread blocks, the tiles of that round are cut along M into
// 2 or 4 pieces (same loads, narrower MMAs), so the round takes a half or a quarter of a tile's time instead of a
// whole one. Every wait is bounded; on expiry the block raises an abort flag, lets its copies land, frees its tensor
// memory and returns.
#pragma once
#include "prefill.cuh"

namespace fq {

constexpr int kPgThreads = 192;
constexpr int kPgEpilogueWarps = 4;

struct PlainGemmParams {
  float* y[8];               // destinations: y[q] is an [M][ldy] matrix (this GPU's, or a peer's mapped here)
  int n_dst;
  int ldy;
  int n_off;                 // first column this launch produces within a destination row
  int M, N, K;
  const float* row_unscale;  // f16 operands: factor per activation row that undoes the row's scaling (else null)
  int tiles_m;               // output tiles along M; tile t covers weight rows 128 * (t / tiles_m), activation rows kTileM * (t % tiles_m)
  int whole_tiles;           // tiles [0, whole_tiles) are work items of their own
  int split_log2;            // each later tile is 1 << split_log2 items, one per piece of kTileM >> split_log2 activation rows
  int n_items;
};

template <int kTileM, int kStages>
struct PlainGemmSmem {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct PgItem {
  int n0, m0;    // first weight row, first activation row of the TILE (what is loaded)
  int col, width;  // the piece: activation rows m0 + col .. m0 + col + width of it (what is multiplied and stored)
};
__device__ __forceinline__ PgItem pg_item(const PlainGemmParams& p, int i, int tile_m) {
  int tile, col = 0, width = tile_m;
  if (i < p.whole_tiles) {
    tile = i;
  } else {
    const int j = i - p.whole_tiles;
    tile = p.whole_tiles + (j >> p.split_log2);
    width = tile_m >> p.split_log2;
    col = (j & ((1 << p.split_log2) - 1)) * width;
  }
  const int tn = tile / p.tiles_m, tm = tile - tn * p.tiles_m;
  // activation rows past M need no products: narrow the piece to the next multiple of 32 rows (possibly to nothing)
  const int left = p.M - (tm * tile_m + col);
  if (left < width) width = left <= 0 ? 0 : (left + 31) & ~31;
  return PgItem{tn * kPfTileN, tm * tile_m, col, width};
}

template <int kTileM, int kStages, bool kTf32, bool kF16, bool kMulti>
__global__ void __launch_bounds__(kPgThreads, 1) plain_gemm_kernel(const PlainGemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                                   const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(1024) uint8_t pg_smem[];
  constexpr int kWBytes = kPfTileN * 128, kXBytes = kTileM * 128, kStageBytes = kWBytes + kXBytes;
  constexpr int kTbufBytes = kPgEpilogueWarps * 32 * 36 * 4;
  using Ctl = PlainGemmSmem<kTileM, kStages>;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pg_smem) + 1023) & ~(uintptr_t)1023);
  float* tbuf_all = reinterpret_cast<float*>(base + kStages * kStageBytes);
  Ctl* sm = reinterpret_cast<Ctl*>(base + kStages * kStageBytes + kTbufBytes);
  const uint32_t base_u32 = smem_u32(base);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kStageK = kTf32 ? 32 : kPfTileK;  // elements per 128-byte row
  const int n_iter = p.K / kStageK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm->full[s], 1);   // the copying thread (plus the bytes of both tiles)
      mbar_init(&sm->empty[s], 1);  // one commit from the MMA thread
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm->acc_full[b], 1);                  // one commit from the MMA thread
      mbar_init(&sm->acc_empty[b], kPgEpilogueWarps);  // one arrival per epilogue warp
    }
    sm->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&sm->tmem_base, 2 * kTileM);  // two f32 accumulators of kTileM columns x 128 lanes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *reinterpret_cast<volatile uint32_t*>(&sm->tmem_base);
  volatile int* abort_flag = &sm->abort_flag;

  if (warp == 0) {
    // ---------------- copies
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      for (int i = blockIdx.x; i < p.n_items && !*abort_flag; i += gridDim.x) {
        const PgItem w = pg_item(p, i, kTileM);
        if (w.width == 0) continue;  // every role skips the same items
        for (int it = 0; it < n_iter && !*abort_flag; ++it) {
          if (issued >= kStages && !mbar_wait_bounded(&sm->empty[s], ph ^ 1u)) {
            record_dev_error(kErrEmptyWait);
            *abort_flag = 1;
            break;
          }
          mbar_arrive_expect_tx(&sm->full[s], (uint32_t)kStageBytes);
          tma_load_2d(base_u32 + s * kStageBytes, &wmap, it * kStageK, w.n0, &sm->full[s]);
          tma_load_2d(base_u32 + s * kStageBytes + kWBytes, &xmap, it * kStageK, w.m0, &sm->full[s]);
          ++issued;
          if (++s == kStages) s = 0, ph ^= 1u;
        }
      }
      if (*abort_flag) {  // leaving early: let the copies already issued land first
        for (int g = (issued > kStages ? issued - kStages : 0); g < issued; ++g)
          if (!mbar_wait_bounded(&sm->full[g % kStages], (g / kStages) & 1)) record_dev_error(kErrDrainWait);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue: one thread
    if (lane == 0) {
      int s = 0, li = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < p.n_items && ok; i += gridDim.x) {
        const PgItem w = pg_item(p, i, kTileM);
        if (w.width == 0) continue;
        const int b = li & 1;
        // the accumulator's previous contents (two items ago) must have been read out
        if (li >= 2 && (*abort_flag || !mbar_wait_bounded(&sm->acc_empty[b], ((li >> 1) & 1) ^ 1u))) {
          if (!*abort_flag) record_dev_error(kErrTmemWait);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t idesc = kTf32 ? umma_idesc_tf32(kPfTileN, w.width) : kF16 ? umma_idesc_f16(kPfTileN, w.width) : umma_idesc_bf16(kPfTileN, w.width);
        const uint32_t acc = tmem_d + (uint32_t)(b * kTileM);
        for (int it = 0; it < n_iter; ++it) {
          if (*abort_flag || !mbar_wait_bounded(&sm->full[s], ph)) {
            if (!*abort_flag) record_dev_error(kErrFullWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = base_u32 + s * kStageBytes, b_addr = a_addr + kWBytes + (uint32_t)w.col * 128u;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // 32 bytes along K per instruction: 16 16-bit values or 8 tf32
            if constexpr (kTf32)
              umma_tf32(acc, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc, (it | kk) != 0);
            else
              umma_bf16(acc, umma_desc_sw128(a_addr + kk * 32), umma_desc_sw128(b_addr + kk * 32), idesc, (it | kk) != 0);
          }
          umma_commit(&sm->empty[s]);  // frees the stage once these MMAs have read it
          if (++s == kStages) s = 0, ph ^= 1u;
        }
        if (ok) umma_commit(&sm->acc_full[b]);  // accumulator complete
        ++li;
      }
    }
  } else {
    // ---------------- epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 (weight rows) and stores Y
    const int q = warp & 3;
    float* tbuf = tbuf_all + (warp - 2) * (32 * 36);  // [32 m][36]: rows 16-byte aligned, shifted banks
    int li = 0;
    for (int i = blockIdx.x; i < p.n_items; i += gridDim.x) {
      const PgItem w = pg_item(p, i, kTileM);
      if (w.width == 0) continue;
      const int b = li & 1;
      bool ready = !*abort_flag;
      if (ready && !mbar_wait_bounded(&sm->acc_full[b], (li >> 1) & 1)) {
        record_dev_error(kErrMmaWait);
        *abort_flag = 1;
        ready = false;
      }
      ready = __all_sync(0xffffffffu, ready);
      if (!ready) break;
      tc_fence_after();
      const int nrow = w.n0 + q * 32;  // first weight row (output column) of this warp
      const int n = nrow + lane;
      // The accumulator arrives one weight row (output column) per lane; Y is row-major in the other direction. For
      // several destinations each warp turns 32 x 32 pieces around in shared memory so that it stores 16 bytes per lane
      // along a row of Y - four times fewer, four times larger stores, which matters most for the peers' copies.
      bool vec_ok = kMulti && p.n_dst > 1 && (p.ldy & 3) == 0 && (p.n_off & 3) == 0 && nrow + 32 <= p.N;
#pragma unroll
      for (int d = 0; d < 8; ++d)
        if (d < p.n_dst) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(p.y[d]) & 15) == 0;
      const int sub_m = lane >> 3, n4 = (lane & 7) * 4;
      const int chunks = w.width >> 5;
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * kTileM + c * 32), v);
        const int mbase = w.m0 + w.col + c * 32;
        if constexpr (kF16) {  // undo the scaling of activation row mbase + j (a power of two: exact)
          const int ml = mbase + lane;
          const float mine = ml < p.M ? p.row_unscale[ml] : 1.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * __shfl_sync(0xffffffffu, mine, j));
        }
        if (kMulti && vec_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) tbuf[j * 36 + lane] = __uint_as_float(v[j]);
          __syncwarp();
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            const int mm = sub_m + 4 * r, m = mbase + mm;
            if (m < p.M) {
              const float4 val = *reinterpret_cast<const float4*>(tbuf + mm * 36 + n4);
              // column-sharded across GPUs: the piece goes straight into every GPU's copy of Y (plain stores over
              // NVLink for the peers'), so the all-gather of the shards happens inside the epilogue
              const size_t off = (size_t)m * p.ldy + p.n_off + nrow + n4;
#pragma unroll
              for (int d = 0; d < 8; ++d)  // constant indices: a runtime index would copy the pointer table to local memory
                if (d < p.n_dst) *reinterpret_cast<float4*>(p.y[d] + off) = val;
            }
          }
          __syncwarp();
        } else if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = mbase + j;
            if (m < p.M) {
              const size_t off = (size_t)m * p.ldy + p.n_off + n;
              p.y[0][off] = __uint_as_float(v[j]);
              if (kMulti && p.n_dst > 1) {
#pragma unroll
                for (int d = 1; d < 8; ++d)
                  if (d < p.n_dst) p.y[d][off] = __uint_as_float(v[j]);
              }
            }
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->acc_empty[b]);
      ++li;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, 2 * kTileM);
}

}  // namespace fq
