// Mixture-of-experts block on the quantized decode path: router, bucketing of (token, slot) pairs by
// expert, gather + activation quantization, the grouped (indexed) quantized mat-vec, and the combine.
//
// What it computes is the reference's sparse MoE forward (fuel-core/src/lazy_nn/moe.rs:92-127 router,
// :296-348 layer): top-K by K rounds of first-maximum argmax with the picked logit pushed down by
// 1e30, softmax over the picked logits (max-subtracted, sequential sum, multiply by the reciprocal:
// fuel-cpu-backend/src/byte_kernels.rs:2259-2305), then for every expert in ascending id the rows of
// the tokens routed to it (ascending token order) go through that expert's FFN and are added back to
// the token scaled by its gate weight - so a token's result is ((0 + w_a*y_a) + w_b*y_b) + ... with
// its experts a < b < ... in ascending id. The expert matrices are GGUF-quantized here (the reference
// keeps experts in f32 and names the grouped quantized kernel as missing:
// fuel-cuda-backend/src/quantized.rs:292-304), and each expert mat-vec is the same integer dot
// product as the plain decode path, on activations re-quantized to Q8_K row by row.
//
// The grouped mat-vec streams each expert's matrix ONCE (skipping experts nobody routed to) through
// the same bulk-copy ring as the decode kernel and applies it to all of that expert's rows.
#pragma once
#include "decode.cuh"
#include "fq_common.cuh"
#include "quantize_act.cuh"

namespace fq {

constexpr float kMoeMaskNeg = -1.0e30f;  // fuel-core/src/lazy_nn/moe.rs:28
constexpr int kMoeMaxTopK = 16;

// ---- router: one warp per token, n_experts <= 1024 -------------------------------------------
__global__ void __launch_bounds__(256) moe_route_kernel(const float* logits, int n_tokens, int n_experts, int top_k,
                                                        int* topk_ids, float* topk_w) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  float v[32];  // this lane's logits: experts lane, lane + 32, ...
  const int per = (n_experts + 31) >> 5;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int e = lane + 32 * j;
    v[j] = (j < per && e < n_experts) ? logits[(size_t)t * n_experts + e] : -INFINITY;
  }
  float picked[kMoeMaxTopK];
  for (int r = 0; r < top_k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < per) {
        const int e = lane + 32 * j;
        if (e < n_experts && (v[j] > bv || (v[j] == bv && e < bi))) bv = v[j], bi = e;  // first maximum wins
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
    }
    picked[r] = bv;
    if (lane == 0) topk_ids[(size_t)t * top_k + r] = bi;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < per && lane + 32 * j == bi) v[j] = __fadd_rn(v[j], kMoeMaskNeg);  // scatter_add of the mask value
  }
  if (lane == 0) {
    float mx = picked[0];
    for (int r = 1; r < top_k; ++r)
      if (picked[r] > mx) mx = picked[r];
    float sum = 0.f;
    for (int r = 0; r < top_k; ++r) {
      picked[r] = expf(picked[r] - mx);
      sum = __fadd_rn(sum, picked[r]);
    }
    const float inv = 1.0f / sum;
    for (int r = 0; r < top_k; ++r) topk_w[(size_t)t * top_k + r] = __fmul_rn(picked[r], inv);
  }
}

// ---- bucketing: pairs (token * top_k + slot) sorted by expert, ascending pair id inside an expert.
// One CTA; the pair list is read into shared memory once (when it fits), then every warp scans it with
// ballots for up to kBucketPerWarp experts at a time, so the order never depends on timing.
constexpr int kBucketPerWarp = 4;

__global__ void __launch_bounds__(1024) moe_bucket_kernel(const int* topk_ids, int n_pairs, int n_experts, int* sorted_ids,
                                                          int* offsets, int in_smem) {
  extern __shared__ int bsm[];  // counts [n_experts + 1], then the pair list if it fits
  int* counts = bsm;
  int* ids_s = bsm + n_experts + 1;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (in_smem)
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) ids_s[p] = topk_ids[p];
  __syncthreads();
  const int* ids = in_smem ? ids_s : topk_ids;
  // pass 1: counts
  for (int e0 = warp * kBucketPerWarp; e0 < n_experts; e0 += nwarps * kBucketPerWarp) {
    int c[kBucketPerWarp];
#pragma unroll
    for (int i = 0; i < kBucketPerWarp; ++i) c[i] = 0;
    for (int p0 = 0; p0 < n_pairs; p0 += 32) {
      const int p = p0 + lane;
      const int id = p < n_pairs ? ids[p] : -1;
#pragma unroll
      for (int i = 0; i < kBucketPerWarp; ++i) c[i] += __popc(__ballot_sync(0xffffffffu, id == e0 + i));
    }
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < kBucketPerWarp; ++i)
        if (e0 + i < n_experts) counts[e0 + i] = c[i];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_experts; ++e) {
      const int c = counts[e];
      counts[e] = run;
      offsets[e] = run;
      run += c;
    }
    counts[n_experts] = run;
    offsets[n_experts] = run;
  }
  __syncthreads();
  // pass 2: positions
  for (int e0 = warp * kBucketPerWarp; e0 < n_experts; e0 += nwarps * kBucketPerWarp) {
    int pos[kBucketPerWarp];
#pragma unroll
    for (int i = 0; i < kBucketPerWarp; ++i) pos[i] = (e0 + i < n_experts) ? counts[e0 + i] : 0;
    for (int p0 = 0; p0 < n_pairs; p0 += 32) {
      const int p = p0 + lane;
      const int id = p < n_pairs ? ids[p] : -1;
#pragma unroll
      for (int i = 0; i < kBucketPerWarp; ++i) {
        const bool hit = id == e0 + i;
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        if (hit) sorted_ids[pos[i] + __popc(bal & ((1u << lane) - 1u))] = p;
        pos[i] += __popc(bal);
      }
    }
  }
}

// The same result in O(pairs) work when a table of per-chunk counts fits shared memory (a chunk = 32 consecutive
// pairs, one warp pass): a pair's place inside its expert is (pairs of that expert in earlier chunks) + (matching
// lanes below it in its own chunk), both independent of timing. One CTA.
__global__ void __launch_bounds__(1024) moe_bucket_chunks_kernel(const int* topk_ids, int n_pairs, int n_experts,
                                                                 int* sorted_ids, int* offsets) {
  extern __shared__ int bsm[];  // cnt [n_chunks][n_experts], then start [n_experts + 1]
  const int n_chunks = (n_pairs + 31) >> 5;
  int* cnt = bsm;
  int* start = bsm + n_chunks * n_experts;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < n_chunks * n_experts; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int c = warp; c < n_chunks; c += nwarps) {
    const int p = 32 * c + lane;
    int id = p < n_pairs ? topk_ids[p] : -1;
    if (id < 0 || id >= n_experts) id = -1;
    const unsigned same = __match_any_sync(0xffffffffu, id);
    if (id >= 0 && lane == __ffs(same) - 1) cnt[c * n_experts + id] = __popc(same);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {  // per expert: counts -> pairs in earlier chunks
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int t = cnt[c * n_experts + e];
      cnt[c * n_experts + e] = run;
      run += t;
    }
    start[e] = run;
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the per-expert totals: a contiguous segment per lane, then across lanes
    const int seg = (n_experts + 31) >> 5, e0 = lane * seg, e1 = min(e0 + seg, n_experts);
    int sum = 0;
    for (int e = e0; e < e1; ++e) sum += start[e];
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    int run = incl - sum;
    for (int e = e0; e < e1; ++e) {
      const int t = start[e];
      start[e] = run;
      offsets[e] = run;
      run += t;
    }
    if (lane == 31) start[n_experts] = incl, offsets[n_experts] = incl;
  }
  __syncthreads();
  for (int c = warp; c < n_chunks; c += nwarps) {
    const int p = 32 * c + lane;
    int id = p < n_pairs ? topk_ids[p] : -1;
    if (id < 0 || id >= n_experts) id = -1;
    const unsigned same = __match_any_sync(0xffffffffu, id);
    if (id >= 0) sorted_ids[start[id] + cnt[c * n_experts + id] + __popc(same & ((1u << lane) - 1u))] = p;
  }
}

// ---- gather + Q8_K quantization: sorted row i <- x[row_ids[i] / divisor] (k a multiple of 256)
__global__ void __launch_bounds__(256) moe_gather_quantize_kernel(const float* x, int k, const int* row_ids, int divisor,
                                                                  int64_t n_blocks, int8_t* out_qs, float* out_d,
                                                                  int16_t* out_bsums) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (blk >= n_blocks) return;
  const int bpr = k >> 8;
  const int64_t row = blk / bpr;
  const int b = (int)(blk - row * bpr);
  const int src_row = row_ids[row] / divisor;
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)src_row * k + b * 256);
  const float4 v0 = src[lane], v1 = src[32 + lane];
  const float e[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  q8k_block_from_regs(e, lane, blk, out_qs, out_d, out_bsums);
}

// ---- silu(gate) * up over rows [gate | up] of width 2f (f a multiple of 256), quantized to Q8_K
__global__ void __launch_bounds__(256) moe_swiglu_quantize_kernel(const float* gu, int f, int64_t n_blocks, int8_t* out_qs,
                                                                  float* out_d, int16_t* out_bsums) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (blk >= n_blocks) return;
  const int bpr = f >> 8;
  const int64_t row = blk / bpr;
  const int b = (int)(blk - row * bpr);
  const float4* gp = reinterpret_cast<const float4*>(gu + (size_t)row * 2 * f + b * 256);
  const float4* up = reinterpret_cast<const float4*>(gu + (size_t)row * 2 * f + f + b * 256);
  const float4 a0 = gp[lane], a1 = gp[32 + lane], b0 = up[lane], b1 = up[32 + lane];
  const float g[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  const float u[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  float e[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
  q8k_block_from_regs(e, lane, blk, out_qs, out_d, out_bsums);
}

// ---- grouped mat-vec: y[out_row(i), :] = W[e] . act[i] for the sorted rows i of every expert e
struct MoeParams {
  const uint8_t* w;      // [n_experts][n][k] blocks
  ActPlanes act;         // activation planes of all sorted rows
  const int* offsets;    // [n_experts + 1] sorted-row ranges
  const int* out_rows;   // sorted row -> output row, or null for the identity
  float* y;              // [rows][n]
  int64_t expert_bytes;  // n * row_bytes
  int n, k, row_bytes, units_per_row, rows_per_stage, num_stages, stage_stride;
  int act_rows;          // activation rows held in shared memory per pass over the weights
  int act_smem_off;      // where they live
};

struct MoeSmemHeader {
  uint64_t full[kDecodeMaxStages];
  uint64_t empty[kDecodeMaxStages];
};

constexpr int kMoeMT = 8;  // activation rows per sweep of a weight row

// An expert's activation rows are used by every one of its weight rows, so they are copied into shared
// memory (up to act_rows at a time) and the CTA's weight rows are streamed through the ring once per such
// group of rows - once in all for the usual handful of rows per expert; later passes hit L2.
template <class Fmt>
__global__ void __launch_bounds__(kDecodeThreads, 2) moe_decode_kernel(const MoeParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  MoeSmemHeader* hd = reinterpret_cast<MoeSmemHeader*>(smem_raw);
  uint8_t* stages = smem_raw + align_up(sizeof(MoeSmemHeader), 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.num_stages, R = p.rows_per_stage;
  const int e = blockIdx.y;
  const int r_begin = (int)((int64_t)p.n * blockIdx.x / gridDim.x);
  const int r_end = (int)((int64_t)p.n * (blockIdx.x + 1) / gridDim.x);
  const int n_iter = (r_end - r_begin + R - 1) / R;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&hd->full[s], 1);
      mbar_init(&hd->empty[s], kDecodeConsumerWarps);
    }
    mbar_init_fence();
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();  // the row ranges come from the bucketing kernel: nothing is streamed for an expert without rows
  const int m_begin = p.offsets[e], m_count = p.offsets[e + 1] - m_begin;
  if (m_count <= 0) return;
  const int n_pass = (m_count + p.act_rows - 1) / p.act_rows;
  const int total_iter = n_pass * n_iter;
  const int64_t base = (int64_t)e * p.expert_bytes;

  if (warp == kDecodeConsumerWarps) {
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      int it = 0;  // stage of rows within the pass
      for (int g = 0; g < total_iter && ok; ++g) {
        const int s = g % S;
        if (g >= S) {
          ok = mbar_wait_bounded(&hd->empty[s], ((g / S) - 1) & 1);
          if (!ok) {
            record_dev_error(kErrEmptyWait);
            break;
          }
        }
        const int row0 = r_begin + it * R;
        const int row1 = (row0 + R < r_end) ? row0 + R : r_end;
        // expert matrices start on 16-byte boundaries and rows are multiples of 16 bytes (checked by the host)
        const int64_t b0 = base + (int64_t)row0 * p.row_bytes, b1 = base + (int64_t)row1 * p.row_bytes;
        mbar_arrive_expect_tx(&hd->full[s], (uint32_t)(b1 - b0));
        bulk_g2s(stages + (size_t)s * p.stage_stride, p.w + b0, (uint32_t)(b1 - b0), &hd->full[s]);
        issued = g + 1;
        if (++it == n_iter) it = 0;
      }
      if (!ok) {
        for (int g = (issued > S ? issued - S : 0); g < issued; ++g)
          if (!mbar_wait_bounded(&hd->full[g % S], (g / S) & 1)) record_dev_error(kErrDrainWait);
      }
    }
    return;
  }

  // ---------------- consumers
  const ActPlanes sp = act_planes(smem_raw + p.act_smem_off, kQ4K, p.act_rows, p.k);
  const int t = threadIdx.x, nt = 32 * kDecodeConsumerWarps;
  const int dpr = p.k >> 8, bpr = p.k >> 4;  // block scales / 16-sums per row
  int g = 0;
  for (int pass = 0; pass < n_pass; ++pass) {
    const int a0 = m_begin + pass * p.act_rows;
    const int ac = (m_count - pass * p.act_rows < p.act_rows) ? m_count - pass * p.act_rows : p.act_rows;
    if (pass > 0) asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecodeConsumerWarps) : "memory");  // previous rows are done with
    {
      const uint4* src = reinterpret_cast<const uint4*>(p.act.qs + (size_t)a0 * p.k);
      uint4* dst = reinterpret_cast<uint4*>(const_cast<int8_t*>(sp.qs));
      for (int i = t; i < ac * (p.k >> 4); i += nt) dst[i] = src[i];
      const float* sd = p.act.d + (size_t)a0 * dpr;
      float* dd = const_cast<float*>(sp.d);
      for (int i = t; i < ac * dpr; i += nt) dd[i] = sd[i];
      const uint4* sb = reinterpret_cast<const uint4*>(p.act.bsums + (size_t)a0 * bpr);
      uint4* db = reinterpret_cast<uint4*>(const_cast<int16_t*>(sp.bsums));
      for (int i = t; i < ac * (bpr >> 3); i += nt) db[i] = sb[i];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecodeConsumerWarps) : "memory");
    for (int it = 0; it < n_iter; ++it, ++g) {
      const int s = g % S;
      if (!mbar_wait_bounded(&hd->full[s], (g / S) & 1)) {
        record_dev_error(kErrFullWait);
        return;
      }
      const int row0 = r_begin + it * R;
      const int rows_here = ((row0 + R < r_end) ? row0 + R : r_end) - row0;
      const uint8_t* sbase = stages + (size_t)s * p.stage_stride;
      for (int r = warp; r < rows_here; r += kDecodeConsumerWarps) {
        const uint8_t* rowp = sbase + (size_t)r * p.row_bytes;
        for (int m0 = 0; m0 < ac; m0 += kMoeMT) {
          const int mc = (ac - m0 < kMoeMT) ? ac - m0 : kMoeMT;
          float acc[kMoeMT];
#pragma unroll
          for (int i = 0; i < kMoeMT; ++i) acc[i] = 0.f;
          for (int u = lane; u < p.units_per_row; u += 32) Fmt::template unit<kMoeMT>(rowp, u, sp, p.k, m0, mc, acc);
#pragma unroll
          for (int i = 0; i < kMoeMT; ++i) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
          }
          if (lane == 0) {
#pragma unroll
            for (int i = 0; i < kMoeMT; ++i) {
              if (i < mc) {
                const int srow = a0 + m0 + i;
                const int orow = p.out_rows ? p.out_rows[srow] : srow;
                p.y[(size_t)orow * p.n + row0 + r] = acc[i];
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hd->empty[s]);
    }
  }
}

// ---- expert parallelism with fixed-capacity chunks. A (source, destination) pair of ranks owns a chunk of
// capacity + 1 rows of `hidden` floats: the rows for that destination, sorted by expert, then one row that holds
// their expert ids as int32 (-1 = unused slot). Sorted position s of this rank's pairs belongs to rank
// q = (the rank whose experts contain it) at place j = s - offsets[q * experts_per_rank].
__device__ __forceinline__ int moe_ep_dest(const int* offsets, int experts_per_rank, int world, int s, int* first) {
  int q = 0;
  while (q + 1 < world && offsets[(q + 1) * experts_per_rank] <= s) ++q;
  *first = offsets[q * experts_per_rank];
  return q;
}
// grid = n_pairs + world blocks: block s < n_pairs copies the row of sorted position s into its slot and writes its
// expert id; block n_pairs + q marks the unused slots of chunk q
__global__ void __launch_bounds__(128) moe_ep_pack_kernel(const float* x, int hidden, const int* sorted_ids, const int* offsets,
                                                          const int* topk_ids, int top_k, int n_pairs, int experts_per_rank,
                                                          int world, int capacity, float* send) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t chunk = (size_t)(capacity + 1) * hidden;
  if ((int)blockIdx.x >= n_pairs) {
    const int q = blockIdx.x - n_pairs;
    const int used = offsets[(q + 1) * experts_per_rank] - offsets[q * experts_per_rank];
    int* ids = reinterpret_cast<int*>(send + q * chunk + (size_t)capacity * hidden);
    for (int j = used + threadIdx.x; j < capacity; j += blockDim.x) ids[j] = -1;
    return;
  }
  const int s = blockIdx.x;
  int first;
  const int q = moe_ep_dest(offsets, experts_per_rank, world, s, &first);
  const int j = s - first, pair = sorted_ids[s];
  const float4* src = reinterpret_cast<const float4*>(x + (size_t)(pair / top_k) * hidden);
  float4* dst = reinterpret_cast<float4*>(send + q * chunk + (size_t)j * hidden);
  for (int c = threadIdx.x; c < (hidden >> 2); c += blockDim.x) dst[c] = src[c];
  if (threadIdx.x == 0) reinterpret_cast<int*>(send + q * chunk + (size_t)capacity * hidden)[j] = topk_ids[pair];
}
// received chunks -> one local expert id per slot (id rows and unused slots: -1)
__global__ void __launch_bounds__(256) moe_ep_local_ids_kernel(const float* recv, int hidden, int capacity, int world,
                                                               int first_expert, int* local_ids) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x, per = capacity + 1;
  if (i >= world * per) return;
  const int q = i / per, j = i - q * per;
  int id = -1;
  if (j < capacity) id = reinterpret_cast<const int*>(recv + ((size_t)q * per + capacity) * hidden)[j];
  local_ids[i] = id >= 0 ? id - first_expert : -1;
}
// returned chunks -> y_pairs in pair order: one block per sorted position
__global__ void __launch_bounds__(128) moe_ep_unpack_kernel(const float* y_back, int hidden, const int* sorted_ids,
                                                            const int* offsets, int n_pairs, int experts_per_rank, int world,
                                                            int capacity, float* y_pairs) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  if (s >= n_pairs) return;
  int first;
  const int q = moe_ep_dest(offsets, experts_per_rank, world, s, &first);
  const float4* src = reinterpret_cast<const float4*>(y_back + ((size_t)q * (capacity + 1) + (s - first)) * hidden);
  float4* dst = reinterpret_cast<float4*>(y_pairs + (size_t)sorted_ids[s] * hidden);
  for (int c = threadIdx.x; c < (hidden >> 2); c += blockDim.x) dst[c] = src[c];
}

// ---- combine: out[t] = ((0 + w*y of the lowest expert id) + next ...) over the token's top_k pairs
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* y_pairs, const int* topk_ids, const float* topk_w,
                                                          int top_k, int n, float* out) {
  __shared__ int ord_s[kMoeMaxTopK];
  __shared__ float w_s[kMoeMaxTopK];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int ord[kMoeMaxTopK];
    for (int s = 0; s < top_k; ++s) ord[s] = s;
    for (int a = 1; a < top_k; ++a) {  // insertion sort of the slots by expert id (ids are distinct)
      const int sa = ord[a], ea = topk_ids[(size_t)t * top_k + sa];
      int b = a - 1;
      while (b >= 0 && topk_ids[(size_t)t * top_k + ord[b]] > ea) {
        ord[b + 1] = ord[b];
        --b;
      }
      ord[b + 1] = sa;
    }
    for (int s = 0; s < top_k; ++s) ord_s[s] = ord[s], w_s[s] = topk_w[(size_t)t * top_k + ord[s]];
  }
  __syncthreads();
  const float* base = y_pairs + (size_t)t * top_k * n;
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(y_pairs) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    for (int c = threadIdx.x; c < (n >> 2); c += blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < top_k; ++s) {
        const float4 v = reinterpret_cast<const float4*>(base + (size_t)ord_s[s] * n)[c];
        const float w = w_s[s];
        acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, w));  // scale, then add: two roundings
        acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, w));
        acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, w));
        acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, w));
      }
      reinterpret_cast<float4*>(out + (size_t)t * n)[c] = acc;
    }
    return;
  }
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < top_k; ++s) acc = __fadd_rn(acc, __fmul_rn(base[(size_t)ord_s[s] * n + c], w_s[s]));
    out[(size_t)t * n + c] = acc;
  }
}

}  // namespace fq
