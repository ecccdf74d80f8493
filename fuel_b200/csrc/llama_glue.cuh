// f32 glue around the quantized mat-vecs of a LLaMA-style decode step, batch 1: what the reference's
// model code runs between its seven quantized linears per layer (fuel-core/src/lazy.rs:7363-7447):
//   RMSNorm with gain     x * 1/sqrt(mean(x^2) + eps) * g      fuel-cpu-backend/src/byte_kernels.rs:2339-2367
//   rotate-half RoPE      lo' = lo*cos - hi*sin, hi' = hi*cos + lo*sin   byte_kernels.rs:1885-1960
//   attention, one query  softmax(q.K^T * scale) . V, max-subtracted softmax   byte_kernels.rs:2259-2305
//   SwiGLU                silu(gate) * up
//   greedy pick           the LAST index holding the maximum (max_by + total_cmp,
//                         fuel-transformers/src/generation/mod.rs:84-93)
// These are callers of the hot path, not the hot path; they are written plainly, with fixed
// reduction orders so a value never depends on how many GPUs share the model.
#pragma once
#include "fq_common.cuh"
#include "peer.cuh"
#include "quantize_act.cuh"

namespace fq {

// No pointer parameter in this file is __restrict__: under programmatic dependent launch these kernels start
// while their predecessor is still writing their inputs, and a read-only-for-the-kernel's-lifetime promise
// would let the compiler move such loads above the dependency wait.

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];  // fixed order
  return t;
}

// token ids -> rows of an f32 embedding table (k a multiple of 4)
__global__ void __launch_bounds__(256) embed_f32_kernel(const float* table, int k, const int* ids, float* out) {
  pdl_launch_dependents();
  pdl_wait();
  const float4* row = reinterpret_cast<const float4*>(table + (size_t)ids[blockIdx.x] * k);
  float4* o = reinterpret_cast<float4*>(out + (size_t)blockIdx.x * k);
  for (int i = threadIdx.x; i < (k >> 2); i += blockDim.x) o[i] = row[i];
}

// token ids -> dequantized Q4_K rows of the embedding table (one CTA per id, 16 threads per super-block)
__global__ void __launch_bounds__(256) embed_q4k_kernel(const uint8_t* table, int row_bytes, int k,
                                                        const int* ids, float* out) {
  pdl_launch_dependents();
  pdl_wait();
  const uint8_t* row = table + (size_t)ids[blockIdx.x] * row_bytes;
  float* o = out + (size_t)blockIdx.x * k;
  for (int u = threadIdx.x; u < (k >> 8) * 8; u += blockDim.x) {  // 16-byte nibble chunks, as dequant_q4k_kernel
    const int blk = u >> 3, cc = u & 7, g = cc >> 1, h = cc & 1;
    const uint8_t* b = row + blk * Q4KL::kBytes;
    const uint4 hdr = *reinterpret_cast<const uint4*>(b);
    const uint4 qv = *reinterpret_cast<const uint4*>(b + Q4KL::kOffQs + 16 * cc);
    const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
    uint32_t scw, mnw;
    if (g < 2) {
      scw = hdr.y & 0x3f3f3f3fu;
      mnw = hdr.z & 0x3f3f3f3fu;
    } else {
      scw = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
      mnw = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
    }
    const int sh = (g & 1) * 16;
    const float d1 = __fmul_rn(d, (float)((scw >> sh) & 0xff)), m1 = __fmul_rn(dmin, (float)((mnw >> sh) & 0xff));
    const float d2 = __fmul_rn(d, (float)((scw >> (sh + 8)) & 0xff)), m2 = __fmul_rn(dmin, (float)((mnw >> (sh + 8)) & 0xff));
    float* dst = o + blk * 256 + 64 * g + 16 * h;
    const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const uint32_t byte = (qw[j] >> (8 * t)) & 0xff;
        dst[4 * j + t] = __fsub_rn(__fmul_rn(d1, (float)(byte & 0xF)), m1);
        dst[32 + 4 * j + t] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
      }
  }
}

// rotate q (n_heads) and k (n_kv) at position *pos, then append k and v to the caches
// caches: [n_kv][max_seq][hd]; cos/sin: [max_seq][hd] (both halves hold the same angles)
__global__ void __launch_bounds__(128) rope_store_kernel(float* q, const float* k,
                                                         const float* v, float* kc,
                                                         float* vc, const float* cosT,
                                                         const float* sinT, const int* pos_p,
                                                         int n_heads, int n_kv, int hd, int max_seq) {
  pdl_launch_dependents();
  pdl_wait();
  const int pos = *pos_p;
  const int head = blockIdx.x, half = hd >> 1;
  const float* cs = cosT + (size_t)pos * hd;
  const float* sn = sinT + (size_t)pos * hd;
  if (head < n_heads) {
    float* x = q + (size_t)head * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float lo = x[i], hi = x[i + half];
      x[i] = __fsub_rn(__fmul_rn(lo, cs[i]), __fmul_rn(hi, sn[i]));
      x[i + half] = __fadd_rn(__fmul_rn(hi, cs[i + half]), __fmul_rn(lo, sn[i + half]));
    }
  } else {
    const int kh = head - n_heads;
    const float* x = k + (size_t)kh * hd;
    float* kd = kc + ((size_t)kh * max_seq + pos) * hd;
    float* vd = vc + ((size_t)kh * max_seq + pos) * hd;
    const float* vs = v + (size_t)kh * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float lo = x[i], hi = x[i + half];
      kd[i] = __fsub_rn(__fmul_rn(lo, cs[i]), __fmul_rn(hi, sn[i]));
      kd[i + half] = __fadd_rn(__fmul_rn(hi, cs[i + half]), __fmul_rn(lo, sn[i + half]));
      vd[i] = vs[i];
      vd[i + half] = vs[i + half];
    }
  }
}

// one query per head against positions 0..*pos of the cache (GQA: head h reads kv head h / (n_heads / n_kv)),
// head_dim 128. The context is cut into kAttnSplits equal chunks, one CTA each (grid = heads x splits):
// a CTA computes its chunk's scores, their maximum, the exponentials' sum and the unnormalized
// weighted sum of V rows; attn_combine_kernel merges the chunks in a fixed order. The split count
// is a constant, so a value never depends on the launch configuration or on how many GPUs there are.
constexpr int kAttnSplits = 8;
constexpr int kAttnPartStride = 132;  // 128 outputs + max + sum (+ pad)

// Rotate-half RoPE of a 128-wide head held four elements per lane (lane l: elements 4l..4l+3; the partner
// element i +- 64 lives in lane l ^ 16). Same operations and roundings as rope_store_kernel.
__device__ __forceinline__ float4 rope128(float4 x, float4 cs, float4 sn, int lane) {
  float4 o;
  o.x = __shfl_xor_sync(0xffffffffu, x.x, 16), o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
  o.z = __shfl_xor_sync(0xffffffffu, x.z, 16), o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
  float4 r;
  if (lane < 16) {  // x[i] = lo * cos[i] - hi * sin[i]
    r.x = __fsub_rn(__fmul_rn(x.x, cs.x), __fmul_rn(o.x, sn.x)), r.y = __fsub_rn(__fmul_rn(x.y, cs.y), __fmul_rn(o.y, sn.y));
    r.z = __fsub_rn(__fmul_rn(x.z, cs.z), __fmul_rn(o.z, sn.z)), r.w = __fsub_rn(__fmul_rn(x.w, cs.w), __fmul_rn(o.w, sn.w));
  } else {          // x[i + 64] = hi * cos[i + 64] + lo * sin[i + 64]
    r.x = __fadd_rn(__fmul_rn(x.x, cs.x), __fmul_rn(o.x, sn.x)), r.y = __fadd_rn(__fmul_rn(x.y, cs.y), __fmul_rn(o.y, sn.y));
    r.z = __fadd_rn(__fmul_rn(x.z, cs.z), __fmul_rn(o.z, sn.z)), r.w = __fadd_rn(__fmul_rn(x.w, cs.w), __fmul_rn(o.w, sn.w));
  }
  return r;
}

// With `rope` set the kernel also does rope_store_kernel's work: q arrives unrotated and is rotated on the fly; the
// current token's k (rotated) and v come from `rope.k` / `rope.v` instead of the cache, and the first head of each
// kv group appends them to the caches (nobody reads cache row *pos in this launch).
struct AttnRope {
  const float* k;     // [n_kv][128] unrotated, or null: q is already rotated and the caches hold position *pos
  const float* v;     // [n_kv][128]
  const float* cosT;  // [max_seq][128]
  const float* sinT;
  float* kc_w;        // the caches, writable
  float* vc_w;
};

__global__ void __launch_bounds__(256) attn_partial_kernel(const float* q, const float* kc,
                                                           const float* vc, float* part,
                                                           const int* pos_p, int n_heads, int n_kv,
                                                           int max_seq, float scale, const AttnRope rope) {
  __shared__ float scores[1024];
  __shared__ float red[8];
  __shared__ float4 vacc[8][32];
  pdl_launch_dependents();
  pdl_wait();
  constexpr int hd = 128;
  const int head = blockIdx.x, split = blockIdx.y, group = n_heads / n_kv, kvh = head / group;
  const int pos = *pos_p;
  const int n_ctx = pos + 1;
  const int chunk = (n_ctx + kAttnSplits - 1) / kAttnSplits;  // <= 1024 for max_seq <= 8192
  const int t0 = split * chunk, t1 = min(t0 + chunk, n_ctx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* out = part + ((size_t)head * kAttnSplits + split) * kAttnPartStride;
  if (t0 >= t1) {  // empty chunk: neutral element
    if (threadIdx.x < hd) out[threadIdx.x] = 0.f;
    if (threadIdx.x == 0) out[128] = -INFINITY, out[129] = 0.f;
    return;
  }
  float4 qv = reinterpret_cast<const float4*>(q + (size_t)head * hd)[lane];
  float4 knew = make_float4(0.f, 0.f, 0.f, 0.f), vnew = knew;
  const bool fused = rope.k != nullptr;
  if (fused) {
    const float4 cs = reinterpret_cast<const float4*>(rope.cosT + (size_t)pos * hd)[lane];
    const float4 sn = reinterpret_cast<const float4*>(rope.sinT + (size_t)pos * hd)[lane];
    qv = rope128(qv, cs, sn, lane);
    knew = rope128(reinterpret_cast<const float4*>(rope.k + (size_t)kvh * hd)[lane], cs, sn, lane);
    vnew = reinterpret_cast<const float4*>(rope.v + (size_t)kvh * hd)[lane];
    if (warp == 0 && head == kvh * group && pos >= t0 && pos < t1) {  // one writer per kv head
      reinterpret_cast<float4*>(rope.kc_w + ((size_t)kvh * max_seq + pos) * hd)[lane] = knew;
      reinterpret_cast<float4*>(rope.vc_w + ((size_t)kvh * max_seq + pos) * hd)[lane] = vnew;
    }
  }
  const float* kbase = kc + (size_t)kvh * max_seq * hd;
  for (int t = t0 + warp; t < t1; t += 8) {
    const float4 kv = (fused && t == pos) ? knew : reinterpret_cast<const float4*>(kbase + (size_t)t * hd)[lane];
    float s = qv.x * kv.x + qv.y * kv.y + qv.z * kv.z + qv.w * kv.w;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) scores[t - t0] = s * scale;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int t = threadIdx.x; t < t1 - t0; t += blockDim.x) mx = fmaxf(mx, scores[t]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  float sum = 0.f;
  for (int t = threadIdx.x; t < t1 - t0; t += blockDim.x) {
    const float e = expf(scores[t] - mx);
    scores[t] = e;
    sum += e;
  }
  const float tot = block_sum_256(sum, red);  // its barriers also order the score updates
  const float* vbase = vc + (size_t)kvh * max_seq * hd;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t = t0 + warp; t < t1; t += 8) {  // a warp per V row, a lane per four columns
    const float pw = scores[t - t0];
    const float4 vv = (fused && t == pos) ? vnew : reinterpret_cast<const float4*>(vbase + (size_t)t * hd)[lane];
    a.x += pw * vv.x, a.y += pw * vv.y, a.z += pw * vv.z, a.w += pw * vv.w;
  }
  vacc[warp][lane] = a;
  __syncthreads();
  if (threadIdx.x < 32) {
    float4 r = vacc[0][lane];
    for (int w = 1; w < 8; ++w) {  // fixed order
      const float4 o = vacc[w][lane];
      r.x += o.x, r.y += o.y, r.z += o.z, r.w += o.w;
    }
    reinterpret_cast<float4*>(out)[lane] = r;
    if (lane == 0) out[128] = mx, out[129] = tot;
  }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* part, float* out) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, d = threadIdx.x;
  const float* p = part + (size_t)head * kAttnSplits * kAttnPartStride;
  float M = -INFINITY;
  for (int s = 0; s < kAttnSplits; ++s) M = fmaxf(M, p[s * kAttnPartStride + 128]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < kAttnSplits; ++s) {
    const float w = expf(p[s * kAttnPartStride + 128] - M);  // exp(-inf) = 0 for empty chunks
    num += w * p[s * kAttnPartStride + d];
    den += w * p[s * kAttnPartStride + 129];
  }
  out[(size_t)head * 128 + d] = num / den;
}

// ---- fused producers: the same results as the plain kernels above followed by the activation
// quantizer, without the f32 round trip and the extra launch (single-GPU step only: with tensor
// parallelism the full vector exists only after an all-gather).

// Rows of `dim` (a multiple of 256, at most 8192; one CTA per row, one warp per 256 elements): optional
// residual add (x += delta, written back), then RMSNorm with gain. kQuant = false stores the f32 row to
// `out`; kQuant = true (one row) quantizes it into the activation planes. Both forms share every
// arithmetic step and its order, so they produce the same values.
// n_parts > 1: the residual delta arrives as n_parts partial vectors (one per GPU of a row-parallel layer, `dim` words
// apart) and is their sum in the balanced pairwise order ((p0 + p1) + (p2 + p3)) + ... — the top of the summation tree
// whose lower levels each GPU's tree-ordered mat-vec has already done, so the value is the one-GPU value bit for bit.
template <bool kQuant, bool kPeer>
__device__ __forceinline__ void add_rmsnorm_body(float* x, const void* delta_v, int n_parts,
                                                 const float* gain, float* out, int dim, float eps,
                                                 int8_t* out_qs, float* out_d,
                                                 int16_t* out_bsums, const PeerCtx* pc) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t base = (size_t)blockIdx.x * dim + warp * 256;
  float e[8];
  float ss = 0.f;
  {
    float4* xr = reinterpret_cast<float4*>(x + base);
    float4 v0 = xr[lane], v1 = xr[32 + lane];
    if (delta_v) {
      // parts are taken in order and merged like a binary counter: lv0[l] / lv1[l] hold the sum of a complete subtree of
      // 2^l parts waiting for its sibling
      float4 lv0[3], lv1[3], d0 = make_float4(0.f, 0.f, 0.f, 0.f), d1 = d0;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (q < n_parts) {
          float4 c0, c1;
          if constexpr (kPeer) {
            // delta arrives from the peers' kernels as stamped pairs (one row per part)
            const uint2* dl = reinterpret_cast<const uint2*>(delta_v) + (size_t)q * dim + warp * 256;
            const uint32_t want = peer_stamp(*pc, pc->wait_seq);
            uint32_t a[4], b[4];
            peer_load_words2<4, 4>(dl + 4 * lane, dl + 128 + 4 * lane, want, a, b, pc->wait_ns);
            c0 = make_float4(__uint_as_float(a[0]), __uint_as_float(a[1]), __uint_as_float(a[2]), __uint_as_float(a[3]));
            c1 = make_float4(__uint_as_float(b[0]), __uint_as_float(b[1]), __uint_as_float(b[2]), __uint_as_float(b[3]));
          } else {
            const float4* dr = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(delta_v) + (size_t)q * dim + base);
            c0 = dr[lane], c1 = dr[32 + lane];
          }
#pragma unroll
          for (int l = 0; l < 3; ++l) {
            if ((q >> l) & 1) {  // a left sibling of this size is waiting: left + right
              c0.x = lv0[l].x + c0.x, c0.y = lv0[l].y + c0.y, c0.z = lv0[l].z + c0.z, c0.w = lv0[l].w + c0.w;
              c1.x = lv1[l].x + c1.x, c1.y = lv1[l].y + c1.y, c1.z = lv1[l].z + c1.z, c1.w = lv1[l].w + c1.w;
            } else {
              lv0[l] = c0, lv1[l] = c1;
              break;
            }
          }
          d0 = c0, d1 = c1;  // after the last part (n_parts a power of two) this is the whole tree
        }
      }
      v0.x += d0.x, v0.y += d0.y, v0.z += d0.z, v0.w += d0.w;
      v1.x += d1.x, v1.y += d1.y, v1.z += d1.z, v1.w += d1.w;
      xr[lane] = v0, xr[32 + lane] = v1;
    }
    e[0] = v0.x, e[1] = v0.y, e[2] = v0.z, e[3] = v0.w, e[4] = v1.x, e[5] = v1.y, e[6] = v1.z, e[7] = v1.w;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += e[i] * e[i];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];  // fixed order
  const float rinv = 1.0f / sqrtf(tot * (1.0f / (float)dim) + eps);
  const float4 g0 = reinterpret_cast<const float4*>(gain + warp * 256)[lane];
  const float4 g1 = reinterpret_cast<const float4*>(gain + warp * 256)[32 + lane];
  const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = e[i] * rinv * gg[i];
  if constexpr (kQuant) {
    q8k_block_from_regs(e, lane, warp, out_qs, out_d, out_bsums);
  } else {
    float4* o = reinterpret_cast<float4*>(out + base);
    o[lane] = make_float4(e[0], e[1], e[2], e[3]);
    o[32 + lane] = make_float4(e[4], e[5], e[6], e[7]);
  }
}

template <bool kQuant>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* x, const float* delta,
                                                           const float* gain, float* out, int dim,
                                                           float eps, int8_t* out_qs, float* out_d,
                                                           int16_t* out_bsums) {
  add_rmsnorm_body<kQuant, false>(x, delta, 1, gain, out, dim, eps, out_qs, out_d, out_bsums, nullptr);
}

// quantizing form whose residual delta is the pairwise sum of n_parts partial vectors [n_parts][dim]
__global__ void __launch_bounds__(1024) add_rmsnorm_q8k_parts_kernel(float* x, const float* parts, int n_parts,
                                                                     const float* gain, int dim, float eps,
                                                                     int8_t* out_qs, float* out_d, int16_t* out_bsums) {
  add_rmsnorm_body<true, false>(x, parts, n_parts, gain, nullptr, dim, eps, out_qs, out_d, out_bsums, nullptr);
}

// quantizing form whose residual delta (stamped pairs) arrives through exchange point pc.wait_seq
__global__ void __launch_bounds__(1024) add_rmsnorm_q8k_peer_kernel(float* x, const uint2* delta, int n_parts,
                                                                    const float* gain, int dim, float eps,
                                                                    int8_t* out_qs, float* out_d,
                                                                    int16_t* out_bsums, const PeerCtx pc) {
  add_rmsnorm_body<true, true>(x, delta, n_parts, gain, nullptr, dim, eps, out_qs, out_d, out_bsums, &pc);
}

// silu(gate) * up, quantized; one warp per 256 elements
__global__ void __launch_bounds__(256) swiglu_q8k_kernel(const float* gate, const float* up,
                                                         int64_t n_blocks, int8_t* out_qs,
                                                         float* out_d, int16_t* out_bsums) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (blk >= n_blocks) return;
  const float4* gp = reinterpret_cast<const float4*>(gate + blk * 256);
  const float4* up4 = reinterpret_cast<const float4*>(up + blk * 256);
  const float4 a0 = gp[lane], a1 = gp[32 + lane], b0 = up4[lane], b1 = up4[32 + lane];
  const float g[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  const float u[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  float e[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
  q8k_block_from_regs(e, lane, blk, out_qs, out_d, out_bsums);
}

// merge of the attention chunks for two heads (256 outputs) per warp, quantized
__global__ void __launch_bounds__(32) attn_combine_q8k_kernel(const float* part, int8_t* out_qs,
                                                              float* out_d, int16_t* out_bsums) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x, blk = blockIdx.x;
  float e[8];
#pragma unroll
  for (int hsel = 0; hsel < 2; ++hsel) {  // elements 4*lane.. belong to head 2*blk, 128 + 4*lane.. to head 2*blk + 1
    const float* p = part + (size_t)(2 * blk + hsel) * kAttnSplits * kAttnPartStride;
    float M = -INFINITY;
    for (int s = 0; s < kAttnSplits; ++s) M = fmaxf(M, p[s * kAttnPartStride + 128]);
    float num[4] = {0, 0, 0, 0}, den = 0.f;
    for (int s = 0; s < kAttnSplits; ++s) {
      const float w = expf(p[s * kAttnPartStride + 128] - M);
      const float4 v = reinterpret_cast<const float4*>(p + s * kAttnPartStride)[lane];
      num[0] += w * v.x, num[1] += w * v.y, num[2] += w * v.z, num[3] += w * v.w;
      den += w * p[s * kAttnPartStride + 129];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) e[4 * hsel + i] = num[i] / den;
  }
  q8k_block_from_regs(e, lane, blk, out_qs, out_d, out_bsums);
}

__global__ void __launch_bounds__(256) swiglu_kernel(const float* gate, const float* up,
                                                     float* out, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float g = gate[i];
    out[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

// index of the LAST maximum (ties and NaN-free data); one CTA
template <bool kPeer>
__device__ __forceinline__ void argmax_last_body(const float* x, int n, int* out, const PeerCtx* pc,
                                                 uint32_t* epoch) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();
  pdl_wait();
  float bv = -INFINITY;
  int bi = -1;
  if constexpr (kPeer) {
    // x is a buffer of n stamped pairs (n even) filled through exchange point pc->wait_seq
    const uint2* xl = reinterpret_cast<const uint2*>(x);
    const uint32_t want = peer_stamp(*pc, pc->wait_seq);
    for (int i = 2 * threadIdx.x; i < n; i += 2 * blockDim.x) {
      uint32_t w[2];
      peer_load_words<2>(xl + i, want, w, pc->wait_ns);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float v = __uint_as_float(w[j]);
        if (v > bv || (v == bv && i + j > bi)) bv = v, bi = i + j;
      }
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = x[i];
      if (v > bv || (v == bv && i > bi)) bv = v, bi = i;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > bv || (ov == bv && oi > bi)) bv = ov, bi = oi;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sv[warp] = bv, si[warp] = bi;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] > bi)) bv = sv[w], bi = si[w];
    *out = bi;
    if constexpr (kPeer) *epoch = *epoch + 1u;  // last kernel of a step: the next step's stamps differ
  }
}

__global__ void __launch_bounds__(1024) argmax_last_kernel(const float* x, int n, int* out) {
  argmax_last_body<false>(x, n, out, nullptr, nullptr);
}

// The reduction of a row-parallel layer by itself: y = the pairwise sum, in rank order, of n_parts partial vectors
// (stamped pairs in this rank's buffer, filled through exchange point pc.wait_seq) - the value add_rmsnorm_q8k_peer adds
// to the residual, for callers whose next op is not that norm. Four words per thread.
__global__ void __launch_bounds__(256) rowpar_reduce_kernel(const uint2* parts, int n_parts, int n, float* y, const PeerCtx pc) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const uint32_t want = peer_stamp(pc, pc.wait_seq);
  float4 lv[3], d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (q < n_parts) {
      uint32_t a[4];
      peer_load_words<4>(parts + (size_t)q * n + i, want, a, pc.wait_ns);
      float4 c = make_float4(__uint_as_float(a[0]), __uint_as_float(a[1]), __uint_as_float(a[2]), __uint_as_float(a[3]));
#pragma unroll
      for (int l = 0; l < 3; ++l) {
        if ((q >> l) & 1) {
          c.x = lv[l].x + c.x, c.y = lv[l].y + c.y, c.z = lv[l].z + c.z, c.w = lv[l].w + c.w;
        } else {
          lv[l] = c;
          break;
        }
      }
      d = c;
    }
  }
  *reinterpret_cast<float4*>(y + i) = d;
}

// logits arrive as stamped pairs through exchange point pc.wait_seq; also advances this rank's step counter
__global__ void __launch_bounds__(1024) argmax_last_peer_kernel(const float* x, int n, int* out,
                                                                const PeerCtx pc, uint32_t* epoch) {
  argmax_last_body<true>(x, n, out, &pc, epoch);
}

}  // namespace fq
