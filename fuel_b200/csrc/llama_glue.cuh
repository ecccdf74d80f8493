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

namespace fq {

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

// rows of `dim`: optional residual add (x += delta, written back), then RMSNorm with gain into out
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                          const float* __restrict__ gain, float* __restrict__ out, int dim,
                                                          float eps) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  float* xr = x + (size_t)blockIdx.x * dim;
  const float* dr = delta ? delta + (size_t)blockIdx.x * dim : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      v += dr[i];
      xr[i] = v;
    }
    ss += v * v;
  }
  const float tot = block_sum_256(ss, red);
  const float rinv = 1.0f / sqrtf(tot * (1.0f / (float)dim) + eps);
  float* o = out + (size_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = xr[i] * rinv * gain[i];
}

// token ids -> dequantized Q4_K rows of the embedding table (one CTA per id, 16 threads per super-block)
__global__ void __launch_bounds__(256) embed_q4k_kernel(const uint8_t* __restrict__ table, int row_bytes, int k,
                                                        const int* __restrict__ ids, float* __restrict__ out) {
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
__global__ void __launch_bounds__(128) rope_store_kernel(float* __restrict__ q, const float* __restrict__ k,
                                                         const float* __restrict__ v, float* __restrict__ kc,
                                                         float* __restrict__ vc, const float* __restrict__ cosT,
                                                         const float* __restrict__ sinT, const int* __restrict__ pos_p,
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
      x[i] = lo * cs[i] - hi * sn[i];
      x[i + half] = hi * cs[i + half] + lo * sn[i + half];
    }
  } else {
    const int kh = head - n_heads;
    const float* x = k + (size_t)kh * hd;
    float* kd = kc + ((size_t)kh * max_seq + pos) * hd;
    float* vd = vc + ((size_t)kh * max_seq + pos) * hd;
    const float* vs = v + (size_t)kh * hd;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float lo = x[i], hi = x[i + half];
      kd[i] = lo * cs[i] - hi * sn[i];
      kd[i + half] = hi * cs[i + half] + lo * sn[i + half];
      vd[i] = vs[i];
      vd[i + half] = vs[i + half];
    }
  }
}

// one query per head against positions 0..*pos of the cache (GQA: head h reads kv head h / (n_heads / n_kv))
// hd must be 128; dynamic shared memory: (max_seq + 8 + 2 * 128) floats
__global__ void __launch_bounds__(256) attn_decode_kernel(const float* __restrict__ q, const float* __restrict__ kc,
                                                          const float* __restrict__ vc, float* __restrict__ out,
                                                          const int* __restrict__ pos_p, int n_heads, int n_kv,
                                                          int max_seq, float scale) {
  extern __shared__ float sm_attn[];
  float* scores = sm_attn;           // [max_seq]
  float* red = sm_attn + max_seq;    // [8]
  float* part = red + 8;             // [2][128]
  pdl_launch_dependents();
  pdl_wait();
  constexpr int hd = 128;
  const int head = blockIdx.x, kvh = head / (n_heads / n_kv);
  const int n_ctx = *pos_p + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float4 qv = reinterpret_cast<const float4*>(q + (size_t)head * hd)[lane];
  const float* kbase = kc + (size_t)kvh * max_seq * hd;
  for (int t = warp; t < n_ctx; t += 8) {
    const float4 kv = reinterpret_cast<const float4*>(kbase + (size_t)t * hd)[lane];
    float s = qv.x * kv.x + qv.y * kv.y + qv.z * kv.z + qv.w * kv.w;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) scores[t] = s * scale;
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int t = threadIdx.x; t < n_ctx; t += blockDim.x) mx = fmaxf(mx, scores[t]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  float sum = 0.f;
  for (int t = threadIdx.x; t < n_ctx; t += blockDim.x) {
    const float e = expf(scores[t] - mx);
    scores[t] = e;
    sum += e;
  }
  const float tot = block_sum_256(sum, red);  // also orders the score writes before the reads below
  const float inv = 1.0f / tot;
  // out[d] = sum_t p_t * v[t][d]: two halves of the context per column, combined in fixed order
  const int d = threadIdx.x & 127, hsel = threadIdx.x >> 7;
  const int t_mid = (n_ctx + 1) >> 1;
  const float* vbase = vc + (size_t)kvh * max_seq * hd;
  float acc = 0.f;
  for (int t = hsel ? t_mid : 0; t < (hsel ? n_ctx : t_mid); ++t) acc += scores[t] * vbase[(size_t)t * hd + d];
  part[hsel * 128 + d] = acc;
  __syncthreads();
  if (hsel == 0) out[(size_t)head * hd + d] = (part[d] + part[128 + d]) * inv;
}

__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                     float* __restrict__ out, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float g = gate[i];
    out[i] = (g / (1.0f + expf(-g))) * up[i];
  }
}

// index of the LAST maximum (ties and NaN-free data); one CTA
__global__ void __launch_bounds__(1024) argmax_last_kernel(const float* __restrict__ x, int n, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();
  pdl_wait();
  float bv = -INFINITY;
  int bi = -1;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = x[i];
    if (v > bv || (v == bv && i > bi)) bv = v, bi = i;
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
  }
}

}  // namespace fq
