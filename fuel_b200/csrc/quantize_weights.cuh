// Weight quantizers on the device: f32 -> Q8_0 / Q4_0 / Q4_K / Q6_K blocks, byte for byte what
// the reference's host quantizers emit (the reference quantizes GPU weights on the CPU and
// uploads them, fuel-cuda-backend/src/quantized.rs:389-412):
//   Q8_0  BlockQ8_0::from_float   fuel-quantized/src/k_quants.rs:629-658
//   Q4_0  BlockQ4_0::from_float   k_quants.rs:199-235
//   Q4_K  BlockQ4K::from_float    k_quants.rs:1470-1528 + make_qkx1_quants, utils.rs:229-286
//   Q6_K  BlockQ6K::from_float    k_quants.rs:2005-2075 + make_qx_quants,   utils.rs:62-191
//   (and Q4_1, Q5_0, Q5_1, Q5_K, Q2_K, Q3_K further down, each cited at its kernel)
// One thread per sub-block runs the reference's sequential fit in the reference's order;
// the few cross-sub-block steps (max scale, packing) go through warp shuffles.
// Every float operation is an explicit round-to-nearest intrinsic so nothing contracts into
// an fma; float->int conversions saturate and send NaN to 0 on both sides.
#pragma once
#include "fq_common.cuh"

namespace fq {

__device__ __forceinline__ int qw_nearest_int(float v) { return __float2int_rz(roundf(v)); }
__device__ __forceinline__ int qw_clamp(int v, int lo, int hi) { return min(max(v, lo), hi); }

// ---------------------------------------------------------------- Q8_0 / Q4_0: one thread per block
__global__ void __launch_bounds__(128) quantize_w_q8_0_kernel(const float* __restrict__ x, int64_t nb,
                                                              uint8_t* __restrict__ out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float v[32];
  const float4* src = reinterpret_cast<const float4*>(x + b * 32);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 t = src[j];
    v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  uint16_t* o = reinterpret_cast<uint16_t*>(out + b * Q8_0L::kBytes);
  o[0] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int q0 = qw_clamp(qw_nearest_int(__fmul_rn(v[2 * j], id)), -128, 127);
    const int q1 = qw_clamp(qw_nearest_int(__fmul_rn(v[2 * j + 1], id)), -128, 127);
    o[1 + j] = (uint16_t)((q0 & 0xff) | ((q1 & 0xff) << 8));
  }
}

__global__ void __launch_bounds__(128) quantize_w_q4_0_kernel(const float* __restrict__ x, int64_t nb,
                                                              uint8_t* __restrict__ out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float v[32];
  const float4* src = reinterpret_cast<const float4*>(x + b * 32);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 t = src[j];
    v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
  }
  float amax = 0.f, mx = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float a = fabsf(v[j]);
    if (amax < a) amax = a, mx = v[j];
  }
  const float d = __fdiv_rn(mx, -8.0f);
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  uint16_t* o = reinterpret_cast<uint16_t*>(out + b * Q4_0L::kBytes);
  o[0] = __half_as_ushort(__float2half_rn(d));
  auto nib = [&](float xv) -> uint32_t {
    // (x*id + 8.5) as u8, saturating, then min 15
    const int t = __float2int_rz(__fadd_rn(__fmul_rn(xv, id), 8.5f));
    return (uint32_t)qw_clamp(t, 0, 15);
  };
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t b0 = nib(v[2 * j]) | (nib(v[16 + 2 * j]) << 4);
    const uint32_t b1 = nib(v[2 * j + 1]) | (nib(v[16 + 2 * j + 1]) << 4);
    o[1 + j] = (uint16_t)(b0 | (b1 << 8));
  }
}

// Q4_1 / Q5_0 / Q5_1 (BlockQ4_1::from_float k_quants.rs:315-351, BlockQ5_0 :424-460, BlockQ5_1 :535-575): one thread
// per block. kFive: a fifth bit per element collected in the 32-bit word qh; kMin: scale over [min, max] with the
// minimum stored, values unsigned. Rust's float -> integer casts saturate and truncate; the additions and products
// are separate roundings.
template <class L, bool kFive, bool kMin>
__global__ void __launch_bounds__(128) quantize_w_legacy32_kernel(const float* __restrict__ x, int64_t nb,
                                                                  uint8_t* __restrict__ out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  float v[32];
  const float4* src = reinterpret_cast<const float4*>(x + b * 32);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 t = src[j];
    v[4 * j] = t.x, v[4 * j + 1] = t.y, v[4 * j + 2] = t.z, v[4 * j + 3] = t.w;
  }
  float d, mn = 0.f;
  if constexpr (kMin) {
    float mx = -INFINITY;
    mn = INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) mn = fminf(v[j], mn), mx = fmaxf(v[j], mx);
    d = __fdiv_rn(__fsub_rn(mx, mn), kFive ? 31.0f : 15.0f);
  } else {
    float amax = 0.f, mx = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float a = fabsf(v[j]);
      if (amax < a) amax = a, mx = v[j];
    }
    d = __fdiv_rn(mx, -16.0f);
  }
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  uint16_t* o = reinterpret_cast<uint16_t*>(out + b * L::kBytes);
  o[0] = __half_as_ushort(__float2half_rn(d));
  if constexpr (kMin) o[1] = __half_as_ushort(__float2half_rn(mn));
  auto quant = [&](float xv) -> uint32_t {
    if constexpr (kMin) {
      // ((x - min) * id + 0.5) as u8 (saturating); Q4_1 then takes min(15, .), Q5_1 keeps the low five bits
      const int t = qw_clamp(__float2int_rz(__fadd_rn(__fmul_rn(__fsub_rn(xv, mn), id), 0.5f)), 0, 255);
      return (uint32_t)(kFive ? t : (t < 15 ? t : 15));
    } else {
      // ((x * id + 16.5) as i8).min(31) as u8
      const int t = qw_clamp(__float2int_rz(__fadd_rn(__fmul_rn(xv, id), 16.5f)), -128, 127);
      return (uint32_t)((t < 31 ? t : 31) & 0xff);
    }
  };
  uint32_t qh = 0;
  uint16_t* qs = reinterpret_cast<uint16_t*>(out + b * L::kBytes + L::kBytes - 16);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t a0 = quant(v[2 * j]), a1 = quant(v[16 + 2 * j]), c0 = quant(v[2 * j + 1]), c1 = quant(v[16 + 2 * j + 1]);
    qs[j] = (uint16_t)(((a0 & 0xf) | ((a1 & 0xf) << 4)) | (((c0 & 0xf) | ((c1 & 0xf) << 4)) << 8));
    if constexpr (kFive) {
      qh |= ((a0 & 0x10) >> 4) << (2 * j);
      qh |= ((a1 & 0x10) >> 4) << (2 * j + 16);
      qh |= ((c0 & 0x10) >> 4) << (2 * j + 1);
      qh |= ((c1 & 0x10) >> 4) << (2 * j + 17);
    }
  }
  if constexpr (kFive) {
    uint16_t* h = reinterpret_cast<uint16_t*>(out + b * L::kBytes + L::kBytes - 20);
    h[0] = (uint16_t)(qh & 0xffff), h[1] = (uint16_t)(qh >> 16);
  }
}

// ---------------------------------------------------------------- Q4_K: one thread per 32-element sub-block
// total order on floats (Rust total_cmp): only matters for -0.0 < +0.0 on finite data
__device__ __forceinline__ bool qw_total_less(float a, float b) {
  int ia = __float_as_int(a), ib = __float_as_int(b);
  ia ^= (int)((unsigned)(ia >> 31) >> 1);
  ib ^= (int)((unsigned)(ib >> 31) >> 1);
  return ia < ib;
}

// kFive: Q5_K (BlockQ5K::from_float, k_quants.rs:1732-1887): the same fit with 32 levels, the fifth bit of element t of
// sub-block s kept as bit s of qh[t].
template <bool kFive>
__global__ void __launch_bounds__(128) quantize_w_q4k_kernel(const float* __restrict__ x, int64_t nb,
                                                             uint8_t* __restrict__ out) {
  constexpr int kNmax = kFive ? 31 : 15;
  constexpr int kBlockBytes = kFive ? Q5KL::kBytes : Q4KL::kBytes;
  constexpr int kQsOff = kFive ? Q5KL::kOffQs : Q4KL::kOffQs;
  const int64_t sub = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // global sub-block index
  const int64_t blk = sub >> 3;
  const int j = (int)(sub & 7);
  const bool live = blk < nb;
  const unsigned lane = threadIdx.x & 31;
  const unsigned gmask = 0xffu << (lane & ~7u);  // the 8 lanes of this super-block
  float v[32];
  if (live) {
    const float4* src = reinterpret_cast<const float4*>(x + sub * 32);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float4 q = src[t];
      v[4 * t] = q.x, v[4 * t + 1] = q.y, v[4 * t + 2] = q.z, v[4 * t + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int t = 0; t < 32; ++t) v[t] = 0.f;
  }
  // make_qkx1_quants(nmax, 5, x) -> (scale, -min)
  float scale = 0.f, negmin = 0.f;
  {
    float mn = v[0], mx = v[0];
#pragma unroll
    for (int t = 1; t < 32; ++t) {
      if (qw_total_less(v[t], mn)) mn = v[t];
      if (!qw_total_less(v[t], mx)) mx = v[t];
    }
    if (mx != mn) {
      if (mn > 0.f) mn = 0.f;
      float iscale = __fdiv_rn((float)kNmax, __fsub_rn(mx, mn));
      scale = __fdiv_rn(1.0f, iscale);
      uint32_t Lp[8];  // 32 levels, 4 bits used of each byte
#pragma unroll
      for (int t = 0; t < 8; ++t) Lp[t] = 0;
      for (int it = 0; it < 5; ++it) {
        float sumlx = 0.f;
        int suml2 = 0;
        bool changed = false;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const float xm = __fsub_rn(v[t], mn);
          const int li = qw_clamp(qw_nearest_int(__fmul_rn(iscale, xm)), 0, kNmax);
          const uint32_t old = (Lp[t >> 2] >> (8 * (t & 3))) & 0xff;
          if ((uint32_t)li != old) {
            Lp[t >> 2] = (Lp[t >> 2] & ~(0xffu << (8 * (t & 3)))) | ((uint32_t)li << (8 * (t & 3)));
            changed = true;
          }
          sumlx = __fadd_rn(sumlx, __fmul_rn(xm, (float)li));
          suml2 += li * li;
        }
        scale = __fdiv_rn(sumlx, (float)suml2);
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const float li = (float)((Lp[t >> 2] >> (8 * (t & 3))) & 0xff);
          sum = __fadd_rn(sum, __fsub_rn(v[t], __fmul_rn(scale, li)));
        }
        mn = __fdiv_rn(sum, 32.0f);
        if (mn > 0.f) mn = 0.f;
        iscale = __fdiv_rn(1.0f, scale);
        if (!changed) break;
      }
      negmin = -mn;
    }
  }
  // max over the eight sub-blocks, folded from 0 in index order (f32::max ignores NaN like fmaxf)
  float max_scale = 0.f, max_min = 0.f;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    max_scale = fmaxf(__shfl_sync(gmask, scale, (lane & ~7u) + s), max_scale);
    max_min = fmaxf(__shfl_sync(gmask, negmin, (lane & ~7u) + s), max_min);
  }
  const float inv_scale = max_scale > 0.f ? __fdiv_rn(63.0f, max_scale) : 0.f;
  const float inv_min = max_min > 0.f ? __fdiv_rn(63.0f, max_min) : 0.f;
  const int ls = min(qw_nearest_int(__fmul_rn(inv_scale, scale)), 63) & 0xff;  // 'as u8' of a value <= 63 (>= 0 here)
  const int lm = min(qw_nearest_int(__fmul_rn(inv_min, negmin)), 63) & 0xff;
  const __half hd = __float2half_rn(__fdiv_rn(max_scale, 63.0f));
  const __half hm = __float2half_rn(__fdiv_rn(max_min, 63.0f));
  // gather all eight (ls, lm) to build the 12 packed scale bytes
  uint32_t lsv[8], lmv[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    lsv[s] = (uint32_t)__shfl_sync(gmask, ls, (lane & ~7u) + s);
    lmv[s] = (uint32_t)__shfl_sync(gmask, lm, (lane & ~7u) + s);
  }
  // re-quantize against the stored (f16-rounded) scales
  const float dsub = __fmul_rn(__half2float(hd), (float)ls);
  uint32_t Lq[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) Lq[t] = 0;
  if (dsub != 0.f) {
    const float dm = __fmul_rn(__half2float(hm), (float)lm);
#pragma unroll
    for (int t = 0; t < 32; ++t) {
      const int l = qw_clamp(qw_nearest_int(__fdiv_rn(__fadd_rn(v[t], dm), dsub)), 0, kNmax);
      Lq[t >> 2] |= (uint32_t)l << (8 * (t & 3));
    }
  }
  // fifth bits: bit t of `high` says element t of this sub-block is above 15; every thread then holds all eight masks
  uint32_t highs[8];
  if constexpr (kFive) {
    uint32_t high = 0;
#pragma unroll
    for (int t = 0; t < 32; ++t) high |= ((Lq[t >> 2] >> (8 * (t & 3) + 4)) & 1u) << t;
#pragma unroll
    for (int t = 0; t < 8; ++t) Lq[t] &= 0x0f0f0f0fu;
#pragma unroll
    for (int s2 = 0; s2 < 8; ++s2) highs[s2] = __shfl_sync(gmask, high, (lane & ~7u) + s2);
  }
  // nibble packing: byte t of group g = L[64g + t] | L[64g + 32 + t] << 4: even sub-block (low) pairs with odd (high)
  uint32_t partner[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) partner[t] = __shfl_xor_sync(gmask, Lq[t], 1);
  if (!live) return;
  uint8_t* ob = out + blk * kBlockBytes;
  if (j == 0) {
    uint8_t sc[12];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      sc[s] = (uint8_t)(lsv[s] | ((lsv[s + 4] >> 4) << 6));
      sc[s + 4] = (uint8_t)(lmv[s] | ((lmv[s + 4] >> 4) << 6));
      sc[s + 8] = (uint8_t)((lsv[s + 4] & 0xF) | ((lmv[s + 4] & 0xF) << 4));
    }
    uint32_t* o32 = reinterpret_cast<uint32_t*>(ob);
    o32[0] = (uint32_t)__half_as_ushort(hd) | ((uint32_t)__half_as_ushort(hm) << 16);
    o32[1] = sc[0] | (sc[1] << 8) | (sc[2] << 16) | ((uint32_t)sc[3] << 24);
    o32[2] = sc[4] | (sc[5] << 8) | (sc[6] << 16) | ((uint32_t)sc[7] << 24);
    o32[3] = sc[8] | (sc[9] << 8) | (sc[10] << 16) | ((uint32_t)sc[11] << 24);
  }
  if constexpr (kFive) {  // thread j writes qh[4j .. 4j + 3]: bit s of qh[t] = fifth bit of element t of sub-block s
    uint32_t word = 0;
#pragma unroll
    for (int tt = 0; tt < 4; ++tt) {
      uint32_t byte = 0;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) byte |= ((highs[s2] >> (4 * j + tt)) & 1u) << s2;
      word |= byte << (8 * tt);
    }
    reinterpret_cast<uint32_t*>(ob + Q5KL::kOffQh)[j] = word;
  }
  // each thread of a pair writes half of the pair's 32 bytes: even -> bytes 0..15, odd -> 16..31
  uint32_t* oq = reinterpret_cast<uint32_t*>(ob + kQsOff + 32 * (j >> 1) + 16 * (j & 1));
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int src = 4 * (j & 1) + t;  // words 0..3 or 4..7 of the 32 levels
    const uint32_t lo = (j & 1) ? partner[src] : Lq[src];
    const uint32_t hi = (j & 1) ? Lq[src] : partner[src];
    oq[t] = lo | (hi << 4);
  }
}

// ---------------------------------------------------------------- Q2_K, Q3_K: one thread per 16-element sub-block,
// the sixteen threads of a super-block are half a warp (BlockQ2K::from_float k_quants.rs:836-895 with
// make_qkx1_quants(3, 5, .); BlockQ3K::from_float :1135-1216 with make_q3_quants(., 4, true), utils.rs:289-354)
__device__ __forceinline__ void qw_load16(const float* x, int64_t sub, bool live, float (&v)[16]) {
  if (live) {
    const float4* src = reinterpret_cast<const float4*>(x + sub * 16);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float4 q = src[t];
      v[4 * t] = q.x, v[4 * t + 1] = q.y, v[4 * t + 2] = q.z, v[4 * t + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int t = 0; t < 16; ++t) v[t] = 0.f;
  }
}
// 16 two-bit levels (bits 2i of lv) of the four sub-blocks that share 16 bytes of qs -> those bytes, written by the
// thread of the first of the four (bit pair 0); sub-block j = 8c + 2g + h supplies bit pair g of bytes 32c + 16h + i
__device__ __forceinline__ void qw_store_qs2(uint32_t lv, int j, unsigned gmask, unsigned base_lane, bool live, uint8_t* qs) {
  const int c = j >> 3, g = (j >> 1) & 3, h = j & 1;
  const uint32_t l1 = __shfl_sync(gmask, lv, base_lane + ((j + 2) & 15));
  const uint32_t l2 = __shfl_sync(gmask, lv, base_lane + ((j + 4) & 15));
  const uint32_t l3 = __shfl_sync(gmask, lv, base_lane + ((j + 6) & 15));
  if (!live || g != 0) return;
  uint32_t* o = reinterpret_cast<uint32_t*>(qs + 32 * c + 16 * h);
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t word = 0;
#pragma unroll
    for (int bb = 0; bb < 4; ++bb) {
      const int i = 4 * wd + bb;
      const uint32_t byte = ((lv >> (2 * i)) & 3u) | (((l1 >> (2 * i)) & 3u) << 2) | (((l2 >> (2 * i)) & 3u) << 4) |
                            (((l3 >> (2 * i)) & 3u) << 6);
      word |= byte << (8 * bb);
    }
    o[wd] = word;
  }
}

__global__ void __launch_bounds__(128) quantize_w_q2k_kernel(const float* __restrict__ x, int64_t nb, uint8_t* __restrict__ out) {
  const int64_t sub = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t blk = sub >> 4;
  const int j = (int)(sub & 15);
  const bool live = blk < nb;
  const unsigned lane = threadIdx.x & 31, base_lane = lane & ~15u;
  const unsigned gmask = 0xffffu << base_lane;
  float v[16];
  qw_load16(x, sub, live, v);
  // make_qkx1_quants(3, 5, x) -> (scale, -min)
  float scale = 0.f, negmin = 0.f;
  {
    float mn = v[0], mx = v[0];
#pragma unroll
    for (int t = 1; t < 16; ++t) {
      if (qw_total_less(v[t], mn)) mn = v[t];
      if (!qw_total_less(v[t], mx)) mx = v[t];
    }
    if (mx != mn) {
      if (mn > 0.f) mn = 0.f;
      float iscale = __fdiv_rn(3.0f, __fsub_rn(mx, mn));
      scale = __fdiv_rn(1.0f, iscale);
      uint32_t Lp = 0;  // 16 levels, two bits each
      for (int it = 0; it < 5; ++it) {
        float sumlx = 0.f;
        int suml2 = 0;
        bool changed = false;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const float xm = __fsub_rn(v[t], mn);
          const int li = qw_clamp(qw_nearest_int(__fmul_rn(iscale, xm)), 0, 3);
          if ((uint32_t)li != ((Lp >> (2 * t)) & 3u)) {
            Lp = (Lp & ~(3u << (2 * t))) | ((uint32_t)li << (2 * t));
            changed = true;
          }
          sumlx = __fadd_rn(sumlx, __fmul_rn(xm, (float)li));
          suml2 += li * li;
        }
        scale = __fdiv_rn(sumlx, (float)suml2);
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < 16; ++t) sum = __fadd_rn(sum, __fsub_rn(v[t], __fmul_rn(scale, (float)((Lp >> (2 * t)) & 3u))));
        mn = __fdiv_rn(sum, 16.0f);
        if (mn > 0.f) mn = 0.f;
        iscale = __fdiv_rn(1.0f, scale);
        if (!changed) break;
      }
      negmin = -mn;
    }
  }
  float max_scale = 0.f, max_min = 0.f;
#pragma unroll
  for (int s2 = 0; s2 < 16; ++s2) {
    max_scale = fmaxf(__shfl_sync(gmask, scale, base_lane + s2), max_scale);
    max_min = fmaxf(__shfl_sync(gmask, negmin, base_lane + s2), max_min);
  }
  int ls = 0, lm = 0;
  __half hd = __float2half_rn(0.f), hm = __float2half_rn(0.f);
  if (max_scale > 0.f) {
    ls = qw_nearest_int(__fmul_rn(__fdiv_rn(15.0f, max_scale), scale)) & 0xff;   // 'as u8'
    hd = __float2half_rn(__fdiv_rn(max_scale, 15.0f));
  }
  if (max_min > 0.f) {
    lm = qw_nearest_int(__fmul_rn(__fdiv_rn(15.0f, max_min), negmin)) & 0xff;
    hm = __float2half_rn(__fdiv_rn(max_min, 15.0f));
  }
  const uint32_t sc_byte = ((uint32_t)ls | ((uint32_t)lm << 4)) & 0xffu;  // scales[j] |= l << 4 in u8 arithmetic
  const float dsub = __fmul_rn(__half2float(hd), (float)(sc_byte & 0xFu));
  uint32_t lv = 0;
  if (dsub != 0.f) {
    const float dm = __fmul_rn(__half2float(hm), (float)(sc_byte >> 4));
#pragma unroll
    for (int t = 0; t < 16; ++t)
      lv |= (uint32_t)qw_clamp(qw_nearest_int(__fdiv_rn(__fadd_rn(v[t], dm), dsub)), 0, 3) << (2 * t);
  }
  uint8_t* ob = out + (live ? blk : 0) * Q2KL::kBytes;
  qw_store_qs2(lv, j, gmask, base_lane, live, ob + Q2KL::kOffQs);
  if (!live) return;
  ob[Q2KL::kOffScales + j] = (uint8_t)sc_byte;
  if (j == 0)
    *reinterpret_cast<uint32_t*>(ob + Q2KL::kOffD) = (uint32_t)__half_as_ushort(hd) | ((uint32_t)__half_as_ushort(hm) << 16);
}

// make_q3_quants(x, 4, true): levels -4 .. 3, weights x^2, up to five refinement sweeps; returns the scale
__device__ __forceinline__ float qw_make_q3_16(const float (&x)[16]) {
  const int nmax = 4;
  float mx = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float ax = fabsf(x[i]);
    if (ax > amax) amax = ax, mx = x[i];
  }
  if (amax == 0.f) return 0.f;
  const float iscale = __fdiv_rn(-(float)nmax, mx);
  int L[16];
  float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int li = qw_clamp(qw_nearest_int(__fmul_rn(iscale, x[i])), -nmax, nmax - 1);
    L[i] = li;
    const float w = __fmul_rn(x[i], x[i]);
    sumlx = __fadd_rn(sumlx, __fmul_rn(__fmul_rn(w, x[i]), (float)li));
    suml2 = __fadd_rn(suml2, __fmul_rn(w, (float)(li * li)));
  }
  for (int it = 0; it < 5; ++it) {
    int changed = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float w = __fmul_rn(x[i], x[i]);
      float slx = __fsub_rn(sumlx, __fmul_rn(__fmul_rn(w, x[i]), (float)L[i]));
      if (slx > 0.f) {
        float sl2 = __fsub_rn(suml2, __fmul_rn(w, (float)(L[i] * L[i])));
        const int nl = qw_clamp(qw_nearest_int(__fdiv_rn(__fmul_rn(x[i], sl2), slx)), -nmax, nmax - 1);
        if (nl != L[i]) {
          slx = __fadd_rn(slx, __fmul_rn(__fmul_rn(w, x[i]), (float)nl));
          sl2 = __fadd_rn(sl2, __fmul_rn(w, (float)(nl * nl)));
          if (sl2 > 0.f && __fmul_rn(__fmul_rn(slx, slx), suml2) > __fmul_rn(__fmul_rn(sumlx, sumlx), sl2)) {
            L[i] = nl;
            sumlx = slx;
            suml2 = sl2;
            ++changed;
          }
        }
      }
    }
    if (!changed) break;
  }
  return __fdiv_rn(sumlx, suml2);
}

__global__ void __launch_bounds__(128) quantize_w_q3k_kernel(const float* __restrict__ x, int64_t nb, uint8_t* __restrict__ out) {
  const int64_t sub = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t blk = sub >> 4;
  const int j = (int)(sub & 15);
  const bool live = blk < nb;
  const unsigned lane = threadIdx.x & 31, base_lane = lane & ~15u;
  const unsigned gmask = 0xffffu << base_lane;
  float v[16];
  qw_load16(x, sub, live, v);
  const float scale = qw_make_q3_16(v);
  // the scale of largest magnitude, first one wins
  float max_scale = 0.f;
#pragma unroll
  for (int s2 = 0; s2 < 16; ++s2) {
    const float sc = __shfl_sync(gmask, scale, base_lane + s2);
    if (fabsf(sc) > fabsf(max_scale)) max_scale = sc;
  }
  int l6 = 0;
  __half hd = __float2half_rn(0.f);
  if (max_scale != 0.f) {
    const float iscale = __fdiv_rn(-32.0f, max_scale);
    l6 = qw_clamp(qw_nearest_int(__fmul_rn(iscale, scale)), -32, 31) + 32;
    hd = __float2half_rn(__fdiv_rn(1.0f, iscale));
  }
  uint32_t l6v[16];
#pragma unroll
  for (int s2 = 0; s2 < 16; ++s2) l6v[s2] = (uint32_t)__shfl_sync(gmask, l6, base_lane + s2);
  const float dsub = __fmul_rn(__half2float(hd), (float)(l6 - 32));
  uint32_t lv = 0, hb = 0;   // low two bits of every level; bit i: level of element i is above 3
  if (dsub != 0.f) {
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const int l = qw_clamp(qw_nearest_int(__fdiv_rn(v[t], dsub)), -4, 3) + 4;
      lv |= (uint32_t)(l & 3) << (2 * t);
      hb |= (uint32_t)(l >> 2) << t;
    }
  }
  uint32_t hbv[16];
#pragma unroll
  for (int s2 = 0; s2 < 16; ++s2) hbv[s2] = __shfl_sync(gmask, hb, base_lane + s2);
  uint8_t* ob = out + (live ? blk : 0) * Q3KL::kBytes;   // 110-byte blocks: 2-byte aligned
  {
    // qs as in Q2_K, but through 16-bit stores
    const int c = j >> 3, g = (j >> 1) & 3, h = j & 1;
    const uint32_t l1 = __shfl_sync(gmask, lv, base_lane + ((j + 2) & 15));
    const uint32_t l2 = __shfl_sync(gmask, lv, base_lane + ((j + 4) & 15));
    const uint32_t l3 = __shfl_sync(gmask, lv, base_lane + ((j + 6) & 15));
    if (live && g == 0) {
      uint16_t* o = reinterpret_cast<uint16_t*>(ob + Q3KL::kOffQs + 32 * c + 16 * h);
#pragma unroll
      for (int hw = 0; hw < 8; ++hw) {
        uint32_t half = 0;
#pragma unroll
        for (int bb = 0; bb < 2; ++bb) {
          const int i = 2 * hw + bb;
          const uint32_t byte = ((lv >> (2 * i)) & 3u) | (((l1 >> (2 * i)) & 3u) << 2) | (((l2 >> (2 * i)) & 3u) << 4) |
                                (((l3 >> (2 * i)) & 3u) << 6);
          half |= byte << (8 * bb);
        }
        o[hw] = (uint16_t)half;
      }
    }
  }
  if (!live) return;
  {
    // hmask[m] bit t = high bit of element m + 32 t = element m % 16 of sub-block 2 t + (m >= 16); thread j writes m = 2j, 2j + 1
    uint32_t half = 0;
#pragma unroll
    for (int bb = 0; bb < 2; ++bb) {
      const int m = 2 * j + bb, par = m >> 4, ii = m & 15;
      uint32_t byte = 0;
#pragma unroll
      for (int t = 0; t < 8; ++t) byte |= ((hbv[2 * t + par] >> ii) & 1u) << t;
      half |= byte << (8 * bb);
    }
    reinterpret_cast<uint16_t*>(ob + Q3KL::kOffHmask)[j] = (uint16_t)half;
  }
  if (j < 12) {
    uint32_t byte;
    if (j < 8) {
      byte = (l6v[j] & 0xFu) | ((l6v[j + 8] & 0xFu) << 4);
    } else {
      const int i = j - 8;
      byte = ((l6v[i] >> 4) & 3u) | (((l6v[i + 4] >> 4) & 3u) << 2) | (((l6v[i + 8] >> 4) & 3u) << 4) | (((l6v[i + 12] >> 4) & 3u) << 6);
    }
    ob[Q3KL::kOffScales + j] = (uint8_t)byte;
  }
  if (j == 0) *reinterpret_cast<uint16_t*>(ob + Q3KL::kOffD) = __half_as_ushort(hd);
}

// ---------------------------------------------------------------- Q6_K: one thread per 16-element sub-block
// make_qx_quants(16, 32, x, L, rmse_type = 1, qw = null): weights x^2; returns the scale, levels in L[0..16) as 0..63
__device__ __forceinline__ float qw_make_qx16(const float (&x)[16], int (&L)[16]) {
  const int nmax = 32;
  float mx = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float ax = fabsf(x[i]);
    if (ax > amax) amax = ax, mx = x[i];
  }
  if (amax == 0.f) {
#pragma unroll
    for (int i = 0; i < 16; ++i) L[i] = 0;
    return 0.f;
  }
  float iscale = __fdiv_rn(-(float)nmax, mx);
  float sumlx = 0.f, suml2 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int l = qw_clamp(qw_nearest_int(__fmul_rn(iscale, x[i])), -nmax, nmax - 1);
    L[i] = l + nmax;
    const float w = __fmul_rn(x[i], x[i]);
    const float lf = (float)l;
    sumlx = __fadd_rn(sumlx, __fmul_rn(__fmul_rn(w, x[i]), lf));
    suml2 = __fadd_rn(suml2, __fmul_rn(__fmul_rn(w, lf), lf));
  }
  float scale = __fdiv_rn(sumlx, suml2);
  float best = __fmul_rn(scale, sumlx);
  for (int itry = 0; itry < 3; ++itry) {
    const float is2 = __fdiv_rn(1.0f, scale);
    float slx = 0.f, sl2 = 0.f;
    bool changed = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int l = qw_clamp(qw_nearest_int(__fmul_rn(is2, x[i])), -nmax, nmax - 1);
      if (l + nmax != L[i]) changed = true;
      const float w = __fmul_rn(x[i], x[i]);
      const float lf = (float)l;
      slx = __fadd_rn(slx, __fmul_rn(__fmul_rn(w, x[i]), lf));
      sl2 = __fadd_rn(sl2, __fmul_rn(__fmul_rn(w, lf), lf));
    }
    if (!changed || sl2 == 0.f || __fmul_rn(slx, slx) <= __fmul_rn(best, sl2)) break;
#pragma unroll
    for (int i = 0; i < 16; ++i) L[i] = nmax + qw_clamp(qw_nearest_int(__fmul_rn(is2, x[i])), -nmax, nmax - 1);
    sumlx = slx;
    suml2 = sl2;
    scale = __fdiv_rn(sumlx, suml2);
    best = __fmul_rn(scale, sumlx);
  }
  for (int itry = 0; itry < 5; ++itry) {
    int n_changed = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float w = __fmul_rn(x[i], x[i]);
      const int l = L[i] - nmax;
      float slx = __fsub_rn(sumlx, __fmul_rn(__fmul_rn(w, x[i]), (float)l));
      if (slx > 0.f) {
        float sl2 = __fsub_rn(suml2, __fmul_rn(__fmul_rn(w, (float)l), (float)l));
        const int nl = qw_clamp(qw_nearest_int(__fdiv_rn(__fmul_rn(x[i], sl2), slx)), -nmax, nmax - 1);
        if (nl != l) {
          slx = __fadd_rn(slx, __fmul_rn(__fmul_rn(w, x[i]), (float)nl));
          sl2 = __fadd_rn(sl2, __fmul_rn(__fmul_rn(w, (float)nl), (float)nl));
          if (sl2 > 0.f && __fmul_rn(__fmul_rn(slx, slx), suml2) > __fmul_rn(__fmul_rn(sumlx, sumlx), sl2)) {
            L[i] = nmax + nl;
            sumlx = slx;
            suml2 = sl2;
            scale = __fdiv_rn(sumlx, suml2);
            best = __fmul_rn(scale, sumlx);
            ++n_changed;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  return scale;
}

// blockDim.x = 128 threads = 8 super-blocks; levels staged in shared memory for packing
__global__ void __launch_bounds__(128) quantize_w_q6k_kernel(const float* __restrict__ x, int64_t nb,
                                                             uint8_t* __restrict__ out) {
  __shared__ uint8_t sL[8][256];
  const int64_t sub = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t blk = sub >> 4;
  const int s = (int)(sub & 15);
  const bool live = blk < nb;
  const unsigned lane = threadIdx.x & 31;
  const unsigned gbase = lane & ~15u;
  const unsigned gmask = 0xffffu << gbase;
  const int lb = threadIdx.x >> 4;  // super-block slot within the CTA
  float v[16];
  if (live) {
    const float4* src = reinterpret_cast<const float4*>(x + sub * 16);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float4 q = src[t];
      v[4 * t] = q.x, v[4 * t + 1] = q.y, v[4 * t + 2] = q.z, v[4 * t + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int t = 0; t < 16; ++t) v[t] = 0.f;
  }
  int L[16];
  const float scale = qw_make_qx16(v, L);
  // largest |scale|, first index wins on ties (strict '>' scan in index order)
  float best_abs = fabsf(scale), best_val = scale;
  int best_idx = s;
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) {
    const float oa = __shfl_xor_sync(gmask, best_abs, off);
    const float ov = __shfl_xor_sync(gmask, best_val, off);
    const int oi = __shfl_xor_sync(gmask, best_idx, off);
    if (oa > best_abs || (oa == best_abs && oi < best_idx)) best_abs = oa, best_val = ov, best_idx = oi;
  }
  // the scan starts from max_abs = 0 with strict '>': if every scale is 0 (or NaN) max_scale stays 0
  const float max_scale = best_abs > 0.f ? best_val : 0.f;
  const float iscale = __fdiv_rn(-128.0f, max_scale);
  const __half hd = __float2half_rn(__fdiv_rn(1.0f, iscale));
  const int ysc = (int)(int8_t)min(qw_nearest_int(__fmul_rn(iscale, scale)), 127);  // 'as i8' wraps below -128
  const float d = __fmul_rn(__half2float(hd), (float)ysc);
  if (d != 0.f) {
#pragma unroll
    for (int t = 0; t < 16; ++t) L[t] = qw_clamp(qw_nearest_int(__fdiv_rn(v[t], d)), -32, 31) + 32;
  }
#pragma unroll
  for (int t = 0; t < 16; ++t) sL[lb][16 * s + t] = (uint8_t)L[t];
  __syncthreads();
  if (!live) return;
  uint8_t* ob = out + blk * Q6KL::kBytes;
  // thread s packs l = 4*(s&7) .. +3 of half (s>>3): 4 bytes of ql (x2) and 4 bytes of qh
  const int half = s >> 3, l0 = 4 * (s & 7);
  const uint8_t* Lb = sL[lb] + 128 * half;
  uint32_t qa = 0, qb = 0, qh = 0;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const uint32_t a = Lb[l0 + t], b = Lb[l0 + t + 32], c = Lb[l0 + t + 64], e = Lb[l0 + t + 96];
    qa |= ((a & 0xF) | ((c & 0xF) << 4)) << (8 * t);
    qb |= ((b & 0xF) | ((e & 0xF) << 4)) << (8 * t);
    qh |= (((a >> 4) | ((b >> 4) << 2) | ((c >> 4) << 4) | ((e >> 4) << 6)) & 0xff) << (8 * t);
  }
  uint16_t* o16 = reinterpret_cast<uint16_t*>(ob);  // 210-byte blocks: 2-byte aligned
  const int wa = (Q6KL::kOffQl + 64 * half + l0) >> 1, wb = (Q6KL::kOffQl + 64 * half + 32 + l0) >> 1,
            wh = (Q6KL::kOffQh + 32 * half + l0) >> 1;
  o16[wa] = (uint16_t)qa, o16[wa + 1] = (uint16_t)(qa >> 16);
  o16[wb] = (uint16_t)qb, o16[wb + 1] = (uint16_t)(qb >> 16);
  o16[wh] = (uint16_t)qh, o16[wh + 1] = (uint16_t)(qh >> 16);
  // scales: thread s writes scale byte s (pairs through a shuffle to keep 16-bit stores)
  const int other = __shfl_xor_sync(gmask, ysc, 1);
  if ((s & 1) == 0) o16[(Q6KL::kOffScales + s) >> 1] = (uint16_t)((ysc & 0xff) | ((other & 0xff) << 8));
  if (s == 0) o16[Q6KL::kOffD >> 1] = __half_as_ushort(hd);
}

}  // namespace fq
