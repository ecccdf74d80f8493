// Block -> float dequantization (f32 / f16 / bf16 out), the exact arithmetic of the
// reference's to_float: Q4_K d1 = d*sc, y = d1*q - m1 with two roundings
// (fuel-quantized/src/k_quants.rs:1595-1622); Q6_K (d*sc)*q left to right (:2158-2189);
// Q8_0 q*d (:611-627); Q4_0 (nibble-8)*d (:177-197). Replaces the reference's
// per-format dequantize FFI calls (fuel-cuda-backend/src/quantized.rs:58-124).
// __fmul_rn / __fsub_rn keep the compiler from contracting into an fma.
#pragma once
#include <cuda_bf16.h>

#include "fq_common.cuh"

namespace fq {

template <typename T> __device__ __forceinline__ T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
// f16 whose finite values beyond the format's range saturate to +-65504 instead of becoming infinite: the form the
// tensor-core path multiplies with (an infinite operand would turn every zero activation into a NaN)
struct half_sat {
  uint16_t bits;
};
template <> __device__ __forceinline__ half_sat cvt_out<half_sat>(float v) {
  half_sat r;
  asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(r.bits) : "f"(v));
  return r;
}

// f32 rounded to tf32 (nearest, ties away: 10 mantissa bits kept): the tensor cores' tf32 operand, which would otherwise
// have its low 13 bits cut off
struct f32_tf32 {
  float v;
};
template <> __device__ __forceinline__ f32_tf32 cvt_out<f32_tf32>(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return f32_tf32{__uint_as_float(r)};
}
__device__ __forceinline__ float as_f32(float v) { return v; }
__device__ __forceinline__ float as_f32(f32_tf32 v) { return v.v; }

// N consecutive outputs (N = 4, 8 or 16) of one thread. With y 16-byte aligned (`vec`; every run then starts on a multiple
// of its own size) they leave as 8- or 16-byte stores instead of one store per element; the values are the same.
template <typename T, int N>
__device__ __forceinline__ void store_run(T* out, const float (&v)[N], bool vec) {
  if (!vec) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = cvt_out<T>(v[i]);
    return;
  }
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
      *reinterpret_cast<float4*>(out + i) = make_float4(as_f32(cvt_out<T>(v[i])), as_f32(cvt_out<T>(v[i + 1])),
                                                        as_f32(cvt_out<T>(v[i + 2])), as_f32(cvt_out<T>(v[i + 3])));
  } else {
    static_assert(sizeof(T) == 2, "16-bit outputs");
    uint32_t wd[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      const T a = cvt_out<T>(v[2 * i]), b = cvt_out<T>(v[2 * i + 1]);
      wd[i] = (uint32_t) * reinterpret_cast<const uint16_t*>(&a) | ((uint32_t) * reinterpret_cast<const uint16_t*>(&b) << 16);
    }
    if constexpr (N % 8 == 0) {
#pragma unroll
      for (int i = 0; i < N / 8; ++i)
        *reinterpret_cast<uint4*>(out + 8 * i) = make_uint4(wd[4 * i], wd[4 * i + 1], wd[4 * i + 2], wd[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < N / 4; ++i) *reinterpret_cast<uint2*>(out + 4 * i) = make_uint2(wd[2 * i], wd[2 * i + 1]);
    }
  }
}
__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
__device__ __forceinline__ uint32_t ldg_u32_2b(const uint8_t* p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }

// one thread per 16-byte nibble chunk: 16 low-nibble + 16 high-nibble elements
template <typename T>
__global__ void __launch_bounds__(256) dequant_q4k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 3;
  const int cc = (int)(u & 7), g = cc >> 1, h = cc & 1;
  const uint8_t* b = w + blk * Q4KL::kBytes;
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
  T* out = y + blk * 256 + 64 * g + 16 * h;
  const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
  float lo[16], hi[16];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const uint32_t byte = (qw[j] >> (8 * t)) & 0xff;
      lo[4 * j + t] = __fsub_rn(__fmul_rn(d1, (float)(byte & 0xF)), m1);
      hi[4 * j + t] = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
    }
  }
  const bool vec = aligned16(y);
  store_run<T, 16>(out, lo, vec);
  store_run<T, 16>(out + 32, hi, vec);
}

// Q5_K (fuel-quantized/src/k_quants.rs:1889-1923): Q4_K's layout and scale packing plus a fifth bit per element in qh —
// bit 2g of qh[t] for element 64g + t, bit 2g+1 for element 64g + 32 + t. One thread per 16-byte nibble chunk.
template <typename T>
__global__ void __launch_bounds__(256) dequant_q5k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 3;
  const int cc = (int)(u & 7), g = cc >> 1, h = cc & 1;
  const uint8_t* b = w + blk * Q5KL::kBytes;
  const uint4 hdr = *reinterpret_cast<const uint4*>(b);
  const uint4 hv = *reinterpret_cast<const uint4*>(b + Q5KL::kOffQh + 16 * h);
  const uint4 qv = *reinterpret_cast<const uint4*>(b + Q5KL::kOffQs + 16 * cc);
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
  T* out = y + blk * 256 + 64 * g + 16 * h;
  const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w}, hw[4] = {hv.x, hv.y, hv.z, hv.w};
  float vlo[16], vhi[16];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const uint32_t byte = (qw[j] >> (8 * t)) & 0xff, hb = (hw[j] >> (8 * t)) & 0xff;
      const uint32_t lo = (byte & 0xF) + (((hb >> (2 * g)) & 1u) << 4), hi = (byte >> 4) + (((hb >> (2 * g + 1)) & 1u) << 4);
      vlo[4 * j + t] = __fsub_rn(__fmul_rn(d1, (float)lo), m1);
      vhi[4 * j + t] = __fsub_rn(__fmul_rn(d2, (float)hi), m2);
    }
  }
  const bool vec = aligned16(y);
  store_run<T, 16>(out, vlo, vec);
  store_run<T, 16>(out + 32, vhi, vec);
}

// one thread per four consecutive l of one 128-half: 16 elements
template <typename T>
__global__ void __launch_bounds__(256) dequant_q6k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 4;
  const int uu = (int)(u & 15), half = uu >> 3, l0 = (uu & 7) * 4;
  const uint8_t* b = w + blk * Q6KL::kBytes;
  const uint32_t ql_a = ldg_u32_2b(b + Q6KL::kOffQl + 64 * half + l0);
  const uint32_t ql_b = ldg_u32_2b(b + Q6KL::kOffQl + 64 * half + 32 + l0);
  const uint32_t qh = ldg_u32_2b(b + Q6KL::kOffQh + 32 * half + l0);
  const float d = h2f_bits(ldg_u16(b + Q6KL::kOffD));
  const int8_t* scp = reinterpret_cast<const int8_t*>(b + Q6KL::kOffScales + 8 * half + (l0 >> 4));
  const float s[4] = {__fmul_rn(d, (float)scp[0]), __fmul_rn(d, (float)scp[2]), __fmul_rn(d, (float)scp[4]),
                      __fmul_rn(d, (float)scp[6])};
  T* out = y + blk * 256 + 128 * half + l0;
  float v1[4], v2[4], v3[4], v4[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int a = (ql_a >> (8 * t)) & 0xff, c = (ql_b >> (8 * t)) & 0xff, hh = (qh >> (8 * t)) & 0xff;
    const int q1 = ((a & 0xF) | ((hh & 3) << 4)) - 32;
    const int q2 = ((c & 0xF) | (((hh >> 2) & 3) << 4)) - 32;
    const int q3 = ((a >> 4) | (((hh >> 4) & 3) << 4)) - 32;
    const int q4 = ((c >> 4) | (((hh >> 6) & 3) << 4)) - 32;
    v1[t] = __fmul_rn(s[0], (float)q1);
    v2[t] = __fmul_rn(s[1], (float)q2);
    v3[t] = __fmul_rn(s[2], (float)q3);
    v4[t] = __fmul_rn(s[3], (float)q4);
  }
  const bool vec = aligned16(y);
  store_run<T, 4>(out, v1, vec);
  store_run<T, 4>(out + 32, v2, vec);
  store_run<T, 4>(out + 64, v3, vec);
  store_run<T, 4>(out + 96, v4, vec);
}

// one thread per 8 elements of a 32-block (4 threads per block)
template <typename T>
__global__ void __launch_bounds__(256) dequant_q8_0_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 2;
  const int part = (int)(u & 3);
  const uint8_t* b = w + blk * Q8_0L::kBytes;
  const float d = h2f_bits(ldg_u16(b));
  T* out = y + blk * 32 + 8 * part;
  float o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t v = ldg_u16(b + Q8_0L::kOffQs + 8 * part + 2 * j);
    o[2 * j] = __fmul_rn((float)(int8_t)(v & 0xff), d);
    o[2 * j + 1] = __fmul_rn((float)(int8_t)(v >> 8), d);
  }
  store_run<T, 8>(out, o, aligned16(y));
}

// one thread per 4 bytes of nibbles: elements 4p..4p+3 and 16+4p..
template <typename T>
__global__ void __launch_bounds__(256) dequant_q4_0_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 2;
  const int part = (int)(u & 3);
  const uint8_t* b = w + blk * Q4_0L::kBytes;
  const float d = h2f_bits(ldg_u16(b));
  const uint32_t v = ldg_u32_2b(b + Q4_0L::kOffQs + 4 * part);
  T* out = y + blk * 32 + 4 * part;
  float lo[4], hi[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int byte = (v >> (8 * t)) & 0xff;
    lo[t] = __fmul_rn((float)((byte & 0xF) - 8), d);
    hi[t] = __fmul_rn((float)((byte >> 4) - 8), d);
  }
  const bool vec = aligned16(y);
  store_run<T, 4>(out, lo, vec);
  store_run<T, 4>(out + 16, hi, vec);
}

// Q4_1 / Q5_0 / Q5_1 (k_quants.rs:354-374, 463-485, 578-602): one thread per 4 bytes of nibbles, elements 4p..4p+3
// and 16+4p..; q*d + m as a product and a sum (two roundings), (q - 16)*d for Q5_0
template <typename T, class L, bool kFive, bool kMin>
__global__ void __launch_bounds__(256) dequant_legacy32_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 2;
  const int part = (int)(u & 3);
  const uint8_t* b = w + blk * L::kBytes;
  const float d = h2f_bits(ldg_u16(b));
  const float m = kMin ? h2f_bits(ldg_u16(b + 2)) : 0.f;
  const uint32_t qh = kFive ? ldg_u32_2b(b + L::kBytes - 20) : 0u;
  const uint32_t v = ldg_u32_2b(b + L::kBytes - 16 + 4 * part);
  T* out = y + blk * 32 + 4 * part;
  float lo[4], hi[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int byte = (v >> (8 * t)) & 0xff, j = 4 * part + t;
    int q0 = byte & 0xF, q1 = byte >> 4;
    if (kFive) q0 |= (int)((qh >> j) & 1u) << 4, q1 |= (int)((qh >> (j + 16)) & 1u) << 4;
    if (kFive && !kMin) q0 -= 16, q1 -= 16;
    const float p0 = __fmul_rn((float)q0, d), p1 = __fmul_rn((float)q1, d);
    lo[t] = kMin ? __fadd_rn(p0, m) : p0;
    hi[t] = kMin ? __fadd_rn(p1, m) : p1;
  }
  const bool vec = aligned16(y);
  store_run<T, 4>(out, lo, vec);
  store_run<T, 4>(out + 16, hi, vec);
}
// Q2_K (k_quants.rs:958-994): y = (d * sc_lo) * q - dmin * sc_hi; Q3_K (:1314-1366): y = (d * (sc - 32)) * q with
// q = low two bits - (high bit set ? 0 : 4). One thread per 4 bytes of qs of one bit pair: 4 elements.
template <typename T>
__global__ void __launch_bounds__(256) dequant_q2k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 6;
  const int e0 = (int)(u & 63) * 4;                       // first of four consecutive elements
  const int c = e0 >> 7, j = (e0 >> 5) & 3, bb = e0 & 31;  // chunk, bit pair, byte within the chunk's 32
  const uint8_t* b = w + blk * Q2KL::kBytes;
  const float d = h2f_bits(ldg_u16(b + Q2KL::kOffD)), mn = h2f_bits(ldg_u16(b + Q2KL::kOffDmin));
  const uint32_t sc = b[e0 >> 4];
  const float dl = __fmul_rn(d, (float)(sc & 0xFu)), ml = __fmul_rn(mn, (float)(sc >> 4));
  const uint32_t v = ldg_u32_2b(b + Q2KL::kOffQs + 32 * c + bb);
  T* out = y + blk * 256 + e0;
  float o[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) o[t] = __fsub_rn(__fmul_rn(dl, (float)((v >> (8 * t + 2 * j)) & 3u)), ml);
  store_run<T, 4>(out, o, aligned16(y));
}
template <typename T>
__global__ void __launch_bounds__(256) dequant_q3k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 6;
  const int e0 = (int)(u & 63) * 4;
  const int c = e0 >> 7, j = (e0 >> 5) & 3, bb = e0 & 31, is = e0 >> 4;
  const uint8_t* b = w + blk * Q3KL::kBytes;
  const float d = h2f_bits(ldg_u16(b + Q3KL::kOffD));
  const uint32_t lo = is < 8 ? (b[Q3KL::kOffScales + is] & 0xFu) : (uint32_t)(b[Q3KL::kOffScales + is - 8] >> 4);
  const uint32_t hi = (b[Q3KL::kOffScales + 8 + (is & 3)] >> (2 * (is >> 2))) & 3u;
  const float dl = __fmul_rn(d, __fsub_rn((float)(int8_t)(lo | (hi << 4)), 32.0f));
  const uint32_t v = ldg_u32_2b(b + Q3KL::kOffQs + 32 * c + bb), hm = ldg_u32_2b(b + Q3KL::kOffHmask + bb);
  T* out = y + blk * 256 + e0;
  float o[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int q = (int)((v >> (8 * t + 2 * j)) & 3u) - (((hm >> (8 * t + 4 * c + j)) & 1u) ? 0 : 4);
    o[t] = __fmul_rn(dl, (float)q);
  }
  store_run<T, 4>(out, o, aligned16(y));
}

// Q8_K blocks back to f32 (x.d * q, k_quants.rs:2269-2280); one thread per 4 elements
template <typename T>
__global__ void __launch_bounds__(256) dequant_q8k_kernel(const uint8_t* __restrict__ w, int64_t n_units, T* __restrict__ y) {
  const int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_units) return;
  const int64_t blk = u >> 6;
  const int part = (int)(u & 63);
  const uint8_t* b = w + blk * Q8KL::kBytes;
  const float d = *reinterpret_cast<const float*>(b);
  const uint32_t v = *reinterpret_cast<const uint32_t*>(b + Q8KL::kOffQs + 4 * part);
  T* out = y + blk * 256 + 4 * part;
  float o[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) o[t] = __fmul_rn(d, (float)(int8_t)((v >> (8 * t)) & 0xff));
  store_run<T, 4>(out, o, aligned16(y));
}

}  // namespace fq
