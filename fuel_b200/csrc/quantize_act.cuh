// Activation quantization: f32 rows -> Q8_K (256-element blocks, for k-quant weights) or
// Q8_0 (32-element blocks), bit-for-bit what the reference's CPU path produces
// (BlockQ8K::from_float, fuel-quantized/src/k_quants.rs:2230-2267;
//  BlockQ8_0::from_float, k_quants.rs:629-658).
//
// One warp per 256 consecutive elements. Two outputs from the same arithmetic:
// the reference's block byte layout (public entry point, parity-tested byte for byte)
// and the plane-split layout the mat-vec kernels read (fq_common.cuh, ActPlanes).
//
// Bit-exactness notes:
//  * round() is half-away-from-zero (roundf), never rint;
//  * the reference scans left to right with a strict '<', so among equal magnitudes
//    the lowest index wins and its sign fixes the sign of the scale — the warp
//    reduction carries (|x|, index) and breaks ties toward the lower index;
//  * plain '/' and '*' (IEEE, no fast-math, nothing here can contract into an fma);
//  * float -> int conversion saturates and maps NaN to 0 on both sides.
#pragma once
#include "fq_common.cuh"

namespace fq {

// One warp quantizes one 256-element block held as e[0..3] = elements 4*lane.., e[4..7] = elements
// 128 + 4*lane..; writes the plane-split layout. Shared by the stand-alone kernel and by the fused
// producers (norm / SwiGLU / attention merge) so all of them emit identical bytes.
struct Q8KLaneBlock {
  uint32_t p0, p1;  // this lane's eight quants, packed
  float d;
  int s0, s1;       // sums of the 16-element groups this lane belongs to (valid in every lane of the group)
};

__device__ __forceinline__ Q8KLaneBlock q8k_block_quantize(const float (&e)[8], int lane) {
  float amax = 0.f, smax = 0.f;
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = fabsf(e[i]);
    if (amax < a) {
      amax = a;
      smax = e[i];
      idx = (i < 4 ? 4 * lane + i : 128 + 4 * lane + (i - 4));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
    const float os = __shfl_xor_sync(0xffffffffu, smax, off);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
    if (oa > amax || (oa == amax && oi < idx)) {
      amax = oa;
      smax = os;
      idx = oi;
    }
  }
  int q[8];
  float d;
  if (amax == 0.f) {
    d = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
  } else {
    const float iscale = -128.0f / smax;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float r = fminf(roundf(iscale * e[i]), 127.0f);
      q[i] = max(__float2int_rz(r), -128);
    }
    d = 1.0f / iscale;
  }
  int s0 = q[0] + q[1] + q[2] + q[3];
  int s1 = q[4] + q[5] + q[6] + q[7];
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
  s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
  const uint32_t p0 = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
                      ((uint32_t)(q[3] & 0xff) << 24);
  const uint32_t p1 = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) |
                      ((uint32_t)(q[7] & 0xff) << 24);
  Q8KLaneBlock b;
  b.p0 = p0, b.p1 = p1, b.d = d, b.s0 = s0, b.s1 = s1;
  return b;
}

__device__ __forceinline__ void q8k_block_store(const Q8KLaneBlock& b, int lane, int64_t blk, int8_t* out_qs,
                                                float* out_d, int16_t* out_bsums) {
  uint32_t* qs = reinterpret_cast<uint32_t*>(out_qs + blk * QK_K);
  qs[lane] = b.p0;
  qs[32 + lane] = b.p1;
  if (lane == 0) out_d[blk] = b.d;
  if ((lane & 3) == 0) {
    out_bsums[blk * 16 + (lane >> 2)] = (int16_t)b.s0;
    out_bsums[blk * 16 + 8 + (lane >> 2)] = (int16_t)b.s1;
  }
}

__device__ __forceinline__ void q8k_block_from_regs(const float (&e)[8], int lane, int64_t blk, int8_t* out_qs,
                                                    float* out_d, int16_t* out_bsums) {
  q8k_block_store(q8k_block_quantize(e, lane), lane, blk, out_qs, out_d, out_bsums);
}

template <bool kRefLayout>
__global__ void __launch_bounds__(256) quantize_q8k_kernel(const float* x, int64_t n_blocks,
                                                           uint8_t* out_ref, int8_t* out_qs,
                                                           float* out_d, int16_t* out_bsums, unsigned* zero_word,
                                                           int early_x) {
  // early_x: x does not come from an earlier kernel of the stream (host data, final when the call was made), so it is
  // loaded before the wait for the predecessors and only the stores are ordered after them: a slow read (host memory
  // over PCIe) then runs beside the previous kernels.
  pdl_launch_dependents();
  if (!early_x) pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (blk >= n_blocks) return;
  const float4* src = reinterpret_cast<const float4*>(x + blk * QK_K);
  const float4 v0 = src[lane];       // elements 4*lane .. 4*lane+3
  const float4 v1 = src[32 + lane];  // elements 128 + 4*lane ..
  const float e[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  if (early_x) pdl_wait();
  if (zero_word && blockIdx.x == 0 && threadIdx.x == 0) *zero_word = 0u;  // a counter the next kernel starts from

  // first-max-wins scan, in index order within the lane
  float amax = 0.f, smax = 0.f;
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = fabsf(e[i]);
    if (amax < a) {
      amax = a;
      smax = e[i];
      idx = (i < 4 ? 4 * lane + i : 128 + 4 * lane + (i - 4));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
    const float os = __shfl_xor_sync(0xffffffffu, smax, off);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
    if (oa > amax || (oa == amax && oi < idx)) {
      amax = oa;
      smax = os;
      idx = oi;
    }
  }

  int q[8];
  float d;
  if (amax == 0.f) {
    d = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
  } else {
    const float iscale = -128.0f / smax;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float r = fminf(roundf(iscale * e[i]), 127.0f);
      q[i] = max(__float2int_rz(r), -128);
    }
    d = 1.0f / iscale;
  }
  // sums of 16 consecutive values = 4 neighbouring lanes x 4 values
  int s0 = q[0] + q[1] + q[2] + q[3];
  int s1 = q[4] + q[5] + q[6] + q[7];
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
  s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 2);

  const uint32_t p0 = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
                      ((uint32_t)(q[3] & 0xff) << 24);
  const uint32_t p1 = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) |
                      ((uint32_t)(q[7] & 0xff) << 24);
  if (kRefLayout) {
    uint8_t* b = out_ref + blk * Q8KL::kBytes;  // 292-byte blocks are 4-byte aligned
    if (lane == 0) *reinterpret_cast<float*>(b + Q8KL::kOffD) = d;
    uint32_t* qs = reinterpret_cast<uint32_t*>(b + Q8KL::kOffQs);
    qs[lane] = p0;
    qs[32 + lane] = p1;
    int16_t* bs = reinterpret_cast<int16_t*>(b + Q8KL::kOffBsums);
    if ((lane & 3) == 0) {
      bs[lane >> 2] = (int16_t)s0;
      bs[8 + (lane >> 2)] = (int16_t)s1;
    }
  } else {
    uint32_t* qs = reinterpret_cast<uint32_t*>(out_qs + blk * QK_K);
    qs[lane] = p0;
    qs[32 + lane] = p1;
    if (lane == 0) out_d[blk] = d;
    if ((lane & 3) == 0) {
      out_bsums[blk * 16 + (lane >> 2)] = (int16_t)s0;
      out_bsums[blk * 16 + 8 + (lane >> 2)] = (int16_t)s1;
    }
  }
}

// One warp per 256 elements = eight Q8_0 blocks; a block is 8 neighbouring lanes of one half.
// kQ81: Q8_1 blocks instead (BlockQ8_1::from_float, k_quants.rs:728-757): the same d and quants, plus
// s = f16(sum of the quants) * d in half arithmetic (both factors f16, their f32 product rounded to f16); 36-byte
// blocks {d, s, qs} in the reference layout, or a third plane out_s (f32) beside qs and d.
template <bool kRefLayout, bool kQ81 = false>
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float* x, int64_t n_groups /* of 256 */,
                                                            int64_t n_blocks32, uint8_t* out_ref,
                                                            int8_t* out_qs, float* out_d, unsigned* zero_word,
                                                            int early_x, float* out_s = nullptr) {
  pdl_launch_dependents();
  if (!early_x) pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t grp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (grp >= n_groups) return;
  // the last group may be partial when k is a multiple of 32 but not of 256
  const int64_t base = grp * QK_K;
  const int64_t blk0 = grp * 8 + (lane >> 3);  // first half: elements 4*lane.. belong to block lane/8
  const int64_t blk1 = blk0 + 4;
  const bool ok0 = blk0 < n_blocks32, ok1 = blk1 < n_blocks32;
  const float4* src = reinterpret_cast<const float4*>(x + base);
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 v0 = ok0 ? src[lane] : z;
  const float4 v1 = ok1 ? src[32 + lane] : z;
  if (early_x) pdl_wait();
  if (zero_word && blockIdx.x == 0 && threadIdx.x == 0) *zero_word = 0u;
  float a0 = fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w)));
  float a1 = fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w)));
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) {
    a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, off));
    a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, off));
  }
  const float d0 = a0 / 127.0f, d1 = a1 / 127.0f;
  const float id0 = d0 != 0.f ? 1.0f / d0 : 0.f;
  const float id1 = d1 != 0.f ? 1.0f / d1 : 0.f;
  auto qz = [](float v, float id) -> uint32_t {
    int r = __float2int_rz(roundf(v * id));
    r = min(max(r, -128), 127);
    return (uint32_t)(r & 0xff);
  };
  const uint32_t p0 = qz(v0.x, id0) | (qz(v0.y, id0) << 8) | (qz(v0.z, id0) << 16) | (qz(v0.w, id0) << 24);
  const uint32_t p1 = qz(v1.x, id1) | (qz(v1.y, id1) << 8) | (qz(v1.z, id1) << 16) | (qz(v1.w, id1) << 24);
  const __half h0 = __float2half_rn(d0), h1 = __float2half_rn(d1);
  const int sub = lane & 7;
  if constexpr (kQ81) {
    int s0 = __dp4a((int)p0, 0x01010101, 0), s1 = __dp4a((int)p1, 0x01010101, 0);  // sum of the four signed quants
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
      s0 += __shfl_xor_sync(0xffffffffu, s0, off);
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
    }
    // (a block whose scale overflows f16 and whose quants sum to zero gives 0 * inf: the reference's x86 build stores
    // the default NaN of that product, sign bit set, 0xFE00 as f16)
    auto s_field = [](int sum, __half d) -> __half {
      const float prod = __half2float(__float2half_rn((float)sum)) * __half2float(d);
      return prod != prod ? __ushort_as_half((unsigned short)0xFE00u) : __float2half_rn(prod);
    };
    const __half sh0 = s_field(s0, h0), sh1 = s_field(s1, h1);
    if (kRefLayout) {  // 36-byte blocks are 4-byte aligned
      if (ok0) {
        uint32_t* b = reinterpret_cast<uint32_t*>(out_ref + blk0 * Q8_1L::kBytes);
        if (sub == 0) b[0] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(sh0) << 16);
        b[1 + sub] = p0;
      }
      if (ok1) {
        uint32_t* b = reinterpret_cast<uint32_t*>(out_ref + blk1 * Q8_1L::kBytes);
        if (sub == 0) b[0] = (uint32_t)__half_as_ushort(h1) | ((uint32_t)__half_as_ushort(sh1) << 16);
        b[1 + sub] = p1;
      }
    } else {
      uint32_t* qs = reinterpret_cast<uint32_t*>(out_qs + base);
      if (ok0) {
        qs[lane] = p0;
        if (sub == 0) out_d[blk0] = __half2float(h0), out_s[blk0] = __half2float(sh0);
      }
      if (ok1) {
        qs[32 + lane] = p1;
        if (sub == 0) out_d[blk1] = __half2float(h1), out_s[blk1] = __half2float(sh1);
      }
    }
    return;
  }
  if (kRefLayout) {
    // 34-byte blocks: 2-byte aligned only -> 16-bit stores
    if (ok0) {
      uint16_t* b = reinterpret_cast<uint16_t*>(out_ref + blk0 * Q8_0L::kBytes);
      if (sub == 0) b[0] = __half_as_ushort(h0);
      b[1 + 2 * sub] = (uint16_t)(p0 & 0xffff);
      b[2 + 2 * sub] = (uint16_t)(p0 >> 16);
    }
    if (ok1) {
      uint16_t* b = reinterpret_cast<uint16_t*>(out_ref + blk1 * Q8_0L::kBytes);
      if (sub == 0) b[0] = __half_as_ushort(h1);
      b[1 + 2 * sub] = (uint16_t)(p1 & 0xffff);
      b[2 + 2 * sub] = (uint16_t)(p1 >> 16);
    }
  } else {
    uint32_t* qs = reinterpret_cast<uint32_t*>(out_qs + base);
    if (ok0) {
      qs[lane] = p0;
      if (sub == 0) out_d[blk0] = __half2float(h0);
    }
    if (ok1) {
      qs[32 + lane] = p1;
      if (sub == 0) out_d[blk1] = __half2float(h1);
    }
  }
}

}  // namespace fq
