// TEST INFRASTRUCTURE — not part of the shipped library.
//
// The dot products in the summation order the reference runs on an x86 host
// built with target-cpu=native: per block an explicit fused multiply-add into
// eight f32 lanes, then a fixed horizontal reduction. This is the order the
// timed CPU baseline uses; it differs from the scalar order only in f32
// rounding of the running sums.
//
// Follows fuel-quantized/src/avx.rs:13-48 (helpers), :51-88 (Q4_0, Q8_0), :92-243 (Q4_1, Q5_0, Q5_1), :380-596 (Q2_K, Q3_K),
// :287-372 (Q6_K), :599-681 (Q4_K).
#include "blocks.h"

#include <immintrin.h>

#include <cstring>

namespace fq_oracle {

// ((hi128 + lo128) -> (r0+r2, r1+r3) -> r0+r1), avx.rs:27-33
static inline float reduce8(__m256 v) {
  __m128 r = _mm_add_ps(_mm256_extractf128_ps(v, 1), _mm256_castps256_ps128(v));
  r = _mm_add_ps(r, _mm_movehl_ps(r, r));
  r = _mm_add_ss(r, _mm_movehdup_ps(r));
  return _mm_cvtss_f32(r);
}

// signed i8 x signed i8, adjacent groups of four summed to i32 then converted;
// |x| * sign-adjusted y keeps maddubs' unsigned-by-signed form exact, avx.rs:14-24,44-48
static inline __m256 dot_i8_quads(__m256i x, __m256i y) {
  const __m256i ax = _mm256_sign_epi8(x, x);
  const __m256i sy = _mm256_sign_epi8(y, x);
  const __m256i p16 = _mm256_maddubs_epi16(ax, sy);
  return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_set1_epi16(1), p16));
}

// avx.rs:51-69
float q4_0_q8_0_dot_avx2(int64_t n, const BlkQ4_0* xs, const BlkQ8_0* ys) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const __m256 d = _mm256_set1_ps(h2f(xs[b].d) * h2f(ys[b].d));
    const __m128i raw = _mm_loadu_si128((const __m128i*)xs[b].qs);
    __m256i nib = _mm256_insertf128_si256(_mm256_castsi128_si256(raw), _mm_srli_epi16(raw, 4), 1);
    nib = _mm256_and_si256(_mm256_set1_epi8(0xF), nib);
    nib = _mm256_sub_epi8(nib, _mm256_set1_epi8(8));
    const __m256i qy = _mm256_loadu_si256((const __m256i*)ys[b].qs);
    acc = _mm256_fmadd_ps(d, dot_i8_quads(nib, qy), acc);
  }
  return reduce8(acc);
}

// avx.rs:72-88
float q8_0_q8_0_dot_avx2(int64_t n, const BlkQ8_0* xs, const BlkQ8_0* ys) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const __m256 d = _mm256_set1_ps(h2f(xs[b].d) * h2f(ys[b].d));
    const __m256i qx = _mm256_loadu_si256((const __m256i*)xs[b].qs);
    const __m256i qy = _mm256_loadu_si256((const __m256i*)ys[b].qs);
    acc = _mm256_fmadd_ps(d, dot_i8_quads(qx, qy), acc);
  }
  return reduce8(acc);
}

// unsigned u8 x signed i8, adjacent groups of four summed to i32 then converted, avx.rs:14-24
static inline __m256 dot_u8_quads(__m256i ux, __m256i y) {
  const __m256i p16 = _mm256_maddubs_epi16(ux, y);
  return _mm256_cvtepi32_ps(_mm256_madd_epi16(_mm256_set1_epi16(1), p16));
}
// 16 bytes of nibbles -> 32 bytes: low nibbles (elements 0..15), then high nibbles (16..31), avx.rs:36-41
static inline __m256i nibbles32(const uint8_t* qs) {
  const __m128i raw = _mm_loadu_si128((const __m128i*)qs);
  const __m256i b = _mm256_insertf128_si256(_mm256_castsi128_si256(raw), _mm_srli_epi16(raw, 4), 1);
  return _mm256_and_si256(_mm256_set1_epi8(0xF), b);
}
// bit i of the 32-bit word -> 0x10 in byte i (the fifth bit of element i), avx.rs:92-124
static inline __m256i fifth_bits32(const uint8_t* qh) {
  uint8_t b[32];
  const uint32_t w = (uint32_t)qh[0] | ((uint32_t)qh[1] << 8) | ((uint32_t)qh[2] << 16) | ((uint32_t)qh[3] << 24);
  for (int i = 0; i < 32; ++i) b[i] = (uint8_t)(((w >> i) & 1u) << 4);
  return _mm256_loadu_si256((const __m256i*)b);
}

// avx.rs:148-173
float q4_1_q8_1_dot_avx2(int64_t n, const BlkQ4_1* xs, const BlkQ8_1* ys) {
  __m256 acc = _mm256_setzero_ps();
  float summs = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const __m256 d = _mm256_set1_ps(h2f(xs[b].d) * h2f(ys[b].d));
    summs += h2f(xs[b].m) * h2f(ys[b].s);
    acc = _mm256_fmadd_ps(d, dot_u8_quads(nibbles32(xs[b].qs), _mm256_loadu_si256((const __m256i*)ys[b].qs)), acc);
  }
  return reduce8(acc) + summs;
}
// avx.rs:176-209
float q5_0_q8_0_dot_avx2(int64_t n, const BlkQ5_0* xs, const BlkQ8_0* ys) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const __m256 d = _mm256_set1_ps(h2f(xs[b].d) * h2f(ys[b].d));
    __m256i q = _mm256_or_si256(nibbles32(xs[b].qs), fifth_bits32(xs[b].qh));
    q = _mm256_sub_epi8(q, _mm256_set1_epi8(16));
    acc = _mm256_fmadd_ps(d, dot_i8_quads(q, _mm256_loadu_si256((const __m256i*)ys[b].qs)), acc);
  }
  return reduce8(acc);
}
// avx.rs:212-243
float q5_1_q8_1_dot_avx2(int64_t n, const BlkQ5_1* xs, const BlkQ8_1* ys) {
  __m256 acc = _mm256_setzero_ps();
  float summs = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const __m256 d = _mm256_set1_ps(h2f(xs[b].d) * h2f(ys[b].d));
    summs += h2f(xs[b].m) * h2f(ys[b].s);
    const __m256i q = _mm256_or_si256(nibbles32(xs[b].qs), fifth_bits32(xs[b].qh));
    acc = _mm256_fmadd_ps(d, dot_u8_quads(q, _mm256_loadu_si256((const __m256i*)ys[b].qs)), acc);
  }
  return reduce8(acc) + summs;
}

// Q2_K and Q3_K in the AVX2 order (avx.rs:380-455, 463-596). Both build, per block, eight i32 lanes: the 32 bytes of
// a quant register cover elements b = 0..31 of a 32-element group, adjacent bytes are paired and adjacent pairs
// added, so lane u holds bytes 4u..4u+3 (lanes 0-3: the group's first 16-element scale, lanes 4-7: its second), summed
// over the eight groups of the block; then one fused multiply-add of the block scale into eight f32 lanes.
static inline __m256 lanes_to_ps(const int32_t (&v)[8]) {
  return _mm256_cvtepi32_ps(_mm256_loadu_si256((const __m256i*)v));
}
float q2k_q8k_dot_avx2(int64_t n, const BlkQ2K* xs, const BlkQ8K* ys) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ2K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    const float d = y.d * h2f(x.d), dmin = -y.d * h2f(x.dmin);
    int32_t mins[8], sumi[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int u = 0; u < 8; ++u)
      mins[u] = (int32_t)(x.scales[2 * u] >> 4) * y.bsums[2 * u] + (int32_t)(x.scales[2 * u + 1] >> 4) * y.bsums[2 * u + 1];
    acc = _mm256_fmadd_ps(_mm256_set1_ps(dmin), lanes_to_ps(mins), acc);
    for (int g = 0; g < 8; ++g)       // 32-element groups: chunk g / 4, bit pair g % 4
      for (int b = 0; b < 32; ++b) {
        const int q = (x.qs[32 * (g / 4) + b] >> (2 * (g % 4))) & 3;
        sumi[b / 4] += (int32_t)(x.scales[2 * g + b / 16] & 0xF) * q * (int32_t)y.qs[32 * g + b];
      }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), lanes_to_ps(sumi), acc);
  }
  return reduce8(acc);
}
float q3k_q8k_dot_avx2(int64_t n, const BlkQ3K* xs, const BlkQ8K* ys) {
  __m256 acc = _mm256_setzero_ps();
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ3K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    const float d = y.d * h2f(x.d);
    uint32_t a[3];
    std::memcpy(a, x.scales, 12);
    const uint32_t m1 = 0x03030303u, m2 = 0x0f0f0f0fu;
    const uint32_t w[4] = {(a[0] & m2) | ((a[2] & m1) << 4), (a[1] & m2) | (((a[2] >> 2) & m1) << 4),
                           ((a[0] >> 4) & m2) | (((a[2] >> 4) & m1) << 4), ((a[1] >> 4) & m2) | (((a[2] >> 6) & m1) << 4)};
    int8_t sc[16];
    std::memcpy(sc, w, 16);
    int32_t sumi[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int g = 0; g < 8; ++g)
      for (int b = 0; b < 32; ++b) {
        const int low = (x.qs[32 * (g / 4) + b] >> (2 * (g % 4))) & 3;
        const int q = low - (((x.hmask[b] >> g) & 1) ? 0 : 4);
        sumi[b / 4] += ((int32_t)sc[2 * g + b / 16] - 32) * q * (int32_t)y.qs[32 * g + b];
      }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), lanes_to_ps(sumi), acc);
  }
  return reduce8(acc);
}

// Broadcast scale pair (2j, 2j+1 as 16-bit words) across a 256-bit register:
// entry i of the 16 words holds 16-bit word number `w` of `src` — the effect of
// the reference's shuffle table, avx.rs:257-272.
static inline __m256i bcast_word(__m256i src, int w) {
  const __m256i idx = _mm256_set1_epi16((short)(((2 * w + 1) << 8) | (2 * w)));
  return _mm256_shuffle_epi8(src, idx);
}

// avx.rs:599-681
float q4k_q8k_dot_avx2(int64_t n, const BlkQ4K* xs, const BlkQ8K* ys) {
  const __m256i low4 = _mm256_set1_epi8(0xF);
  __m256 acc = _mm256_setzero_ps();
  __m128 acc_m = _mm_setzero_ps();
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ4K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    const float d = y.d * h2f(x.d);
    const float dmin = -y.d * h2f(x.dmin);

    uint32_t u[4];
    std::memcpy(u, x.scales, 12);
    u[3] = ((u[2] >> 4) & 0x0f0f0f0fu) | (((u[1] >> 6) & 0x03030303u) << 4);
    const uint32_t keep = u[1] & 0x3f3f3f3fu;
    u[1] = (u[2] & 0x0f0f0f0fu) | (((u[0] >> 6) & 0x03030303u) << 4);
    u[2] = keep;
    u[0] &= 0x3f3f3f3fu;
    // words 0..7 = the eight scales, words 8..15 = the eight mins
    const __m256i sc_mn = _mm256_cvtepu8_epi16(_mm_set_epi32((int)u[3], (int)u[2], (int)u[1], (int)u[0]));

    const __m256i bs = _mm256_loadu_si256((const __m256i*)y.bsums);
    const __m128i pair_sums = _mm_hadd_epi16(_mm256_extracti128_si256(bs, 0), _mm256_extracti128_si256(bs, 1));
    const __m128i mprod = _mm_madd_epi16(_mm256_extracti128_si256(sc_mn, 1), pair_sums);
    acc_m = _mm_fmadd_ps(_mm_set1_ps(dmin), _mm_cvtepi32_ps(mprod), acc_m);

    const __m128i sc128 = _mm256_extracti128_si256(sc_mn, 0);
    const __m256i scales = _mm256_insertf128_si256(_mm256_castsi128_si256(sc128), sc128, 1);

    __m256i sumi = _mm256_setzero_si256();
    const uint8_t* q4 = x.qs;
    const int8_t* q8 = y.qs;
    for (int j = 0; j < QK_K / 64; ++j) {
      const __m256i s_lo = bcast_word(scales, 2 * j);
      const __m256i s_hi = bcast_word(scales, 2 * j + 1);
      const __m256i bits = _mm256_loadu_si256((const __m256i*)q4);
      q4 += 32;
      const __m256i lo = _mm256_and_si256(bits, low4);
      const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(bits, 4), low4);
      const __m256i y_lo = _mm256_loadu_si256((const __m256i*)q8);
      q8 += 32;
      sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(s_lo, _mm256_maddubs_epi16(lo, y_lo)));
      const __m256i y_hi = _mm256_loadu_si256((const __m256i*)q8);
      q8 += 32;
      sumi = _mm256_add_epi32(sumi, _mm256_madd_epi16(s_hi, _mm256_maddubs_epi16(hi, y_hi)));
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
  }
  acc_m = _mm_add_ps(acc_m, _mm_movehl_ps(acc_m, acc_m));
  acc_m = _mm_add_ss(acc_m, _mm_movehdup_ps(acc_m));
  return reduce8(acc) + _mm_cvtss_f32(acc_m);
}

// avx.rs:684-793: as Q4_K's, with the fifth bits merged in before the multiply, and the mins term kept as one scalar
// f32 sum (dmin * the block's integer total) instead of four lanes.
float q5k_q8k_dot_avx2(int64_t n, const BlkQ5K* xs, const BlkQ8K* ys) {
  const __m256i low4 = _mm256_set1_epi8(0xF);
  __m256 acc = _mm256_setzero_ps();
  float summs = 0.f;
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ5K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    const float d = y.d * h2f(x.d);
    const float dmin = -y.d * h2f(x.dmin);

    uint32_t u[4];
    std::memcpy(u, x.scales, 12);
    u[3] = ((u[2] >> 4) & 0x0f0f0f0fu) | (((u[1] >> 6) & 0x03030303u) << 4);
    const uint32_t keep = u[1] & 0x3f3f3f3fu;
    u[1] = (u[2] & 0x0f0f0f0fu) | (((u[0] >> 6) & 0x03030303u) << 4);
    u[2] = keep;
    u[0] &= 0x3f3f3f3fu;
    const __m256i sc_mn = _mm256_cvtepu8_epi16(_mm_set_epi32((int)u[3], (int)u[2], (int)u[1], (int)u[0]));

    const __m256i bs = _mm256_loadu_si256((const __m256i*)y.bsums);
    const __m128i pair_sums = _mm_hadd_epi16(_mm256_extracti128_si256(bs, 0), _mm256_extracti128_si256(bs, 1));
    const __m128i mprod = _mm_madd_epi16(_mm256_extracti128_si256(sc_mn, 1), pair_sums);
    const __m128i zero = _mm_setzero_si128();
    const __m128i tot = _mm_hadd_epi32(_mm_hadd_epi32(mprod, zero), zero);
    summs += dmin * (float)_mm_extract_epi32(tot, 0);

    const __m128i sc128 = _mm256_extracti128_si256(sc_mn, 0);
    const __m256i scales = _mm256_insertf128_si256(_mm256_castsi128_si256(sc128), sc128, 1);
    const __m256i hbits = _mm256_loadu_si256((const __m256i*)x.qh);

    __m256i sumi = _mm256_setzero_si256();
    const uint8_t* q5 = x.qs;
    const int8_t* q8 = y.qs;
    for (int j = 0; j < QK_K / 64; ++j) {
      const __m256i s_lo = bcast_word(scales, 2 * j);
      const __m256i s_hi = bcast_word(scales, 2 * j + 1);
      const __m256i bits = _mm256_loadu_si256((const __m256i*)q5);
      q5 += 32;
      // bit 2j (2j+1) of every qh byte moved to bit 4 of the same byte
      const __m256i h0 = _mm256_slli_epi16(_mm256_srl_epi16(_mm256_and_si256(hbits, _mm256_set1_epi8((char)(1 << (2 * j)))),
                                                            _mm_cvtsi32_si128(2 * j)), 4);
      const __m256i h1 = _mm256_slli_epi16(_mm256_srl_epi16(_mm256_and_si256(hbits, _mm256_set1_epi8((char)(2 << (2 * j)))),
                                                            _mm_cvtsi32_si128(2 * j + 1)), 4);
      const __m256i lo = _mm256_add_epi8(_mm256_and_si256(bits, low4), h0);
      const __m256i hi = _mm256_add_epi8(_mm256_and_si256(_mm256_srli_epi16(bits, 4), low4), h1);
      const __m256i y_lo = _mm256_loadu_si256((const __m256i*)q8);
      q8 += 32;
      const __m256i y_hi = _mm256_loadu_si256((const __m256i*)q8);
      q8 += 32;
      const __m256i p0 = _mm256_madd_epi16(s_lo, _mm256_maddubs_epi16(lo, y_lo));
      const __m256i p1 = _mm256_madd_epi16(s_hi, _mm256_maddubs_epi16(hi, y_hi));
      sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p0, p1));
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
  }
  return reduce8(acc) + summs;
}

// Byte `b` of the 16 scales broadcast to 8 bytes, then the next one to the other
// 8 — the 128-bit pattern {s[2i] x8, s[2i+1] x8} of avx.rs:246-255.
static inline __m128i bcast_scale_pair(__m128i scales, int i) {
  const __m128i idx = _mm_set_epi64x(0x0101010101010101LL * (2 * i + 1), 0x0101010101010101LL * (2 * i));
  return _mm_shuffle_epi8(scales, idx);
}

// avx.rs:287-372
float q6k_q8k_dot_avx2(int64_t n, const BlkQ6K* xs, const BlkQ8K* ys) {
  const __m256i low4 = _mm256_set1_epi8(0xF);
  const __m256i low2 = _mm256_set1_epi8(3);
  const __m256i off32 = _mm256_set1_epi8(32);
  __m256 acc = _mm256_setzero_ps();
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ6K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    const float d = y.d * h2f(x.d);
    const uint8_t* ql = x.ql;
    const uint8_t* qh = x.qh;
    const int8_t* q8 = y.qs;
    const __m128i scales = _mm_loadu_si128((const __m128i*)x.scales);
    __m256i sumi = _mm256_setzero_si256();
    for (int j = 0; j < QK_K / 128; ++j) {
      const __m256i l1 = _mm256_loadu_si256((const __m256i*)ql);
      const __m256i l2 = _mm256_loadu_si256((const __m256i*)(ql + 32));
      ql += 64;
      const __m256i h = _mm256_loadu_si256((const __m256i*)qh);
      qh += 32;
      __m256i q[4];
      q[0] = _mm256_or_si256(_mm256_and_si256(l1, low4), _mm256_slli_epi16(_mm256_and_si256(h, low2), 4));
      q[1] = _mm256_or_si256(_mm256_and_si256(l2, low4),
                             _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), low2), 4));
      q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), low4),
                             _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), low2), 4));
      q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l2, 4), low4),
                             _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), low2), 4));
      __m256i p[4];
      for (int t = 0; t < 4; ++t) {
        const __m256i yv = _mm256_loadu_si256((const __m256i*)q8);
        q8 += 32;
        // (q - 32) * y computed as q*y - 32*y on unsigned q, all in i16 pairs
        const __m256i bias = _mm256_maddubs_epi16(off32, yv);
        const __m256i raw = _mm256_maddubs_epi16(q[t], yv);
        const __m256i sc16 = _mm256_cvtepi8_epi16(bcast_scale_pair(scales, 4 * j + t));
        p[t] = _mm256_madd_epi16(sc16, _mm256_sub_epi16(raw, bias));
      }
      sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p[0], p[1]));
      sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p[2], p[3]));
    }
    acc = _mm256_fmadd_ps(_mm256_set1_ps(d), _mm256_cvtepi32_ps(sumi), acc);
  }
  return reduce8(acc);
}

}  // namespace fq_oracle
