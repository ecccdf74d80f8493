// TEST INFRASTRUCTURE — not part of the shipped library.
//
// Block layouts and scalar helpers for the CPU restatement of the reference's
// k-quant arithmetic. Layouts follow fuel-quantized/src/k_quants.rs:56-169
// (#[repr(C)] structs, little-endian f16 scale fields).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace fq_oracle {

constexpr int QK_K = 256;   // fuel-quantized/src/k_quants.rs:12
constexpr int QK_S = 32;    // QK4_0 / QK8_0, k_quants.rs:15-20

#pragma pack(push, 1)
struct BlkQ4_0 { uint16_t d; uint8_t qs[16]; };                                   // k_quants.rs:58-62
struct BlkQ4_1 { uint16_t d; uint16_t m; uint8_t qs[16]; };                       // k_quants.rs:66-71
struct BlkQ5_0 { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; };                    // k_quants.rs:75-80
struct BlkQ5_1 { uint16_t d; uint16_t m; uint8_t qh[4]; uint8_t qs[16]; };        // k_quants.rs:84-90
struct BlkQ8_0 { uint16_t d; int8_t qs[32]; };                                    // k_quants.rs:94-98
struct BlkQ8_1 { uint16_t d; uint16_t s; int8_t qs[32]; };                        // k_quants.rs:102-107
struct BlkQ2K  { uint8_t scales[16]; uint8_t qs[64]; uint16_t d; uint16_t dmin; };   // k_quants.rs:110-116
struct BlkQ3K  { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; }; // k_quants.rs:120-126
struct BlkQ4K  { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; }; // k_quants.rs:132-138
struct BlkQ6K  { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; }; // k_quants.rs:154-160
struct BlkQ8K  { float d; int8_t qs[256]; int16_t bsums[16]; };                   // k_quants.rs:164-169
#pragma pack(pop)
static_assert(sizeof(BlkQ4_0) == 18, "Q4_0");
static_assert(sizeof(BlkQ8_0) == 34, "Q8_0");
static_assert(sizeof(BlkQ4_1) == 20 && sizeof(BlkQ5_0) == 22 && sizeof(BlkQ5_1) == 24 && sizeof(BlkQ8_1) == 36, "legacy blocks");
static_assert(sizeof(BlkQ2K) == 84 && sizeof(BlkQ3K) == 110, "Q2_K / Q3_K");
static_assert(sizeof(BlkQ4K) == 144, "Q4_K");
struct BlkQ5K  { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; }; // k_quants.rs:142-148
static_assert(sizeof(BlkQ5K) == 176, "Q5_K");
static_assert(sizeof(BlkQ6K) == 210, "Q6_K");
static_assert(sizeof(BlkQ8K) == 292, "Q8_K");

// GGUF type ids, fuel-ir/src/quantized.rs:35-75.
enum : int { GGML_Q4_0 = 2, GGML_Q4_1 = 3, GGML_Q5_0 = 6, GGML_Q5_1 = 7, GGML_Q8_0 = 8, GGML_Q8_1 = 9, GGML_Q2K = 10, GGML_Q3K = 11, GGML_Q4K = 12, GGML_Q5K = 13, GGML_Q6K = 14, GGML_Q8K = 15 };

// IEEE binary16 <-> binary32, round-to-nearest-even, what `half::f16` does.
static inline float h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

static inline uint16_t f2h(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  uint32_t ex = (x >> 23) & 0xff;
  uint32_t man = x & 0x7fffffu;
  if (ex == 0xff) {  // inf / nan (quiet bit forced, payload top bits kept)
    return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
  }
  int e = (int)ex - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7c00u);  // overflow -> inf
  if (e <= 0) {
    if (e < -10) return sign;  // underflows to zero (below half the smallest subnormal)
    man |= 0x800000u;
    int shift = 14 - e;  // 14..24
    uint32_t hman = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (hman & 1))) ++hman;
    return (uint16_t)(sign | hman);
  }
  uint32_t hman = man >> 13;
  uint32_t rem = man & 0x1fffu;
  uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | hman);
  if (rem > 0x1000u || (rem == 0x1000u && (hman & 1))) ++out;  // carry may bump the exponent; that is correct
  return out;
}

// Rust `as` casts saturate and send NaN to 0; C++ casts are undefined there.
static inline int32_t sat_i32(float v) {
  if (v != v) return 0;
  if (v >= 2147483648.0f) return INT32_MAX;
  if (v <= -2147483648.0f) return INT32_MIN;
  return (int32_t)v;
}
static inline int8_t sat_i8(float v) {
  if (v != v) return 0;
  if (v >= 127.0f) return 127;
  if (v <= -128.0f) return -128;
  return (int8_t)v;
}
static inline uint8_t sat_u8(float v) {
  if (v != v) return 0;
  if (v >= 255.0f) return 255;
  if (v <= 0.0f) return 0;
  return (uint8_t)v;
}
// fuel-quantized/src/utils.rs:1-3 — f32::round is half-away-from-zero.
static inline int32_t nearest_int(float v) { return sat_i32(roundf(v)); }
static inline int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

// fuel-quantized/src/utils.rs:50-60
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

}  // namespace fq_oracle
