// TEST INFRASTRUCTURE — not part of the shipped library.
//
// CPU restatement of the reference's block quantizers, dequantizers and the
// scalar ("unopt") dot products, in the reference's arithmetic order. Compile
// with -ffp-contract=off: Rust never contracts a*b+c into an fma, and several
// results below depend on the two roundings.
//
// Parity pin: the reference holds no golden vectors for Q4_K / Q6_K / Q8_0; the
// restatement is pinned by (1) the source it follows, cited per function,
// (2) the reference's own Q4_0 known-answer tests restated in tests/, and
// (3) an independent implementation of the same byte layouts (gguf-py).
#include "blocks.h"

#include <algorithm>
#include <vector>

namespace fq_oracle {

// ---------------------------------------------------------------- Q4_0
// fuel-quantized/src/k_quants.rs:199-235
void q4_0_from_float(const float* xs, int64_t k, BlkQ4_0* ys) {
  const int64_t nb = k / QK_S;
  for (int64_t i = 0; i < nb; ++i) {
    const float* x = xs + i * QK_S;
    float amax = 0.f, mx = 0.f;
    for (int j = 0; j < QK_S; ++j) {
      float a = fabsf(x[j]);
      if (amax < a) { amax = a; mx = x[j]; }
    }
    const float d = mx / -8.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    for (int j = 0; j < QK_S / 2; ++j) {
      const float x0 = x[j] * id;
      const float x1 = x[QK_S / 2 + j] * id;
      const uint8_t a = std::min<uint8_t>(15, sat_u8(x0 + 8.5f));
      const uint8_t b = std::min<uint8_t>(15, sat_u8(x1 + 8.5f));
      ys[i].qs[j] = (uint8_t)(a | (b << 4));
    }
  }
}

// fuel-quantized/src/k_quants.rs:177-197
void q4_0_to_float(const BlkQ4_0* xs, int64_t k, float* ys) {
  const int64_t nb = k / QK_S;
  for (int64_t i = 0; i < nb; ++i) {
    const float d = h2f(xs[i].d);
    for (int j = 0; j < QK_S / 2; ++j) {
      const int x0 = (xs[i].qs[j] & 0x0F) - 8;
      const int x1 = (xs[i].qs[j] >> 4) - 8;
      ys[i * QK_S + j] = (float)x0 * d;
      ys[i * QK_S + j + QK_S / 2] = (float)x1 * d;
    }
  }
}

// fuel-quantized/src/k_quants.rs:252-269
float q4_0_q8_0_dot_scalar(int64_t n, const BlkQ4_0* xs, const BlkQ8_0* ys) {
  float sumf = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    int32_t s = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      const int v0 = (xs[b].qs[j] & 0x0F) - 8;
      const int v1 = (xs[b].qs[j] >> 4) - 8;
      s += v0 * ys[b].qs[j] + v1 * ys[b].qs[j + QK_S / 2];
    }
    sumf += (float)s * h2f(xs[b].d) * h2f(ys[b].d);
  }
  return sumf;
}

// ---------------------------------------------------------------- Q4_1 (partner: Q8_1)
static inline uint32_t qh_word(const uint8_t* qh) { return (uint32_t)qh[0] | ((uint32_t)qh[1] << 8) | ((uint32_t)qh[2] << 16) | ((uint32_t)qh[3] << 24); }

// fuel-quantized/src/k_quants.rs:315-351
void q4_1_from_float(const float* xs, int64_t k, BlkQ4_1* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float* x = xs + i * QK_S;
    float mn = INFINITY, mx = -INFINITY;
    for (int j = 0; j < QK_S; ++j) {
      mn = fminf(x[j], mn);
      mx = fmaxf(x[j], mx);
    }
    const float d = (mx - mn) / 15.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    ys[i].m = f2h(mn);
    for (int j = 0; j < QK_S / 2; ++j) {
      const float x0 = (x[j] - mn) * id, x1 = (x[QK_S / 2 + j] - mn) * id;
      const uint8_t a = std::min<uint8_t>(15, sat_u8(x0 + 0.5f)), b = std::min<uint8_t>(15, sat_u8(x1 + 0.5f));
      ys[i].qs[j] = (uint8_t)(a | (b << 4));
    }
  }
}
// k_quants.rs:354-374
void q4_1_to_float(const BlkQ4_1* xs, int64_t k, float* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float d = h2f(xs[i].d), m = h2f(xs[i].m);
    for (int j = 0; j < QK_S / 2; ++j) {
      ys[i * QK_S + j] = (float)(xs[i].qs[j] & 0x0F) * d + m;
      ys[i * QK_S + j + QK_S / 2] = (float)(xs[i].qs[j] >> 4) * d + m;
    }
  }
}
// k_quants.rs:285-313
float q4_1_q8_1_dot_scalar(int64_t n, const BlkQ4_1* xs, const BlkQ8_1* ys) {
  float sumf = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    int32_t s = 0;
    for (int j = 0; j < QK_S / 2; ++j) s += (xs[b].qs[j] & 0x0F) * ys[b].qs[j] + (xs[b].qs[j] >> 4) * ys[b].qs[j + QK_S / 2];
    sumf += (float)s * h2f(xs[b].d) * h2f(ys[b].d) + h2f(xs[b].m) * h2f(ys[b].s);
  }
  return sumf;
}

// ---------------------------------------------------------------- Q5_0 (partner: Q8_0)
// k_quants.rs:424-460. (x + 16.5) as i8 saturates, then min(31), then reinterpreted as u8.
void q5_0_from_float(const float* xs, int64_t k, BlkQ5_0* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float* x = xs + i * QK_S;
    float amax = 0.f, mx = 0.f;
    for (int j = 0; j < QK_S; ++j) {
      const float a = fabsf(x[j]);
      if (amax < a) { amax = a; mx = x[j]; }
    }
    const float d = mx / -16.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    uint32_t qh = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      const uint8_t a = (uint8_t)std::min<int8_t>(sat_i8(x[j] * id + 16.5f), 31);
      const uint8_t b = (uint8_t)std::min<int8_t>(sat_i8(x[j + QK_S / 2] * id + 16.5f), 31);
      ys[i].qs[j] = (uint8_t)((a & 0x0F) | ((b & 0x0F) << 4));
      qh |= (((uint32_t)a & 0x10) >> 4) << j;
      qh |= (((uint32_t)b & 0x10) >> 4) << (j + QK_S / 2);
    }
    ys[i].qh[0] = (uint8_t)qh, ys[i].qh[1] = (uint8_t)(qh >> 8), ys[i].qh[2] = (uint8_t)(qh >> 16), ys[i].qh[3] = (uint8_t)(qh >> 24);
  }
}
// k_quants.rs:463-485
void q5_0_to_float(const BlkQ5_0* xs, int64_t k, float* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float d = h2f(xs[i].d);
    const uint32_t qh = qh_word(xs[i].qh);
    for (int j = 0; j < QK_S / 2; ++j) {
      const int h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
      ys[i * QK_S + j] = (float)(((xs[i].qs[j] & 0x0F) | h0) - 16) * d;
      ys[i * QK_S + j + QK_S / 2] = (float)(((xs[i].qs[j] >> 4) | h1) - 16) * d;
    }
  }
}
// k_quants.rs:401-422
float q5_0_q8_0_dot_scalar(int64_t n, const BlkQ5_0* xs, const BlkQ8_0* ys) {
  float sumf = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const uint32_t qh = qh_word(xs[b].qh);
    int32_t s = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      const int h0 = (int)(((qh >> j) & 1u) << 4), h1 = (int)((qh >> (j + 12)) & 0x10u);
      const int x0 = ((xs[b].qs[j] & 0x0F) | h0) - 16, x1 = ((xs[b].qs[j] >> 4) | h1) - 16;
      s += x0 * ys[b].qs[j] + x1 * ys[b].qs[j + QK_S / 2];
    }
    sumf += (float)s * h2f(xs[b].d) * h2f(ys[b].d);
  }
  return sumf;
}

// ---------------------------------------------------------------- Q5_1 (partner: Q8_1)
// k_quants.rs:535-575
void q5_1_from_float(const float* xs, int64_t k, BlkQ5_1* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float* x = xs + i * QK_S;
    float mn = INFINITY, mx = -INFINITY;
    for (int j = 0; j < QK_S; ++j) {
      mn = fminf(x[j], mn);
      mx = fmaxf(x[j], mx);
    }
    const float d = (mx - mn) / 31.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    ys[i].m = f2h(mn);
    uint32_t qh = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      const uint8_t a = sat_u8((x[j] - mn) * id + 0.5f), b = sat_u8((x[QK_S / 2 + j] - mn) * id + 0.5f);
      ys[i].qs[j] = (uint8_t)((a & 0x0F) | ((b & 0x0F) << 4));
      qh |= (((uint32_t)a & 0x10) >> 4) << j;
      qh |= (((uint32_t)b & 0x10) >> 4) << (j + QK_S / 2);
    }
    ys[i].qh[0] = (uint8_t)qh, ys[i].qh[1] = (uint8_t)(qh >> 8), ys[i].qh[2] = (uint8_t)(qh >> 16), ys[i].qh[3] = (uint8_t)(qh >> 24);
  }
}
// k_quants.rs:578-602
void q5_1_to_float(const BlkQ5_1* xs, int64_t k, float* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float d = h2f(xs[i].d), m = h2f(xs[i].m);
    const uint32_t qh = qh_word(xs[i].qh);
    for (int j = 0; j < QK_S / 2; ++j) {
      const int h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
      ys[i * QK_S + j] = (float)((xs[i].qs[j] & 0x0F) | h0) * d + m;
      ys[i * QK_S + j + QK_S / 2] = (float)((xs[i].qs[j] >> 4) | h1) * d + m;
    }
  }
}
// k_quants.rs:501-533
float q5_1_q8_1_dot_scalar(int64_t n, const BlkQ5_1* xs, const BlkQ8_1* ys) {
  float sumf = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    const uint32_t qh = qh_word(xs[b].qh);
    int32_t s = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      const int h0 = (int)(((qh >> j) << 4) & 0x10u), h1 = (int)((qh >> (j + 12)) & 0x10u);
      s += ((xs[b].qs[j] & 0xF) | h0) * ys[b].qs[j] + ((xs[b].qs[j] >> 4) | h1) * ys[b].qs[j + QK_S / 2];
    }
    sumf += (float)s * h2f(xs[b].d) * h2f(ys[b].d) + h2f(xs[b].m) * h2f(ys[b].s);
  }
  return sumf;
}

// ---------------------------------------------------------------- Q8_1 (activation partner of Q4_1 / Q5_1)
// k_quants.rs:728-757. s = f16(sum) * d in half arithmetic: both factors rounded to f16, the f32 product rounded to f16.
void q8_1_from_float(const float* xs, int64_t k, BlkQ8_1* ys) {
  for (int64_t i = 0; i < k / QK_S; ++i) {
    const float* x = xs + i * QK_S;
    float amax = 0.f;
    for (int j = 0; j < QK_S; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    int32_t sum = 0;
    for (int j = 0; j < QK_S / 2; ++j) {
      ys[i].qs[j] = sat_i8(roundf(x[j] * id));
      ys[i].qs[j + QK_S / 2] = sat_i8(roundf(x[j + QK_S / 2] * id));
      sum += ys[i].qs[j] + ys[i].qs[j + QK_S / 2];
    }
    ys[i].s = f2h(h2f(f2h((float)sum)) * h2f(ys[i].d));
  }
}
void q8_1_to_float(const BlkQ8_1* xs, int64_t k, float* ys) {  // not in the reference (its to_float is unimplemented); for the pins
  for (int64_t i = 0; i < k / QK_S; ++i)
    for (int j = 0; j < QK_S; ++j) ys[i * QK_S + j] = (float)xs[i].qs[j] * h2f(xs[i].d);
}

// ---------------------------------------------------------------- Q8_0
// fuel-quantized/src/k_quants.rs:629-658. The scale is stored as RNE f16 but the
// elements are quantized with the unrounded f32 reciprocal.
void q8_0_from_float(const float* xs, int64_t k, BlkQ8_0* ys) {
  const int64_t nb = k / QK_S;
  for (int64_t i = 0; i < nb; ++i) {
    const float* x = xs + i * QK_S;
    float amax = 0.f;
    for (int j = 0; j < QK_S; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float d = amax / 127.0f;
    const float id = d != 0.f ? 1.0f / d : 0.f;
    ys[i].d = f2h(d);
    for (int j = 0; j < QK_S; ++j) ys[i].qs[j] = sat_i8(roundf(x[j] * id));
  }
}

// fuel-quantized/src/k_quants.rs:611-627
void q8_0_to_float(const BlkQ8_0* xs, int64_t k, float* ys) {
  const int64_t nb = k / QK_S;
  for (int64_t i = 0; i < nb; ++i) {
    const float d = h2f(xs[i].d);
    for (int j = 0; j < QK_S; ++j) ys[i * QK_S + j] = (float)xs[i].qs[j] * d;
  }
}

// fuel-quantized/src/k_quants.rs:674-692
float q8_0_q8_0_dot_scalar(int64_t n, const BlkQ8_0* xs, const BlkQ8_0* ys) {
  float sumf = 0.f;
  for (int64_t b = 0; b < n / QK_S; ++b) {
    int32_t s = 0;
    for (int j = 0; j < QK_S; ++j) s += (int32_t)xs[b].qs[j] * (int32_t)ys[b].qs[j];
    sumf += (float)s * h2f(xs[b].d) * h2f(ys[b].d);
  }
  return sumf;
}

// ---------------------------------------------------------------- Q8_K
// fuel-quantized/src/k_quants.rs:2230-2267. Strict '<' keeps the first of equal
// magnitudes; the signed value of that element fixes the sign of d. The zero
// branch leaves bsums untouched in the reference, which always runs it on a
// zero-filled allocation (k_quants.rs:2304) — so zeros are written here.
void q8k_from_float(const float* xs, int64_t k, BlkQ8K* ys) {
  const int64_t nb = k / QK_K;
  for (int64_t i = 0; i < nb; ++i) {
    const float* x = xs + i * QK_K;
    BlkQ8K& y = ys[i];
    float mx = 0.f, amax = 0.f;
    for (int j = 0; j < QK_K; ++j) {
      const float a = fabsf(x[j]);
      if (amax < a) { amax = a; mx = x[j]; }
    }
    if (amax == 0.f) {
      y.d = 0.f;
      std::memset(y.qs, 0, sizeof(y.qs));
      std::memset(y.bsums, 0, sizeof(y.bsums));
      continue;
    }
    const float iscale = -128.0f / mx;
    for (int j = 0; j < QK_K; ++j) {
      const float v = roundf(iscale * x[j]);
      y.qs[j] = sat_i8(fminf(v, 127.0f));
    }
    for (int j = 0; j < QK_K / 16; ++j) {
      int32_t s = 0;
      for (int t = 0; t < 16; ++t) s += y.qs[j * 16 + t];
      y.bsums[j] = (int16_t)s;
    }
    y.d = 1.0f / iscale;
  }
}

// fuel-quantized/src/k_quants.rs:2269-2280
void q8k_to_float(const BlkQ8K* xs, int64_t k, float* ys) {
  for (int64_t i = 0; i < k / QK_K; ++i)
    for (int j = 0; j < QK_K; ++j) ys[i * QK_K + j] = xs[i].d * (float)xs[i].qs[j];
}

// ---------------------------------------------------------------- Q4_K
// fuel-quantized/src/utils.rs:229-286. Returns (scale, -min) with min <= 0.
static void make_qkx1(int nmax, int ntry, const float* x, int n, float* out_scale, float* out_negmin) {
  std::vector<uint8_t> L(n, 0);
  // min_by keeps the first minimum, max_by the last maximum, under total order
  // (only -0.0 < +0.0 distinguishes that from '<' on non-NaN data).
  auto total_less = [](float a, float b) {
    int32_t ia, ib;
    std::memcpy(&ia, &a, 4);
    std::memcpy(&ib, &b, 4);
    ia ^= (int32_t)((uint32_t)(ia >> 31) >> 1);
    ib ^= (int32_t)((uint32_t)(ib >> 31) >> 1);
    return ia < ib;
  };
  float mn = x[0], mx = x[0];
  for (int i = 1; i < n; ++i) {
    if (total_less(x[i], mn)) mn = x[i];
    if (!total_less(x[i], mx)) mx = x[i];
  }
  if (mx == mn) { *out_scale = 0.f; *out_negmin = 0.f; return; }
  if (mn > 0.f) mn = 0.f;  // min.min(0.)
  float iscale = (float)nmax / (mx - mn);
  float scale = 1.0f / iscale;
  for (int t = 0; t < ntry; ++t) {
    float sumlx = 0.f;
    int32_t suml2 = 0;
    bool did_change = false;
    for (int i = 0; i < n; ++i) {
      const int32_t li = clampi(nearest_int(iscale * (x[i] - mn)), 0, nmax);
      const uint8_t c = (uint8_t)li;
      if (c != L[i]) { L[i] = c; did_change = true; }
      sumlx += (x[i] - mn) * (float)li;
      suml2 += li * li;
    }
    scale = sumlx / (float)suml2;
    float sum = 0.f;
    for (int i = 0; i < n; ++i) sum += x[i] - scale * (float)L[i];
    mn = sum / (float)n;
    if (mn > 0.f) mn = 0.f;
    iscale = 1.0f / scale;
    if (!did_change) break;
  }
  *out_scale = scale;
  *out_negmin = -mn;
}

// fuel-quantized/src/k_quants.rs:1470-1528
void q4k_from_float(const float* xs, int64_t k, BlkQ4K* ys) {
  const int64_t nb = k / QK_K;
  for (int64_t ib = 0; ib < nb; ++ib) {
    const float* x = xs + ib * QK_K;
    BlkQ4K& blk = ys[ib];
    float mins[8], scales[8];
    for (int j = 0; j < 8; ++j) make_qkx1(15, 5, x + 32 * j, 32, &scales[j], &mins[j]);
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; ++j) max_scale = fmaxf(scales[j], max_scale);
    for (int j = 0; j < 8; ++j) max_min = fmaxf(mins[j], max_min);
    const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
    const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
    std::memset(blk.scales, 0, sizeof(blk.scales));
    for (int j = 0; j < 8; ++j) {
      const uint8_t ls = (uint8_t)std::min(nearest_int(inv_scale * scales[j]), 63);
      const uint8_t lm = (uint8_t)std::min(nearest_int(inv_min * mins[j]), 63);
      if (j < 4) {
        blk.scales[j] = ls;
        blk.scales[j + 4] = lm;
      } else {
        blk.scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        blk.scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
        blk.scales[j] |= (uint8_t)((lm >> 4) << 6);
      }
    }
    blk.d = f2h(max_scale / 63.0f);
    blk.dmin = f2h(max_min / 63.0f);
    uint8_t L[QK_K] = {0};
    for (int j = 0; j < 8; ++j) {
      uint8_t sc, m;
      scale_min_k4(j, blk.scales, &sc, &m);
      const float d = h2f(blk.d) * (float)sc;
      if (d != 0.f) {
        const float dm = h2f(blk.dmin) * (float)m;
        for (int t = 0; t < 32; ++t)
          L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / d), 0, 15);
      }
    }
    for (int j = 0; j < QK_K; j += 64)
      for (int t = 0; t < 32; ++t) blk.qs[(j / 64) * 32 + t] = (uint8_t)(L[j + t] | (L[j + t + 32] << 4));
  }
}

// fuel-quantized/src/k_quants.rs:1595-1622: d1 = d*sc; y = d1*q - m1 (two roundings).
void q4k_to_float(const BlkQ4K* xs, int64_t k, float* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const BlkQ4K& b = xs[ib];
    float* y = ys + ib * QK_K;
    const float d = h2f(b.d), mn = h2f(b.dmin);
    int is = 0, o = 0;
    for (int j = 0; j < QK_K; j += 64) {
      const uint8_t* q = b.qs + j / 2;
      uint8_t sc, m;
      scale_min_k4(is, b.scales, &sc, &m);
      const float d1 = d * (float)sc, m1 = mn * (float)m;
      scale_min_k4(is + 1, b.scales, &sc, &m);
      const float d2 = d * (float)sc, m2 = mn * (float)m;
      for (int t = 0; t < 32; ++t) y[o++] = d1 * (float)(q[t] & 0xF) - m1;
      for (int t = 0; t < 32; ++t) y[o++] = d2 * (float)(q[t] >> 4) - m2;
      is += 2;
    }
  }
}

// fuel-quantized/src/k_quants.rs:1388-1468 (canonical summation order).
float q4k_q8k_dot_scalar(int64_t n, const BlkQ4K* xs, const BlkQ8K* ys) {
  int8_t a8[QK_K];
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float sumf = 0.f;
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ4K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    for (int g = 0; g < 4; ++g)
      for (int t = 0; t < 32; ++t) {
        a8[64 * g + t] = (int8_t)(x.qs[32 * g + t] & 0xF);
        a8[64 * g + 32 + t] = (int8_t)(x.qs[32 * g + t] >> 4);
      }
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; ++j) scale_min_k4(j, x.scales, &sc[j], &mn[j]);
    int32_t sumi = 0;
    for (int j = 0; j < 16; ++j) sumi += (int32_t)y.bsums[j] * (int32_t)mn[j / 2];
    int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 8; ++j)
      for (int t = 0; t < 32; ++t) {
        const int16_t p = (int16_t)((int16_t)y.qs[32 * j + t] * (int16_t)a8[32 * j + t]);
        acc[t & 7] += (int32_t)sc[j] * (int32_t)p;
      }
    const float d = h2f(x.d) * y.d;
    for (int l = 0; l < 8; ++l) lane[l] += d * (float)acc[l];
    const float dmin = h2f(x.dmin) * y.d;
    sumf -= dmin * (float)sumi;
  }
  float s = 0.f;
  for (int l = 0; l < 8; ++l) s += lane[l];
  return sumf + s;
}

// ---------------------------------------------------------------- Q5_K
// fuel-quantized/src/k_quants.rs:1729-1796: Q4_K's fit with 32 levels; the fifth bit of element 64g+t goes to bit 2g of
// qh[t], that of element 64g+32+t to bit 2g+1.
void q5k_from_float(const float* xs, int64_t k, BlkQ5K* ys) {
  const int64_t nb = k / QK_K;
  for (int64_t ib = 0; ib < nb; ++ib) {
    const float* x = xs + ib * QK_K;
    BlkQ5K& blk = ys[ib];
    float mins[8], scales[8];
    for (int j = 0; j < 8; ++j) make_qkx1(31, 5, x + 32 * j, 32, &scales[j], &mins[j]);
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; ++j) max_scale = fmaxf(scales[j], max_scale);
    for (int j = 0; j < 8; ++j) max_min = fmaxf(mins[j], max_min);
    const float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
    const float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
    std::memset(blk.scales, 0, sizeof(blk.scales));
    for (int j = 0; j < 8; ++j) {
      const uint8_t ls = (uint8_t)std::min(nearest_int(inv_scale * scales[j]), 63);
      const uint8_t lm = (uint8_t)std::min(nearest_int(inv_min * mins[j]), 63);
      if (j < 4) {
        blk.scales[j] = ls;
        blk.scales[j + 4] = lm;
      } else {
        blk.scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        blk.scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
        blk.scales[j] |= (uint8_t)((lm >> 4) << 6);
      }
    }
    blk.d = f2h(max_scale / 63.0f);
    blk.dmin = f2h(max_min / 63.0f);
    uint8_t L[QK_K] = {0};
    for (int j = 0; j < 8; ++j) {
      uint8_t sc, m;
      scale_min_k4(j, blk.scales, &sc, &m);
      const float d = h2f(blk.d) * (float)sc;
      if (d != 0.f) {
        const float dm = h2f(blk.dmin) * (float)m;
        for (int t = 0; t < 32; ++t)
          L[32 * j + t] = (uint8_t)clampi(nearest_int((x[32 * j + t] + dm) / d), 0, 31);
      }
    }
    std::memset(blk.qh, 0, sizeof(blk.qh));
    for (int g = 0; g < 4; ++g)
      for (int t = 0; t < 32; ++t) {
        uint8_t l1 = L[64 * g + t], l2 = L[64 * g + 32 + t];
        if (l1 > 15) { l1 -= 16; blk.qh[t] |= (uint8_t)(1u << (2 * g)); }
        if (l2 > 15) { l2 -= 16; blk.qh[t] |= (uint8_t)(2u << (2 * g)); }
        blk.qs[32 * g + t] = (uint8_t)(l1 | (l2 << 4));
      }
  }
}

// fuel-quantized/src/k_quants.rs:1889-1923: y = d1 * (nibble + 16*bit) - m1, the sum inside the brackets exact.
void q5k_to_float(const BlkQ5K* xs, int64_t k, float* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const BlkQ5K& b = xs[ib];
    float* y = ys + ib * QK_K;
    const float d = h2f(b.d), mn = h2f(b.dmin);
    int o = 0;
    for (int g = 0; g < 4; ++g) {
      const uint8_t* q = b.qs + 32 * g;
      uint8_t sc, m;
      scale_min_k4(2 * g, b.scales, &sc, &m);
      const float d1 = d * (float)sc, m1 = mn * (float)m;
      scale_min_k4(2 * g + 1, b.scales, &sc, &m);
      const float d2 = d * (float)sc, m2 = mn * (float)m;
      for (int t = 0; t < 32; ++t) y[o++] = d1 * ((float)(q[t] & 0xF) + ((b.qh[t] >> (2 * g)) & 1 ? 16.f : 0.f)) - m1;
      for (int t = 0; t < 32; ++t) y[o++] = d2 * ((float)(q[t] >> 4) + ((b.qh[t] >> (2 * g + 1)) & 1 ? 16.f : 0.f)) - m2;
    }
  }
}

// fuel-quantized/src/k_quants.rs:1644-1727 (canonical summation order; Q4_K's with 5-bit values).
float q5k_q8k_dot_scalar(int64_t n, const BlkQ5K* xs, const BlkQ8K* ys) {
  int8_t a8[QK_K];
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float sumf = 0.f;
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ5K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    for (int g = 0; g < 4; ++g)
      for (int t = 0; t < 32; ++t) {
        a8[64 * g + t] = (int8_t)((x.qs[32 * g + t] & 0xF) + (((x.qh[t] >> (2 * g)) & 1) ? 16 : 0));
        a8[64 * g + 32 + t] = (int8_t)((x.qs[32 * g + t] >> 4) + (((x.qh[t] >> (2 * g + 1)) & 1) ? 16 : 0));
      }
    uint8_t sc[8], mn[8];
    for (int j = 0; j < 8; ++j) scale_min_k4(j, x.scales, &sc[j], &mn[j]);
    int32_t sumi = 0;
    for (int j = 0; j < 16; ++j) sumi += (int32_t)y.bsums[j] * (int32_t)mn[j / 2];
    int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < 8; ++j)
      for (int t = 0; t < 32; ++t) {
        const int16_t p = (int16_t)((int16_t)y.qs[32 * j + t] * (int16_t)a8[32 * j + t]);
        acc[t & 7] += (int32_t)sc[j] * (int32_t)p;
      }
    const float d = h2f(x.d) * y.d;
    for (int l = 0; l < 8; ++l) lane[l] += d * (float)acc[l];
    const float dmin = h2f(x.dmin) * y.d;
    sumf -= dmin * (float)sumi;
  }
  float s = 0.f;
  for (int l = 0; l < 8; ++l) s += lane[l];
  return sumf + s;
}

// ---------------------------------------------------------------- Q2_K, Q3_K
// Element e of a block sits in qs[32 * (e / 128) + e % 32], bits 2 * ((e % 128) / 32) .. +1; every 16 elements share
// scale index e / 16.

// fuel-quantized/src/k_quants.rs:836-895: sixteen (scale, min) fits of 16 elements (make_qkx1_quants(3, 5, .)), 4-bit
// scales and mins against the block's largest, then the elements against the stored f16 values
void q2k_from_float(const float* xs, int64_t k, BlkQ2K* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const float* x = xs + ib * QK_K;
    BlkQ2K& blk = ys[ib];
    float mins[16], scales[16];
    for (int j = 0; j < 16; ++j) make_qkx1(3, 5, x + 16 * j, 16, &scales[j], &mins[j]);
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 16; ++j) max_scale = fmaxf(scales[j], max_scale);
    for (int j = 0; j < 16; ++j) max_min = fmaxf(mins[j], max_min);
    if (max_scale > 0.f) {
      const float iscale = 15.0f / max_scale;
      for (int j = 0; j < 16; ++j) blk.scales[j] = (uint8_t)nearest_int(iscale * scales[j]);
      blk.d = f2h(max_scale / 15.0f);
    } else {
      for (int j = 0; j < 16; ++j) blk.scales[j] = 0;
      blk.d = f2h(0.f);
    }
    if (max_min > 0.f) {
      const float iscale = 15.0f / max_min;
      for (int j = 0; j < 16; ++j) blk.scales[j] |= (uint8_t)((uint8_t)nearest_int(iscale * mins[j]) << 4);
      blk.dmin = f2h(max_min / 15.0f);
    } else {
      blk.dmin = f2h(0.f);
    }
    uint8_t L[QK_K] = {0};
    for (int j = 0; j < 16; ++j) {
      const float d = h2f(blk.d) * (float)(blk.scales[j] & 0xF);
      if (d == 0.f) continue;
      const float dm = h2f(blk.dmin) * (float)(blk.scales[j] >> 4);
      for (int t = 0; t < 16; ++t) L[16 * j + t] = (uint8_t)clampi(nearest_int((x[16 * j + t] + dm) / d), 0, 3);
    }
    for (int j = 0; j < QK_K; j += 128)
      for (int l = 0; l < 32; ++l)
        blk.qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
  }
}

// fuel-quantized/src/utils.rs:289-354 with do_rmse: the scale of 16 elements for levels -nmax .. nmax-1, refined by
// moving one level at a time while the weighted fit improves (weights x^2)
static float make_q3(const float* x, int n, int nmax) {
  float mx = 0.f, amax = 0.f;
  for (int i = 0; i < n; ++i) {
    const float ax = fabsf(x[i]);
    if (ax > amax) { amax = ax; mx = x[i]; }
  }
  if (amax == 0.f) return 0.f;
  const float iscale = -(float)nmax / mx;
  int8_t L[32];
  float sumlx = 0.f, suml2 = 0.f;
  for (int i = 0; i < n; ++i) {
    const int32_t li = clampi(sat_i32(roundf(iscale * x[i])), -nmax, nmax - 1);
    L[i] = (int8_t)li;
    const float w = x[i] * x[i];
    sumlx += w * x[i] * (float)li;
    suml2 += w * (float)(li * li);
  }
  for (int it = 0; it < 5; ++it) {
    int changed = 0;
    for (int i = 0; i < n; ++i) {
      const float w = x[i] * x[i];
      float slx = sumlx - w * x[i] * (float)L[i];
      if (slx > 0.f) {
        float sl2 = suml2 - w * (float)((int32_t)L[i] * (int32_t)L[i]);
        int32_t nl = clampi(sat_i32(roundf(x[i] * sl2 / slx)), -nmax, nmax - 1);
        if (nl != (int32_t)L[i]) {
          slx += w * x[i] * (float)nl;
          sl2 += w * (float)(nl * nl);
          if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
            L[i] = (int8_t)nl;
            sumlx = slx;
            suml2 = sl2;
            ++changed;
          }
        }
      }
    }
    if (!changed) break;
  }
  return sumlx / suml2;
}

// fuel-quantized/src/k_quants.rs:1135-1216
void q3k_from_float(const float* xs, int64_t k, BlkQ3K* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const float* x = xs + ib * QK_K;
    BlkQ3K& blk = ys[ib];
    float scales[16];
    for (int j = 0; j < 16; ++j) scales[j] = make_q3(x + 16 * j, 16, 4);
    float max_scale = 0.f;
    for (int j = 0; j < 16; ++j)
      if (fabsf(scales[j]) > fabsf(max_scale)) max_scale = scales[j];
    std::memset(blk.scales, 0, sizeof(blk.scales));
    if (max_scale != 0.f) {
      const float iscale = -32.0f / max_scale;
      for (int j = 0; j < 16; ++j) {
        int32_t l = clampi(nearest_int(iscale * scales[j]), -32, 31) + 32;
        if (j < 8) blk.scales[j] = (uint8_t)(l & 0xF);
        else blk.scales[j - 8] |= (uint8_t)((l & 0xF) << 4);
        l >>= 4;
        blk.scales[j % 4 + 8] |= (uint8_t)(l << (2 * (j / 4)));
      }
      blk.d = f2h(1.0f / iscale);
    } else {
      blk.d = f2h(0.f);
    }
    int8_t L[QK_K] = {0};
    for (int j = 0; j < 16; ++j) {
      int sc = j < 8 ? (blk.scales[j] & 0xF) : (blk.scales[j - 8] >> 4);
      sc = (int)(int8_t)(sc | (((blk.scales[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
      const float d = h2f(blk.d) * (float)sc;
      if (d != 0.f)
        for (int t = 0; t < 16; ++t) L[16 * j + t] = (int8_t)(clampi(nearest_int(x[16 * j + t] / d), -4, 3) + 4);
    }
    std::memset(blk.hmask, 0, sizeof(blk.hmask));
    for (int e = 0; e < QK_K; ++e)
      if (L[e] > 3) {
        blk.hmask[e % 32] |= (uint8_t)(1u << (e / 32));
        L[e] -= 4;
      }
    for (int j = 0; j < QK_K; j += 128)
      for (int l = 0; l < 32; ++l)
        blk.qs[j / 4 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 2) | (L[j + l + 64] << 4) | (L[j + l + 96] << 6));
  }
}

// fuel-quantized/src/k_quants.rs:958-994: y = (d * sc_lo) * q - (dmin * sc_hi), product and difference rounded separately
void q2k_to_float(const BlkQ2K* xs, int64_t k, float* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const BlkQ2K& x = xs[ib];
    const float d = h2f(x.d), mn = h2f(x.dmin);
    for (int e = 0; e < QK_K; ++e) {
      const uint8_t sc = x.scales[e / 16];
      const float dl = d * (float)(sc & 0xF), ml = mn * (float)(sc >> 4);
      const int q = (x.qs[32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3;
      ys[ib * QK_K + e] = dl * (float)q - ml;
    }
  }
}
// k_quants.rs:783-833
float q2k_q8k_dot_scalar(int64_t n, const BlkQ2K* xs, const BlkQ8K* ys) {
  float sumf = 0.f;
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ2K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    int32_t summs = 0;
    for (int j = 0; j < 16; ++j) summs += (int32_t)y.bsums[j] * (int32_t)(x.scales[j] >> 4);
    const float dall = y.d * h2f(x.d), dmin = y.d * h2f(x.dmin);
    int32_t isum = 0;
    for (int g = 0; g < 16; ++g) {  // groups of 16 elements in index order
      int32_t part = 0;
      for (int l = 0; l < 16; ++l) {
        const int e = 16 * g + l;
        part += (int32_t)y.qs[e] * (int32_t)((x.qs[32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3);
      }
      isum += (int32_t)(x.scales[g] & 0xF) * part;
    }
    sumf += dall * (float)isum - dmin * (float)summs;
  }
  return sumf;
}

// the sixteen 6-bit scales of a Q3_K block, still offset by 32 (k_quants.rs:1095-1103, 1319-1327)
static inline void q3k_scales(const uint8_t* sc12, int8_t out[16]) {
  uint32_t a[3];
  std::memcpy(a, sc12, 12);
  const uint32_t m1 = 0x03030303u, m2 = 0x0f0f0f0fu, tmp = a[2];
  const uint32_t w[4] = {(a[0] & m2) | ((tmp & m1) << 4), (a[1] & m2) | (((tmp >> 2) & m1) << 4),
                         ((a[0] >> 4) & m2) | (((tmp >> 4) & m1) << 4), ((a[1] >> 4) & m2) | (((tmp >> 6) & m1) << 4)};
  std::memcpy(out, w, 16);
}
static inline int q3k_value(const BlkQ3K& x, int e) {  // in [-4, 3]
  const int low = (x.qs[32 * (e / 128) + e % 32] >> (2 * ((e % 128) / 32))) & 3;
  const int bit = 4 * (e / 128) + (e % 128) / 32;
  return low - (((x.hmask[e % 32] >> bit) & 1) ? 0 : 4);
}
// k_quants.rs:1314-1366
void q3k_to_float(const BlkQ3K* xs, int64_t k, float* ys) {
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const BlkQ3K& x = xs[ib];
    int8_t sc[16];
    q3k_scales(x.scales, sc);
    const float d = h2f(x.d);
    for (int e = 0; e < QK_K; ++e) {
      const float dl = d * ((float)sc[e / 16] - 32.0f);
      ys[ib * QK_K + e] = dl * (float)q3k_value(x, e);
    }
  }
}
// k_quants.rs:1013-1133: eight running integer lanes per block (element e adds to lane e % 8), scaled by d per block
// into eight f32 lanes, summed in index order at the end
float q3k_q8k_dot_scalar(int64_t n, const BlkQ3K* xs, const BlkQ8K* ys) {
  float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ3K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    int8_t sc[16];
    q3k_scales(x.scales, sc);
    int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int e = 0; e < QK_K; ++e) {
      const int16_t p = (int16_t)((int16_t)y.qs[e] * (int16_t)q3k_value(x, e));
      aux32[e % 8] += ((int32_t)sc[e / 16] - 32) * (int32_t)p;
    }
    const float d = h2f(x.d) * y.d;
    for (int l = 0; l < 8; ++l) sums[l] += d * (float)aux32[l];
  }
  float s = 0.f;
  for (int l = 0; l < 8; ++l) s += sums[l];
  return s;
}

// ---------------------------------------------------------------- Q6_K
// fuel-quantized/src/utils.rs:62-191 with rmse_type=1, qw=null (weights x^2).
// Writes L[i] in [0, 2*nmax) and returns the fitted scale.
static float make_qx(int n, int nmax, const float* x, int8_t* L) {
  float mx = 0.f, amax = 0.f;
  for (int i = 0; i < n; ++i) {
    const float ax = fabsf(x[i]);
    if (ax > amax) { amax = ax; mx = x[i]; }
  }
  if (amax == 0.f) {
    for (int i = 0; i < n; ++i) L[i] = 0;
    return 0.f;
  }
  float iscale = -(float)nmax / mx;
  float sumlx = 0.f, suml2 = 0.f;
  for (int i = 0; i < n; ++i) {
    const int32_t l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
    L[i] = (int8_t)(l + nmax);
    const float w = x[i] * x[i];
    const float lf = (float)l;
    sumlx += w * x[i] * lf;
    suml2 += w * lf * lf;
  }
  float scale = sumlx / suml2;
  float best = scale * sumlx;
  for (int itry = 0; itry < 3; ++itry) {
    const float is2 = 1.0f / scale;
    float slx = 0.f, sl2 = 0.f;
    bool changed = false;
    for (int i = 0; i < n; ++i) {
      const int32_t l = clampi(nearest_int(is2 * x[i]), -nmax, nmax - 1);
      if (l + nmax != (int32_t)L[i]) changed = true;
      const float w = x[i] * x[i];
      const float lf = (float)l;
      slx += w * x[i] * lf;
      sl2 += w * lf * lf;
    }
    if (!changed || sl2 == 0.f || slx * slx <= best * sl2) break;
    for (int i = 0; i < n; ++i) L[i] = (int8_t)(nmax + clampi(nearest_int(is2 * x[i]), -nmax, nmax - 1));
    sumlx = slx;
    suml2 = sl2;
    scale = sumlx / suml2;
    best = scale * sumlx;
  }
  for (int itry = 0; itry < 5; ++itry) {
    int n_changed = 0;
    for (int i = 0; i < n; ++i) {
      const float w = x[i] * x[i];
      const int32_t l = (int32_t)L[i] - nmax;
      float slx = sumlx - w * x[i] * (float)l;
      if (slx > 0.f) {
        float sl2 = suml2 - w * (float)l * (float)l;
        int32_t nl = clampi(nearest_int(x[i] * sl2 / slx), -nmax, nmax - 1);
        if (nl != l) {
          slx += w * x[i] * (float)nl;
          sl2 += w * (float)nl * (float)nl;
          if (sl2 > 0.f && slx * slx * suml2 > sumlx * sumlx * sl2) {
            L[i] = (int8_t)(nmax + nl);
            sumlx = slx;
            suml2 = sl2;
            scale = sumlx / suml2;
            best = scale * sumlx;
            ++n_changed;
          }
        }
      }
    }
    if (n_changed == 0) break;
  }
  (void)best;
  return scale;
}

// fuel-quantized/src/k_quants.rs:2005-2075. The level scratch L persists across
// blocks, as in the reference (it only matters when a sub-block scale is zero).
void q6k_from_float(const float* xs, int64_t k, BlkQ6K* ys) {
  int8_t L[QK_K] = {0};
  float scales[16];
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const float* x = xs + ib * QK_K;
    BlkQ6K& y = ys[ib];
    float max_scale = 0.f, max_abs = 0.f;
    for (int s = 0; s < 16; ++s) {
      const float sc = make_qx(16, 32, x + 16 * s, L + 16 * s);
      scales[s] = sc;
      const float a = fabsf(sc);
      if (a > max_abs) { max_abs = a; max_scale = sc; }
    }
    const float iscale = -128.0f / max_scale;
    y.d = f2h(1.0f / iscale);
    for (int s = 0; s < 16; ++s) y.scales[s] = (int8_t)std::min(nearest_int(iscale * scales[s]), 127);
    for (int s = 0; s < 16; ++s) {
      const float d = h2f(y.d) * (float)y.scales[s];
      if (d == 0.f) continue;
      for (int t = 0; t < 16; ++t) {
        const int32_t ll = clampi(nearest_int(x[16 * s + t] / d), -32, 31);
        L[16 * s + t] = (int8_t)(ll + 32);
      }
    }
    uint8_t* ql = y.ql;
    uint8_t* qh = y.qh;
    for (int j = 0; j < QK_K; j += 128) {
      for (int t = 0; t < 32; ++t) {
        const int8_t a = L[j + t], b = L[j + t + 32], c = L[j + t + 64], e = L[j + t + 96];
        ql[t] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
        ql[t + 32] = (uint8_t)((b & 0xF) | ((e & 0xF) << 4));
        // i8 arithmetic in the reference: '>>' is arithmetic and '<<' wraps in 8 bits.
        qh[t] = (uint8_t)((int8_t)(a >> 4) | (int8_t)((int8_t)(b >> 4) << 2) | (int8_t)((int8_t)(c >> 4) << 4) |
                          (int8_t)((int8_t)(e >> 4) << 6));
      }
      ql += 64;
      qh += 32;
    }
  }
}

static inline void q6k_unpack(const BlkQ6K& x, int8_t* out) {
  for (int j = 0; j < QK_K; j += 128) {
    const uint8_t* ql = x.ql + j / 2;
    const uint8_t* qh = x.qh + j / 4;
    for (int t = 0; t < 32; ++t) {
      out[j + t] = (int8_t)((int)((ql[t] & 0xF) | ((qh[t] & 3) << 4)) - 32);
      out[j + t + 32] = (int8_t)((int)((ql[t + 32] & 0xF) | (((qh[t] >> 2) & 3) << 4)) - 32);
      out[j + t + 64] = (int8_t)((int)((ql[t] >> 4) | (((qh[t] >> 4) & 3) << 4)) - 32);
      out[j + t + 96] = (int8_t)((int)((ql[t + 32] >> 4) | (((qh[t] >> 6) & 3) << 4)) - 32);
    }
  }
}

// fuel-quantized/src/k_quants.rs:2158-2189: (d * sc) * q, left to right.
void q6k_to_float(const BlkQ6K* xs, int64_t k, float* ys) {
  int8_t q[QK_K];
  for (int64_t ib = 0; ib < k / QK_K; ++ib) {
    const BlkQ6K& x = xs[ib];
    q6k_unpack(x, q);
    const float d = h2f(x.d);
    for (int e = 0; e < QK_K; ++e) {
      const int half = e / 128, r = e % 128;
      const int is = 8 * half + (r % 32) / 16 + 2 * (r / 32);
      ys[ib * QK_K + e] = d * (float)x.scales[is] * (float)q[e];
    }
  }
}

// fuel-quantized/src/k_quants.rs:1946-2003 — f32 lanes, one multiply-add per product.
float q6k_q8k_dot_scalar(int64_t n, const BlkQ6K* xs, const BlkQ8K* ys) {
  int8_t q[QK_K];
  float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int64_t ib = 0; ib < n / QK_K; ++ib) {
    const BlkQ6K& x = xs[ib];
    const BlkQ8K& y = ys[ib];
    q6k_unpack(x, q);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < 16; ++s) {
      const float sc = (float)x.scales[s];
      for (int t = 0; t < 16; ++t) {
        const int16_t p = (int16_t)((int16_t)y.qs[16 * s + t] * (int16_t)q[16 * s + t]);
        acc[t & 7] += sc * (float)p;
      }
    }
    const float d = h2f(x.d) * y.d;
    for (int l = 0; l < 8; ++l) lane[l] += acc[l] * d;
  }
  float s = 0.f;
  for (int l = 0; l < 8; ++l) s += lane[l];
  return s;
}

}  // namespace fq_oracle
