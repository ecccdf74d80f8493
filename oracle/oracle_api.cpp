// TEST INFRASTRUCTURE — not part of the shipped library.
//
// C entry points over the restatement, loaded with ctypes by tests/, by the
// smoke check and by the benchmark's CPU-baseline leg. The matmul driver follows
// fuel-quantized/src/k_quants.rs:2284-2331: quantize every activation row to the
// weight format's dot-product partner (Q8_K for k-quants, Q8_0 for Q4_0/Q8_0),
// then one dot product per (row, output column). OpenMP over output columns
// stands in for the reference's rayon split of the same loop.
#include "blocks.h"

#include <omp.h>

#include <vector>

namespace fq_oracle {
void q4_0_from_float(const float*, int64_t, BlkQ4_0*);
void q4_0_to_float(const BlkQ4_0*, int64_t, float*);
float q4_0_q8_0_dot_scalar(int64_t, const BlkQ4_0*, const BlkQ8_0*);
void q4_1_from_float(const float*, int64_t, BlkQ4_1*);
void q4_1_to_float(const BlkQ4_1*, int64_t, float*);
float q4_1_q8_1_dot_scalar(int64_t, const BlkQ4_1*, const BlkQ8_1*);
float q4_1_q8_1_dot_avx2(int64_t, const BlkQ4_1*, const BlkQ8_1*);
void q5_0_from_float(const float*, int64_t, BlkQ5_0*);
void q5_0_to_float(const BlkQ5_0*, int64_t, float*);
float q5_0_q8_0_dot_scalar(int64_t, const BlkQ5_0*, const BlkQ8_0*);
float q5_0_q8_0_dot_avx2(int64_t, const BlkQ5_0*, const BlkQ8_0*);
void q5_1_from_float(const float*, int64_t, BlkQ5_1*);
void q5_1_to_float(const BlkQ5_1*, int64_t, float*);
float q5_1_q8_1_dot_scalar(int64_t, const BlkQ5_1*, const BlkQ8_1*);
float q5_1_q8_1_dot_avx2(int64_t, const BlkQ5_1*, const BlkQ8_1*);
void q8_1_from_float(const float*, int64_t, BlkQ8_1*);
void q8_1_to_float(const BlkQ8_1*, int64_t, float*);
void q2k_from_float(const float*, int64_t, BlkQ2K*);
void q3k_from_float(const float*, int64_t, BlkQ3K*);
void q2k_to_float(const BlkQ2K*, int64_t, float*);
float q2k_q8k_dot_scalar(int64_t, const BlkQ2K*, const BlkQ8K*);
float q2k_q8k_dot_avx2(int64_t, const BlkQ2K*, const BlkQ8K*);
void q3k_to_float(const BlkQ3K*, int64_t, float*);
float q3k_q8k_dot_scalar(int64_t, const BlkQ3K*, const BlkQ8K*);
float q3k_q8k_dot_avx2(int64_t, const BlkQ3K*, const BlkQ8K*);
void q8_0_from_float(const float*, int64_t, BlkQ8_0*);
void q8_0_to_float(const BlkQ8_0*, int64_t, float*);
float q8_0_q8_0_dot_scalar(int64_t, const BlkQ8_0*, const BlkQ8_0*);
void q8k_from_float(const float*, int64_t, BlkQ8K*);
void q8k_to_float(const BlkQ8K*, int64_t, float*);
void q4k_from_float(const float*, int64_t, BlkQ4K*);
void q4k_to_float(const BlkQ4K*, int64_t, float*);
float q4k_q8k_dot_scalar(int64_t, const BlkQ4K*, const BlkQ8K*);
void q5k_from_float(const float*, int64_t, BlkQ5K*);
void q5k_to_float(const BlkQ5K*, int64_t, float*);
float q5k_q8k_dot_scalar(int64_t, const BlkQ5K*, const BlkQ8K*);
void q6k_from_float(const float*, int64_t, BlkQ6K*);
void q6k_to_float(const BlkQ6K*, int64_t, float*);
float q6k_q8k_dot_scalar(int64_t, const BlkQ6K*, const BlkQ8K*);
float q4_0_q8_0_dot_avx2(int64_t, const BlkQ4_0*, const BlkQ8_0*);
float q8_0_q8_0_dot_avx2(int64_t, const BlkQ8_0*, const BlkQ8_0*);
float q4k_q8k_dot_avx2(int64_t, const BlkQ4K*, const BlkQ8K*);
float q5k_q8k_dot_avx2(int64_t, const BlkQ5K*, const BlkQ8K*);
float q6k_q8k_dot_avx2(int64_t, const BlkQ6K*, const BlkQ8K*);
}  // namespace fq_oracle

using namespace fq_oracle;

namespace {

struct Fmt {
  int block_elems;
  int block_bytes;
  int act_type;  // dot-product partner
};

bool fmt_of(int type, Fmt* f) {
  switch (type) {
    case GGML_Q4_0: *f = {32, 18, GGML_Q8_0}; return true;
    case GGML_Q4_1: *f = {32, 20, GGML_Q8_1}; return true;
    case GGML_Q5_0: *f = {32, 22, GGML_Q8_0}; return true;
    case GGML_Q5_1: *f = {32, 24, GGML_Q8_1}; return true;
    case GGML_Q8_1: *f = {32, 36, GGML_Q8_1}; return true;
    case GGML_Q8_0: *f = {32, 34, GGML_Q8_0}; return true;
    case GGML_Q2K: *f = {256, 84, GGML_Q8K}; return true;
    case GGML_Q3K: *f = {256, 110, GGML_Q8K}; return true;
    case GGML_Q4K: *f = {256, 144, GGML_Q8K}; return true;
    case GGML_Q5K: *f = {256, 176, GGML_Q8K}; return true;
    case GGML_Q6K: *f = {256, 210, GGML_Q8K}; return true;
    case GGML_Q8K: *f = {256, 292, GGML_Q8K}; return true;
    default: return false;
  }
}

void quantize_span(int type, const float* x, int64_t elems, void* out) {
  switch (type) {
    case GGML_Q4_0: q4_0_from_float(x, elems, (BlkQ4_0*)out); break;
    case GGML_Q4_1: q4_1_from_float(x, elems, (BlkQ4_1*)out); break;
    case GGML_Q5_0: q5_0_from_float(x, elems, (BlkQ5_0*)out); break;
    case GGML_Q5_1: q5_1_from_float(x, elems, (BlkQ5_1*)out); break;
    case GGML_Q8_1: q8_1_from_float(x, elems, (BlkQ8_1*)out); break;
    case GGML_Q8_0: q8_0_from_float(x, elems, (BlkQ8_0*)out); break;
    case GGML_Q2K: q2k_from_float(x, elems, (BlkQ2K*)out); break;
    case GGML_Q3K: q3k_from_float(x, elems, (BlkQ3K*)out); break;
    case GGML_Q4K: q4k_from_float(x, elems, (BlkQ4K*)out); break;
    case GGML_Q5K: q5k_from_float(x, elems, (BlkQ5K*)out); break;
    case GGML_Q6K: q6k_from_float(x, elems, (BlkQ6K*)out); break;
    case GGML_Q8K: q8k_from_float(x, elems, (BlkQ8K*)out); break;
  }
}

void dequantize_span(int type, const void* in, int64_t elems, float* y) {
  switch (type) {
    case GGML_Q4_0: q4_0_to_float((const BlkQ4_0*)in, elems, y); break;
    case GGML_Q4_1: q4_1_to_float((const BlkQ4_1*)in, elems, y); break;
    case GGML_Q5_0: q5_0_to_float((const BlkQ5_0*)in, elems, y); break;
    case GGML_Q5_1: q5_1_to_float((const BlkQ5_1*)in, elems, y); break;
    case GGML_Q8_1: q8_1_to_float((const BlkQ8_1*)in, elems, y); break;
    case GGML_Q8_0: q8_0_to_float((const BlkQ8_0*)in, elems, y); break;
    case GGML_Q2K: q2k_to_float((const BlkQ2K*)in, elems, y); break;
    case GGML_Q3K: q3k_to_float((const BlkQ3K*)in, elems, y); break;
    case GGML_Q4K: q4k_to_float((const BlkQ4K*)in, elems, y); break;
    case GGML_Q5K: q5k_to_float((const BlkQ5K*)in, elems, y); break;
    case GGML_Q6K: q6k_to_float((const BlkQ6K*)in, elems, y); break;
    case GGML_Q8K: q8k_to_float((const BlkQ8K*)in, elems, y); break;
  }
}

float dot(int type, int order, int64_t k, const void* w, const void* a) {
  if (order == 0) {
    switch (type) {
      case GGML_Q4_0: return q4_0_q8_0_dot_scalar(k, (const BlkQ4_0*)w, (const BlkQ8_0*)a);
      case GGML_Q4_1: return q4_1_q8_1_dot_scalar(k, (const BlkQ4_1*)w, (const BlkQ8_1*)a);
      case GGML_Q5_0: return q5_0_q8_0_dot_scalar(k, (const BlkQ5_0*)w, (const BlkQ8_0*)a);
      case GGML_Q5_1: return q5_1_q8_1_dot_scalar(k, (const BlkQ5_1*)w, (const BlkQ8_1*)a);
      case GGML_Q8_0: return q8_0_q8_0_dot_scalar(k, (const BlkQ8_0*)w, (const BlkQ8_0*)a);
      case GGML_Q2K: return q2k_q8k_dot_scalar(k, (const BlkQ2K*)w, (const BlkQ8K*)a);
      case GGML_Q3K: return q3k_q8k_dot_scalar(k, (const BlkQ3K*)w, (const BlkQ8K*)a);
      case GGML_Q4K: return q4k_q8k_dot_scalar(k, (const BlkQ4K*)w, (const BlkQ8K*)a);
      case GGML_Q5K: return q5k_q8k_dot_scalar(k, (const BlkQ5K*)w, (const BlkQ8K*)a);
      case GGML_Q6K: return q6k_q8k_dot_scalar(k, (const BlkQ6K*)w, (const BlkQ8K*)a);
    }
  } else {
    switch (type) {
      case GGML_Q4_0: return q4_0_q8_0_dot_avx2(k, (const BlkQ4_0*)w, (const BlkQ8_0*)a);
      case GGML_Q4_1: return q4_1_q8_1_dot_avx2(k, (const BlkQ4_1*)w, (const BlkQ8_1*)a);
      case GGML_Q5_0: return q5_0_q8_0_dot_avx2(k, (const BlkQ5_0*)w, (const BlkQ8_0*)a);
      case GGML_Q5_1: return q5_1_q8_1_dot_avx2(k, (const BlkQ5_1*)w, (const BlkQ8_1*)a);
      case GGML_Q8_0: return q8_0_q8_0_dot_avx2(k, (const BlkQ8_0*)w, (const BlkQ8_0*)a);
      case GGML_Q2K: return q2k_q8k_dot_avx2(k, (const BlkQ2K*)w, (const BlkQ8K*)a);
      case GGML_Q3K: return q3k_q8k_dot_avx2(k, (const BlkQ3K*)w, (const BlkQ8K*)a);
      case GGML_Q4K: return q4k_q8k_dot_avx2(k, (const BlkQ4K*)w, (const BlkQ8K*)a);
      case GGML_Q5K: return q5k_q8k_dot_avx2(k, (const BlkQ5K*)w, (const BlkQ8K*)a);
      case GGML_Q6K: return q6k_q8k_dot_avx2(k, (const BlkQ6K*)w, (const BlkQ8K*)a);
    }
  }
  return 0.f;
}

}  // namespace

extern "C" {

int fq_oracle_block_elems(int type) {
  Fmt f;
  return fmt_of(type, &f) ? f.block_elems : 0;
}
int fq_oracle_block_bytes(int type) {
  Fmt f;
  return fmt_of(type, &f) ? f.block_bytes : 0;
}
int fq_oracle_act_type(int type) {
  Fmt f;
  return fmt_of(type, &f) ? f.act_type : 0;
}

uint16_t fq_oracle_f32_to_f16(float v) { return f2h(v); }
float fq_oracle_f16_to_f32(uint16_t v) { return h2f(v); }

// from_float over `elems` values (a multiple of the block size). Every block is
// independent in the reference, so blocks are spread over threads.
int fq_oracle_quantize(int type, const float* x, int64_t elems, void* out, int nthreads) {
  Fmt f;
  if (!fmt_of(type, &f) || elems % f.block_elems) return 2;
  const int64_t nb = elems / f.block_elems;
  const int64_t chunk = 64;
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#pragma omp parallel for schedule(dynamic) num_threads(nthreads)
  for (int64_t b0 = 0; b0 < nb; b0 += chunk) {
    const int64_t nbk = (nb - b0 < chunk) ? nb - b0 : chunk;
    quantize_span(type, x + b0 * f.block_elems, nbk * f.block_elems, (uint8_t*)out + b0 * f.block_bytes);
  }
  return 0;
}

int fq_oracle_dequantize(int type, const void* in, int64_t elems, float* y, int nthreads) {
  Fmt f;
  if (!fmt_of(type, &f) || elems % f.block_elems) return 2;
  const int64_t nb = elems / f.block_elems;
  const int64_t chunk = 256;
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#pragma omp parallel for schedule(static) num_threads(nthreads)
  for (int64_t b0 = 0; b0 < nb; b0 += chunk) {
    const int64_t nbk = (nb - b0 < chunk) ? nb - b0 : chunk;
    dequantize_span(type, (const uint8_t*)in + b0 * f.block_bytes, nbk * f.block_elems, y + b0 * f.block_elems);
  }
  return 0;
}

// Activation rows -> the weight format's dot-product partner blocks.
int fq_oracle_quantize_act(int weight_type, const float* x, int64_t m, int64_t k, void* out) {
  Fmt f;
  if (!fmt_of(weight_type, &f) || k % f.block_elems) return 2;
  Fmt a;
  fmt_of(f.act_type, &a);
  const int64_t row_bytes = k / a.block_elems * a.block_bytes;
  for (int64_t r = 0; r < m; ++r) quantize_span(f.act_type, x + r * k, k, (uint8_t*)out + r * row_bytes);
  return 0;
}

float fq_oracle_vec_dot(int type, int order, int64_t k, const void* w, const void* act) {
  return dot(type, order, k, w, act);
}

// dst[m, n] = lhs[m, k] x rhs_t[n, k-blocks]^T. order: 0 = scalar (canonical), 1 = AVX2.
int fq_oracle_matmul(int type, int order, int64_t m, int64_t k, int64_t n, const float* lhs, const void* rhs_t,
                     float* dst, int nthreads) {
  Fmt f;
  if (!fmt_of(type, &f) || type == GGML_Q8K || k % f.block_elems) return 2;
  if (m == 0 || n == 0) return 0;
  Fmt a;
  fmt_of(f.act_type, &a);
  const int64_t act_row_bytes = k / a.block_elems * a.block_bytes;
  const int64_t w_row_bytes = k / f.block_elems * f.block_bytes;
  std::vector<uint8_t> act((size_t)(m * act_row_bytes));
  for (int64_t r = 0; r < m; ++r) quantize_span(f.act_type, lhs + r * k, k, act.data() + r * act_row_bytes);
  if (nthreads <= 0) nthreads = omp_get_max_threads();
  for (int64_t r = 0; r < m; ++r) {
    const uint8_t* arow = act.data() + r * act_row_bytes;
    float* drow = dst + r * n;
#pragma omp parallel for schedule(static, 128) num_threads(nthreads)
    for (int64_t c = 0; c < n; ++c) drow[c] = dot(type, order, k, (const uint8_t*)rhs_t + c * w_row_bytes, arow);
  }
  return 0;
}

int fq_oracle_max_threads() { return omp_get_max_threads(); }

}  // extern "C"
