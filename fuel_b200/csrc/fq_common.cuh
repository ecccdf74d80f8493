// Shared definitions for the sm_100a quantized-matmul kernels: GGUF block layouts,
// status codes, the internal activation layout, and thin PTX wrappers
// (mbarrier, 1-D bulk TMA copies, programmatic dependent launch).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fq {

// ---- status codes: the reference's FFI convention for kernel providers
// (fuel-cuda-backend/src/baracuda/status.rs:5-12) plus one for a bounded wait that expired.
enum Status : int32_t {
  kOk = 0,
  kMisaligned = 1,
  kInvalidProblem = 2,
  kNotSupported = 3,
  kWorkspace = 4,
  kLaunchFailure = 5,
};

// ---- GGUF type ids (fuel-ir/src/quantized.rs:35-75)
enum GgmlType : int32_t { kF32 = 0, kF16 = 1, kQ4_0 = 2, kQ4_1 = 3, kQ5_0 = 6, kQ5_1 = 7, kQ8_0 = 8, kQ8_1 = 9, kQ2K = 10, kQ3K = 11, kQ4K = 12, kQ5K = 13, kQ6K = 14, kQ8K = 15, kBF16 = 30 };

constexpr int QK_K = 256;
constexpr int QK_S = 32;

// Byte layouts (fuel-quantized/src/k_quants.rs:56-169). Offsets only; the kernels
// address blocks by byte because Q6_K / Q8_0 / Q4_0 rows are only 2-byte aligned.
struct Q4_0L { static constexpr int kBytes = 18, kElems = 32, kOffD = 0, kOffQs = 2; };
struct Q4_1L { static constexpr int kBytes = 20, kElems = 32, kOffD = 0, kOffM = 2, kOffQs = 4; };
struct Q5_0L { static constexpr int kBytes = 22, kElems = 32, kOffD = 0, kOffQh = 2, kOffQs = 6; };
struct Q5_1L { static constexpr int kBytes = 24, kElems = 32, kOffD = 0, kOffM = 2, kOffQh = 4, kOffQs = 8; };
struct Q8_0L { static constexpr int kBytes = 34, kElems = 32, kOffD = 0, kOffQs = 2; };
struct Q8_1L { static constexpr int kBytes = 36, kElems = 32, kOffD = 0, kOffS = 2, kOffQs = 4; };
struct Q2KL { static constexpr int kBytes = 84, kElems = 256, kOffScales = 0, kOffQs = 16, kOffD = 80, kOffDmin = 82; };
struct Q3KL { static constexpr int kBytes = 110, kElems = 256, kOffHmask = 0, kOffQs = 32, kOffScales = 96, kOffD = 108; };
struct Q4KL { static constexpr int kBytes = 144, kElems = 256, kOffD = 0, kOffDmin = 2, kOffScales = 4, kOffQs = 16; };
struct Q5KL { static constexpr int kBytes = 176, kElems = 256, kOffD = 0, kOffDmin = 2, kOffScales = 4, kOffQh = 16, kOffQs = 48; };
struct Q6KL { static constexpr int kBytes = 210, kElems = 256, kOffQl = 0, kOffQh = 128, kOffScales = 192, kOffD = 208; };
struct Q8KL { static constexpr int kBytes = 292, kElems = 256, kOffD = 0, kOffQs = 4, kOffBsums = 260; };

__host__ __device__ inline int block_elems(int t) {
  switch (t) {
    case kQ4_0: case kQ4_1: case kQ5_0: case kQ5_1: case kQ8_0: case kQ8_1: return 32;
    case kQ2K: case kQ3K: case kQ4K: case kQ5K: case kQ6K: case kQ8K: return 256;
    default: return 0;
  }
}
__host__ __device__ inline int block_bytes(int t) {
  switch (t) {
    case kQ4_0: return 18;
    case kQ4_1: return 20;
    case kQ5_0: return 22;
    case kQ5_1: return 24;
    case kQ8_1: return 36;
    case kQ8_0: return 34;
    case kQ2K: return 84;
    case kQ3K: return 110;
    case kQ4K: return 144;
    case kQ5K: return 176;
    case kQ6K: return 210;
    case kQ8K: return 292;
    default: return 0;
  }
}
// The reference quantizes activations to the weight format's dot-product partner
// (GgmlType::VecDotType, k_quants.rs:174,275,380,491,608,1372,1930): Q8_K for k-quants, Q8_1 for the formats with a
// per-block minimum (Q4_1, Q5_1), Q8_0 otherwise.
__host__ __device__ inline int act_type_for(int t) {
  return (t == kQ2K || t == kQ3K || t == kQ4K || t == kQ5K || t == kQ6K) ? kQ8K : (t == kQ4_1 || t == kQ5_1) ? kQ8_1 : kQ8_0;
}

// ---- internal activation layout ("packed"): the same numbers as the reference's
// Q8_K / Q8_0 blocks, split into planes so every plane is 16-byte aligned:
//   qs    int8  [m][k]
//   d     f32   [m][k / act_block]      (for Q8_0: the f16-rounded scale widened to f32)
//   bsums int16 [m][k / 16]             (Q8_K only)
//         Q8_1 instead keeps, in the same slot, f32 [m][k / 32]: the block's s = d * sum(q), f16-rounded as the
//         reference stores it (k_quants.rs:728-757), widened to f32 (same byte count as the int16 plane)
struct ActPlanes {
  const int8_t* qs;
  const float* d;
  const int16_t* bsums;
};
__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
__host__ __device__ inline size_t act_packed_bytes(int weight_type, int64_t m, int64_t k) {
  const int at = act_type_for(weight_type);
  const int be = block_elems(at);
  size_t b = align_up((size_t)m * k, 256) + align_up((size_t)m * (k / be) * 4, 256);
  if (at == kQ8K || at == kQ8_1) b += align_up((size_t)m * (k / 16) * 2, 256);
  return b;
}
__host__ __device__ inline ActPlanes act_planes(void* base, int weight_type, int64_t m, int64_t k) {
  const int at = act_type_for(weight_type);
  const int be = block_elems(at);
  uint8_t* p = (uint8_t*)base;
  ActPlanes a;
  a.qs = (const int8_t*)p;
  p += align_up((size_t)m * k, 256);
  a.d = (const float*)p;
  p += align_up((size_t)m * (k / be) * 4, 256);
  a.bsums = (at == kQ8K || at == kQ8_1) ? (const int16_t*)p : nullptr;
  return a;
}

// ---- device-side error word. A kernel whose bounded wait expires records where it
// gave up here and returns; the host reads it with fuelq_device_error().
enum DevErr : int { kErrNone = 0, kErrFullWait = 1, kErrEmptyWait = 2, kErrDrainWait = 3, kErrMmaWait = 4, kErrTmemWait = 5, kErrPeerWait = 6 };

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  // the last operand is a suspend-time hint in ns: the thread may sleep in hardware up to that
  // long waiting for the phase instead of spinning through issue slots
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may suspend up to the hint above and then backs off, so
// the default bound is about two seconds) and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 1500000u) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 2) __nanosleep(i < 64 ? 40 : 400);  // back off: waiting warps should not eat issue slots
  }
  return false;
}
// The same for a producer thread that must react at once: a thread suspended on the long hint above was measured
// to wake only when other warps of its thread block became active (microseconds after the phase completed, while
// they sat in griddepcontrol.wait), which left rings half empty. Short suspends, polled; about two seconds in all.
__device__ __forceinline__ bool mbar_try_wait_short(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(200u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_poll_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < 8000000u; ++i) {
    if (mbar_try_wait_short(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Bulk prefetch of a global range into L2 (no shared-memory destination, no completion to wait on).
// Address 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start before its predecessor finishes; it must not touch data the
// predecessor writes until pdl_wait() returns. Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streams a weight buffer from HBM into L2 ahead of the kernel that will read it. Launched
// with programmatic dependent launch it runs beside the PREVIOUS mat-vec, so the HBM transfer
// of the next matrix overlaps the current one's arithmetic and the dependency bubble between
// kernels. It ends with pdl_wait() so that kernels ordered after it still wait, transitively,
// for everything before it.
__global__ void __launch_bounds__(32) prefetch_l2_kernel(const uint8_t* __restrict__ w, long long bytes) {
  pdl_launch_dependents();
  const long long chunk = 4096;
  const long long n_chunks = (bytes & ~15ll) / chunk;
  const long long per = (n_chunks + gridDim.x - 1) / gridDim.x;
  const long long c0 = per * blockIdx.x;
  long long c1 = c0 + per;
  if (c1 > n_chunks) c1 = n_chunks;
  for (long long c = c0 + threadIdx.x; c < c1; c += 32) bulk_prefetch_l2(w + c * chunk, (uint32_t)chunk);
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    const long long done = n_chunks * chunk, rest = (bytes & ~15ll) - done;
    if (rest > 0) bulk_prefetch_l2(w + done, (uint32_t)rest);
  }
  pdl_wait();
}


// n f32 words from device memory to a device-mapped host buffer (or any other place), 16 bytes per thread where
// both addresses allow it: the write-back of a small result without a copy-engine hand-off.
__global__ void __launch_bounds__(256) copy_out_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, long long n,
                                                           int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x, nt = (long long)gridDim.x * blockDim.x;
  if (vec) {
    const long long n4 = n >> 2;
    for (long long i = t; i < n4; i += nt) reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    for (long long i = (n4 << 2) + t; i < n; i += nt) dst[i] = src[i];
  } else {
    for (long long i = t; i < n; i += nt) dst[i] = src[i];
  }
}

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

// unaligned-by-2 32-bit read from shared memory: two aligned words and a funnel shift
__device__ __forceinline__ uint32_t lds_u32_2b(const uint8_t* p) {
  const uint32_t a = smem_u32(p);
  const uint32_t base = a & ~3u;
  uint32_t lo, hi;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lo) : "r"(base));
  asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(hi) : "r"(base));
  return __funnelshift_r(lo, hi, (a & 2u) * 8u);
}
__device__ __forceinline__ uint32_t lds_u16(const uint8_t* p) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(smem_u32(p)));
  return v;
}
__device__ __forceinline__ float h2f_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// defined once: the library is a single translation unit
__device__ int g_fq_dev_error = 0;
__device__ __forceinline__ void record_dev_error(int code) { atomicCAS(&g_fq_dev_error, 0, code); }

#endif  // __CUDACC__

}  // namespace fq
