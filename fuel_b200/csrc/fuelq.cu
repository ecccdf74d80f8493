// libfuelq.so — C ABI over the sm_100a kernels (see include/fuelq.h for the contract).
// Single translation unit: the kernels live in the .cuh files included below.
#include "../../include/fuelq.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "decode.cuh"
#include "decode_regs.cuh"
#include "dequantize.cuh"
#include "fq_common.cuh"
#include "llama_glue.cuh"
#include "mma_batch.cuh"
#include "moe.cuh"
#include "moe_mma.cuh"
#include "plain_gemm.cuh"
#include "prefill.cuh"
#include "quantize_act.cuh"
#include "quantize_weights.cuh"

namespace fq {

namespace {

struct Options {
  int64_t pdl = 0;
  int64_t decode_max_m = 0;   // crossover to the tensor-core GEMM; 0 = the library's choice (see prefill_available)
  int64_t decode_grid = 0;
  int64_t dbg_stage_kb = 0, dbg_max_stages = 0, dbg_smem_kb = 0;
  int64_t l2_prefetch = 0;
  int64_t dbg_depth = 0;
  int64_t dbg_pre = -1;
  int64_t decode_kernel = 0;  // 0 auto, 1 generic (activations through L1), 2 register-resident only
  int64_t moe_kernel = 0;     // development switch: 1 = grouped mat-vec on the dp4a kernel even where the tensor-core form fits
  int64_t peer_wait_ms = 4000; // deadline of the exchange polls in the tensor-parallel kernels
  int64_t prefill_tf32 = 0;   // tensor-core path in tf32 instead of 16-bit operands
  int64_t prefill_bf16 = 0;   // 16-bit operands as bf16 instead of f16
  int64_t fused_quant = 0;    // f32 activations with m <= 2: quantize inside the mat-vec kernel
  int64_t dbg_mb_groups = 0, dbg_mb_min_m = 2, dbg_mb_rpc = 0;
  int64_t dbg_host_wb = 0;     // write-back to a host buffer: 0 = by launch mode, 1 = own kernel, 2 = inside the mat-vec kernel
  int64_t dbg_host_early = 1;  // host activations loaded before the wait for earlier kernels
  int64_t dbg_slab_kb = 0;     // tensor-core path through dequantized slabs: slab size in KiB (0 = 128 MiB)
  int64_t prefill_one_kernel = 0;  // Q4_K / Q6_K / Q8_0 dequantized inside the GEMM kernel instead of by slabs
  int64_t dbg_no_split = 0;    // the slab GEMM's last partial round of tiles is not cut into pieces
};
Options g_opt;

struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
};
DeviceInfo g_dev[64];

bool device_info(DeviceInfo** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  DeviceInfo& d = g_dev[dev];
  if (d.sm_count == 0) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
    if (cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess)
      return false;
  }
  *out = &d;
  return true;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

bool supported_weight(int t) {
  return t == kQ4_0 || t == kQ4_1 || t == kQ5_0 || t == kQ5_1 || t == kQ8_0 || t == kQ2K || t == kQ3K || t == kQ4K || t == kQ5K ||
         t == kQ6K;
}

// launch with or without the programmatic-dependent-launch attribute
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ------------------------------------------------------------------ activation quantization
int32_t quantize_act_impl(int weight_type, int64_t m, int64_t k, const float* x, void* ref_out, void* packed,
                          cudaStream_t stream, unsigned* zero_word = nullptr, bool early_x = false) {
  if (!supported_weight(weight_type)) return kNotSupported;
  const int at = act_type_for(weight_type);
  const int be = block_elems(at);
  if (m < 0 || k <= 0 || k % be) return kInvalidProblem;
  if (m == 0) return kOk;
  if (!x || (!ref_out && !packed)) return kInvalidProblem;
  if (!aligned(x, 16)) return kMisaligned;
  const int64_t total = m * k;
  const int warps_per_cta = 8;
  if (at == kQ8K) {
    const int64_t nb = total / QK_K;
    const dim3 grid((unsigned)((nb + warps_per_cta - 1) / warps_per_cta)), block(32 * warps_per_cta);
    cudaError_t e;
    if (ref_out) {
      if (!aligned(ref_out, 4)) return kMisaligned;
      e = launch(quantize_q8k_kernel<true>, grid, block, 0, stream, x, nb, (uint8_t*)ref_out, (int8_t*)nullptr,
                 (float*)nullptr, (int16_t*)nullptr, zero_word, (int)early_x);
    } else {
      ActPlanes a = act_planes(packed, weight_type, m, k);
      e = launch(quantize_q8k_kernel<false>, grid, block, 0, stream, x, nb, (uint8_t*)nullptr, (int8_t*)a.qs,
                 (float*)a.d, (int16_t*)a.bsums, zero_word, (int)early_x);
    }
    return e == cudaSuccess ? kOk : kLaunchFailure;
  }
  const int64_t nb32 = total / QK_S;
  const int64_t ng = (total + QK_K - 1) / QK_K;
  const dim3 grid((unsigned)((ng + warps_per_cta - 1) / warps_per_cta)), block(32 * warps_per_cta);
  cudaError_t e;
  if (at == kQ8_1) {
    if (ref_out) {
      if (!aligned(ref_out, 4)) return kMisaligned;
      e = launch(quantize_q8_0_kernel<true, true>, grid, block, 0, stream, x, ng, nb32, (uint8_t*)ref_out, (int8_t*)nullptr,
                 (float*)nullptr, zero_word, (int)early_x, (float*)nullptr);
    } else {
      ActPlanes a = act_planes(packed, weight_type, m, k);
      e = launch(quantize_q8_0_kernel<false, true>, grid, block, 0, stream, x, ng, nb32, (uint8_t*)nullptr, (int8_t*)a.qs,
                 (float*)a.d, zero_word, (int)early_x, (float*)a.bsums);
    }
  } else if (ref_out) {
    if (!aligned(ref_out, 2)) return kMisaligned;
    e = launch(quantize_q8_0_kernel<true, false>, grid, block, 0, stream, x, ng, nb32, (uint8_t*)ref_out, (int8_t*)nullptr,
               (float*)nullptr, zero_word, (int)early_x, (float*)nullptr);
  } else {
    ActPlanes a = act_planes(packed, weight_type, m, k);
    e = launch(quantize_q8_0_kernel<false, false>, grid, block, 0, stream, x, ng, nb32, (uint8_t*)nullptr, (int8_t*)a.qs,
               (float*)a.d, zero_word, (int)early_x, (float*)nullptr);
  }
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ------------------------------------------------------------------ decode mat-vec
struct DecodePlan {
  int rows_per_stage, nseg, num_stages, stage_stride, grid;
  size_t smem;
};

// Stage sizing: whole rows per stage; eight or more work items per stage so every consumer
// warp has one. Short rows: a multiple of 8 rows. Long rows: fewer rows, each cut into
// k-segments (4 rows x 2, 2 x 4, 1 x 8).
int32_t plan_decode(int type, int64_t n, int64_t k, const DeviceInfo& di, DecodePlan* pl) {
  const int row_bytes = (int)(k / block_elems(type) * block_bytes(type));
  const size_t header = align_up(sizeof(DecodeSmemHeader), 128);
  const size_t per_cta_budget = ((size_t)di.max_smem_optin + 1024) / 2 - 1024 - 512;  // two CTAs per SM
  const size_t ring_budget = per_cta_budget - header;
  const int stage_target = 24 * 1024;
  int fit = (stage_target - 32) / row_bytes;
  if (fit < 8 && 8 * row_bytes + 32 <= 32 * 1024) fit = 8;  // a row per consumer warp beats splitting rows along k (3 KB rows)
  int R, nseg;
  if (fit >= 8) {
    R = fit & ~7;
    if (R > 32) R = 32;
    nseg = 1;
  } else if (fit >= 4) {
    R = 4, nseg = 2;
  } else if (fit >= 2) {
    R = 2, nseg = 4;
  } else {
    R = 1, nseg = 8;
  }
  const int stride = (int)align_up((size_t)R * row_bytes + 32, 128);
  int stages = (int)(ring_budget / stride);
  if (stages < 2) {  // very long rows: one CTA per SM
    const size_t big = (size_t)di.max_smem_optin - header;
    stages = (int)(big / stride);
    if (stages < 2) return kNotSupported;
  }
  if (stages > kDecodeMaxStages) stages = kDecodeMaxStages;
  int grid = g_opt.decode_grid > 0 ? (int)g_opt.decode_grid : 2 * di.sm_count;
  if (grid > n) grid = (int)n;
  pl->rows_per_stage = R;
  pl->nseg = nseg;
  pl->num_stages = stages;
  pl->stage_stride = stride;
  pl->grid = grid;
  pl->smem = header + (size_t)stages * stride;
  return kOk;
}

template <class Fmt>
cudaError_t launch_decode_fmt(const DecodeParams& p, const DecodePlan& pl, cudaStream_t stream) {
  void (*kern)(const DecodeParams) = nullptr;
  if (p.m == 1)
    kern = decode_matvec_kernel<Fmt, 1>;
  else if (p.m == 2)
    kern = decode_matvec_kernel<Fmt, 2>;
  else if (p.m <= 4)
    kern = decode_matvec_kernel<Fmt, 4>;
  else
    kern = decode_matvec_kernel<Fmt, 8>;
  // raise the dynamic shared-memory limit once per (kernel, device) to the most any plan uses
  static bool attr_set[4][64] = {};
  const int slot = p.m == 1 ? 0 : p.m == 2 ? 1 : p.m <= 4 ? 2 : 3;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[slot][dev]) {
    DeviceInfo* di;
    if (!device_info(&di)) return cudaErrorInvalidDevice;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[slot][dev] = true;
  }
  return launch(kern, dim3(pl.grid), dim3(kDecodeThreads), pl.smem, stream, p);
}

// ---- register-resident variant (decode_regs.cuh): M <= 2, rows that fit NU <= 2 units per lane
struct RegsPlan {
  int rows_per_stage, ks, nu, num_stages, stage_stride, grid;
  size_t smem;
};

// `reserve`: bytes of shared memory kept free after the stage ring (the tensor-parallel form stages its activations there)
int32_t plan_decode_regs(int units_per_row, int row_bytes, int64_t n, const DeviceInfo& di, RegsPlan* pl, size_t reserve = 0,
                         int force_ks = 0) {
  int ks = 1;
  while (ks < 8 && (units_per_row + ks - 1) / ks > 32) ks *= 2;  // one unit per lane if eight slices allow it
  if ((units_per_row + ks - 1) / ks > 64) return kNotSupported;
  const int per_slice = (units_per_row + ks - 1) / ks;
  pl->ks = ks;
  pl->nu = per_slice > 32 ? 2 : 1;
  if (force_ks) pl->ks = ks = force_ks, pl->nu = 1;  // the tree form lays the lanes out itself
  const int n_rgroups = kDecodeConsumerWarps / ks;
  const size_t header = align_up(sizeof(DecodeRegsSmemHeader), 128);
  const size_t per_cta_budget = ((size_t)di.max_smem_optin + 1024) / 2 - 1024 - 512;
  if (reserve + header + 4096 > per_cta_budget) return kNotSupported;
  const size_t ring_budget = (g_opt.dbg_smem_kb ? (size_t)g_opt.dbg_smem_kb * 1024 : per_cta_budget) - header - reserve;
  const int stage_target = g_opt.dbg_stage_kb ? (int)g_opt.dbg_stage_kb * 1024 : 40 * 1024;  // two rows per consumer warp per stage at k = 4096
  int fit = (stage_target - 32) / row_bytes;
  if (fit > 32) fit = 32;
  int R = fit >= n_rgroups ? fit / n_rgroups * n_rgroups : (fit >= 1 ? fit : 1);
  const int stride = (int)align_up((size_t)R * row_bytes + 32, 128);
  int stages = (int)(ring_budget / stride);
  if (stages < 2) return kNotSupported;
  if (stages > kDecodeMaxStages) stages = kDecodeMaxStages;
  if (g_opt.dbg_max_stages && stages > g_opt.dbg_max_stages) stages = (int)g_opt.dbg_max_stages;
  int grid = g_opt.decode_grid > 0 ? (int)g_opt.decode_grid : 2 * di.sm_count;
  if (grid > n) grid = (int)n;
  pl->rows_per_stage = R;
  pl->num_stages = stages;
  pl->stage_stride = stride;
  pl->grid = grid;
  pl->smem = header + (size_t)stages * stride + reserve;
  return kOk;
}

template <class Fmt, int M, int NU>
cudaError_t launch_decode_regs(const DecodeRegsParams& p, const RegsPlan& pl, cudaStream_t stream) {
  static bool attr_set[64] = {};
  auto kern = decode_regs_kernel<Fmt, M, NU>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    DeviceInfo* di;
    if (!device_info(&di)) return cudaErrorInvalidDevice;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch(kern, dim3(pl.grid), dim3(kDecodeThreads), pl.smem, stream, p);
}

template <class Fmt, int NU>
cudaError_t launch_decode_regs_peer(const DecodeRegsParams& p, const DecodeRegsPeer& g, const RegsPlan& pl,
                                    cudaStream_t stream) {
  static bool attr_set[64] = {};
  auto kern = decode_regs_peer_kernel<Fmt, NU>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    DeviceInfo* di;
    if (!device_info(&di)) return cudaErrorInvalidDevice;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch(kern, dim3(pl.grid), dim3(kDecodeThreads), pl.smem, stream, p, g);
}

// returns kNotSupported when this variant does not cover the problem (the caller falls back)
// host_y / host_done: the last thread block to finish also copies y (n words) to the device-mapped host buffer host_y;
// *host_done is a device word that is zero when the kernel starts.
int32_t decode_regs_impl(int type, int64_t m, int64_t n, int64_t k, const void* w, const ActPlanes& planes, float* y,
                         cudaStream_t stream, const DecodeRegsPeer* peer = nullptr, const float* x_f32 = nullptr,
                         float* host_y = nullptr, unsigned* host_done = nullptr) {
  if (peer && m != 1) return kNotSupported;
  if (host_y && (peer || m != 1 || !host_done)) return kNotSupported;
  if (x_f32 && (peer || (type != kQ4K && type != kQ6K))) return kNotSupported;
  if (peer && type == kQ5K) return kNotSupported;
  if (m > 2 || (type != kQ4K && type != kQ5K && type != kQ6K && type != kQ8_0)) return kNotSupported;
  if (type == kQ8_0 && k % 128) return kNotSupported;  // its lane unit is four blocks
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  DecodeRegsParams p;
  p.units_per_row = (int)(k / 128);  // every format's lane unit covers 128 elements
  p.row_bytes = (int)(k / block_elems(type) * block_bytes(type));
  RegsPlan pl;
  // Activations staged in shared memory (quantized in the kernel) are dead
  // once the consumers hold them in registers, so they borrow the LAST stage buffer of the ring: the
  // producer fills that stage only after the consumers report their activations loaded.
  const size_t staged = x_f32 ? align_up(act_packed_bytes(kQ4K, m, k), 128) : 0;
  int32_t st = plan_decode_regs(p.units_per_row, p.row_bytes, n, *di, &pl, 0);
  if (st != kOk) return st;
  size_t reserve = 0;
  if (staged > (size_t)pl.stage_stride || pl.num_stages < 3) {  // does not fit a stage: keep it beside the ring
    reserve = staged;
    st = plan_decode_regs(p.units_per_row, p.row_bytes, n, *di, &pl, reserve);
    if (st != kOk) return st;
  }
  const int staged_off = reserve ? (int)(pl.smem - reserve) : (int)(pl.smem - pl.stage_stride);
  // in-kernel quantization of a small matrix: one thread block per SM (half as many blocks repeat the quantization)
  if (x_f32 && g_opt.decode_grid == 0 && n * (int64_t)p.row_bytes <= (12 << 20) && pl.grid > di->sm_count) pl.grid = di->sm_count;
  p.w = (const uint8_t*)w;
  p.act = planes;
  p.x_f32 = x_f32;
  p.act_smem_off = staged_off;
  p.host_y = host_y;
  p.host_done = host_done;
  p.y = y;
  p.n = n;
  p.k = (int)k;
  p.m = (int)m;
  p.total_bytes = n * (int64_t)p.row_bytes;
  p.rows_per_stage = pl.rows_per_stage;
  p.ks = pl.ks;
  p.num_stages = pl.num_stages;
  p.stage_stride = pl.stage_stride;
  p.rows_q = (int)(n / pl.grid);
  p.rows_rem = (int)(n % pl.grid);
  for (int sl = 0; sl <= 8; ++sl) p.u_begin[sl] = sl <= pl.ks ? (int)((int64_t)p.units_per_row * sl / pl.ks) : p.units_per_row;
  p.depth = g_opt.dbg_depth ? (int)g_opt.dbg_depth : 3;
  if (p.depth >= pl.num_stages) p.depth = pl.num_stages - 1;
  p.pre_stages = g_opt.dbg_pre >= 0 ? (int)g_opt.dbg_pre : 1;  // one weight stage in flight until the activations are held
  if (staged && !reserve) p.pre_stages = pl.num_stages - 1;
  cudaError_t e;
  if (peer) {
#define FQ_REGS_PEER(FMT) \
  e = pl.nu == 1 ? launch_decode_regs_peer<FMT, 1>(p, *peer, pl, stream) : launch_decode_regs_peer<FMT, 2>(p, *peer, pl, stream)
    switch (type) {
      case kQ4K: FQ_REGS_PEER(Q4KRegs); break;
      case kQ6K: FQ_REGS_PEER(Q6KRegs); break;
      default: FQ_REGS_PEER(Q8_0Regs); break;
    }
#undef FQ_REGS_PEER
    return e == cudaSuccess ? kOk : kLaunchFailure;
  }
#define FQ_REGS_DISPATCH(FMT)                                                                                          \
  do {                                                                                                                 \
    if (m == 1)                                                                                                        \
      e = pl.nu == 1 ? launch_decode_regs<FMT, 1, 1>(p, pl, stream) : launch_decode_regs<FMT, 1, 2>(p, pl, stream);    \
    else                                                                                                               \
      e = pl.nu == 1 ? launch_decode_regs<FMT, 2, 1>(p, pl, stream) : launch_decode_regs<FMT, 2, 2>(p, pl, stream);    \
  } while (0)
  switch (type) {
    case kQ4K: FQ_REGS_DISPATCH(Q4KRegs); break;
    case kQ5K: FQ_REGS_DISPATCH(Q5KRegs); break;
    case kQ6K: FQ_REGS_DISPATCH(Q6KRegs); break;
    default: FQ_REGS_DISPATCH(Q8_0Regs); break;
  }
#undef FQ_REGS_DISPATCH
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- tree-ordered mat-vec (decode_regs.cuh, kTree): m = 1, the row's k range cut into n_leaves leaves of
// leaf_blocks[l] 256-element blocks; `peer` scatters the result to every rank
template <class Fmt>
cudaError_t launch_decode_tree(const DecodeRegsParams& p, const DecodeRegsPeer* g, const RegsPlan& pl, cudaStream_t stream) {
  static bool attr_set[2][64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  DeviceInfo* di;
  if (!device_info(&di)) return cudaErrorInvalidDevice;
  if (g) {
    auto kern = decode_regs_tree_peer_kernel<Fmt>;
    if (!attr_set[1][dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
      if (e != cudaSuccess) return e;
      attr_set[1][dev] = true;
    }
    return launch(kern, dim3(pl.grid), dim3(kDecodeThreads), pl.smem, stream, p, *g);
  }
  auto kern = decode_regs_tree_kernel<Fmt>;
  if (!attr_set[0][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[0][dev] = true;
  }
  return launch(kern, dim3(pl.grid), dim3(kDecodeThreads), pl.smem, stream, p);
}

int32_t decode_tree_impl(int type, int64_t n, int64_t k, const void* w, const ActPlanes& planes, float* y, int n_leaves,
                         const int32_t* leaf_blocks, const DecodeRegsPeer* peer, cudaStream_t stream) {
  if (type != kQ4K && type != kQ6K) return kNotSupported;
  if (n_leaves != 1 && n_leaves != 2 && n_leaves != 4 && n_leaves != 8) return kInvalidProblem;
  if (!leaf_blocks || k % 256) return kInvalidProblem;
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  DecodeRegsParams p;
  int64_t blocks = 0;
  int max_units = 1;
  p.leaf_u0[0] = 0;
  for (int l = 0; l < 8; ++l) {
    const int b = l < n_leaves ? leaf_blocks[l] : 0;
    if (b < 0) return kInvalidProblem;
    blocks += b;
    p.leaf_u0[l + 1] = p.leaf_u0[l] + 2 * b;  // a lane unit is half a 256-block
    if (2 * b > max_units) max_units = 2 * b;
  }
  if (blocks * 256 != k) return kInvalidProblem;
  if (max_units > 32) return kNotSupported;
  int lw = 1;
  while (lw < max_units) lw *= 2;
  const int lanes = lw * n_leaves;
  const int ks = lanes <= 32 ? 1 : lanes / 32;
  p.n_leaves = n_leaves;
  p.leaf_lw = lw;
  p.units_per_row = (int)(k / 128);
  p.row_bytes = (int)(k / 256 * block_bytes(type));
  RegsPlan pl;
  const int32_t st = plan_decode_regs(p.units_per_row, p.row_bytes, n, *di, &pl, 0, ks);
  if (st != kOk) return st;
  p.w = (const uint8_t*)w;
  p.act = planes;
  p.x_f32 = nullptr;
  p.host_y = nullptr;
  p.host_done = nullptr;
  p.act_smem_off = 0;
  p.y = y;
  p.n = n;
  p.k = (int)k;
  p.m = 1;
  p.total_bytes = n * (int64_t)p.row_bytes;
  p.rows_per_stage = pl.rows_per_stage;
  p.ks = pl.ks;
  p.num_stages = pl.num_stages;
  p.stage_stride = pl.stage_stride;
  p.rows_q = (int)(n / pl.grid);
  p.rows_rem = (int)(n % pl.grid);
  for (int sl = 0; sl <= 8; ++sl) p.u_begin[sl] = 0;
  p.depth = g_opt.dbg_depth ? (int)g_opt.dbg_depth : 3;
  if (p.depth >= pl.num_stages) p.depth = pl.num_stages - 1;
  p.pre_stages = g_opt.dbg_pre >= 0 ? (int)g_opt.dbg_pre : 1;  // one weight stage in flight until the activations are held
  const cudaError_t e = type == kQ4K ? launch_decode_tree<Q4KRegs>(p, peer, pl, stream)
                                     : launch_decode_tree<Q6KRegs>(p, peer, pl, stream);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t decode_impl(int type, int64_t m, int64_t n, int64_t k, const void* w, const ActPlanes& planes, float* y,
                    cudaStream_t stream) {
  if (g_opt.decode_kernel != 1) {
    const int32_t st = decode_regs_impl(type, m, n, k, w, planes, y, stream);
    if (st != kNotSupported || g_opt.decode_kernel == 2) return st;
  }
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  DecodePlan pl;
  const int32_t st = plan_decode(type, n, k, *di, &pl);
  if (st != kOk) return st;
  DecodeParams p;
  p.w = (const uint8_t*)w;
  p.act = planes;
  p.y = y;
  p.n = n;
  p.k = (int)k;
  p.m = (int)m;
  p.row_bytes = (int)(k / block_elems(type) * block_bytes(type));
  p.total_bytes = n * (int64_t)p.row_bytes;
  p.rows_per_stage = pl.rows_per_stage;
  p.nseg = pl.nseg;
  p.num_stages = pl.num_stages;
  p.stage_stride = pl.stage_stride;
  cudaError_t e;
  switch (type) {
    case kQ4K:
      p.units_per_row = (int)(k / 256) * Q4KDecode::kUnitsPerBlock;
      e = launch_decode_fmt<Q4KDecode>(p, pl, stream);
      break;
    case kQ6K:
      p.units_per_row = (int)(k / 256) * Q6KDecode::kUnitsPerBlock;
      e = launch_decode_fmt<Q6KDecode>(p, pl, stream);
      break;
    case kQ8_0:
      p.units_per_row = (int)(k / 32);
      e = launch_decode_fmt<Q8_0Decode>(p, pl, stream);
      break;
    case kQ4_0:
      p.units_per_row = (int)(k / 32);
      e = launch_decode_fmt<Q4_0Decode>(p, pl, stream);
      break;
    case kQ2K:
      p.units_per_row = (int)(k / 256) * Q2KDecode::kUnitsPerBlock;
      e = launch_decode_fmt<Q2KDecode>(p, pl, stream);
      break;
    case kQ3K:
      p.units_per_row = (int)(k / 256) * Q3KDecode::kUnitsPerBlock;
      e = launch_decode_fmt<Q3KDecode>(p, pl, stream);
      break;
    case kQ4_1:
      p.units_per_row = (int)(k / 32);
      e = launch_decode_fmt<Q4_1Decode>(p, pl, stream);
      break;
    case kQ5_0:
      p.units_per_row = (int)(k / 32);
      e = launch_decode_fmt<Q5_0Decode>(p, pl, stream);
      break;
    case kQ5_1:
      p.units_per_row = (int)(k / 32);
      e = launch_decode_fmt<Q5_1Decode>(p, pl, stream);
      break;
    default:
      return kNotSupported;
  }
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// The address at which kernels on the current device can read or write a host buffer in place: non-null only for
// page-locked memory that is mapped into the device's address space. Pageable memory (and anything the driver
// does not know) gives null, and the caller copies instead.
void* mapped_alias(const void* host_ptr) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, host_ptr) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

// Weight stream-in ahead of use (see prefetch_l2_kernel). One small CTA per SM.
int32_t prefetch_impl(const void* w, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return kOk;
  if (!w) return kInvalidProblem;
  if (!aligned(w, 16)) return kMisaligned;
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  const cudaError_t e = launch(prefetch_l2_kernel, dim3(di->sm_count), dim3(32), 0, stream, (const uint8_t*)w,
                               (long long)bytes);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// Tensor-core form (Q4_K): kNotSupported when the shared-memory plan does not fit, so the caller can fall back.
int32_t moe_mma_impl(int n_groups, int64_t n, int64_t k, const void* w, const ActPlanes& act, const int* offsets,
                     int fixed_rows, const int* out_rows, float* y, cudaStream_t stream) {
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  MmaParams p;
  p.row_bytes = (int)(k / 256 * Q4KL::kBytes);
  const size_t header = align_up(sizeof(MmaSmemHeader), 128);
  const size_t per_cta = ((size_t)di->max_smem_optin + 1024) / 2 - 1024 - 512;
  const size_t part_bytes = kDecodeConsumerWarps * 128 * sizeof(float);
  // k in as few chunks as shared memory allows: one chunk of the activation rows plus two stages of eight weight rows
  const int nblk = (int)(k / 256);
  int R = 0, kc_blocks = 0;
  size_t stride = 0, act_bytes = 0, ring = 0;
  for (int chunks = 1; chunks <= 16 && !R; ++chunks) {
    const int kc = (nblk + chunks - 1) / chunks;
    const size_t ab = mma_act_bytes(kc);
    if (header + ab + part_bytes >= per_cta) continue;
    const size_t rg = per_cta - header - ab - part_bytes;
    for (int cand = 32; cand >= 8; cand >>= 1) {
      const size_t st = align_up((size_t)cand * (kc * Q4KL::kBytes + 16), 128);
      if (2 * st <= rg) {
        R = cand, stride = st, kc_blocks = kc, act_bytes = ab, ring = rg;
        break;
      }
    }
  }
  if (!R) return kNotSupported;
  int stages = (int)(ring / stride);
  if (stages > 4) stages = 4;
  p.w = (const uint8_t*)w;
  p.act = act;
  p.offsets = offsets;
  p.fixed_rows = fixed_rows;
  p.out_rows = out_rows;
  p.y = y;
  p.n = (int)n;
  p.k = (int)k;
  p.group_bytes = n * (int64_t)p.row_bytes;
  p.rows_per_stage = R;
  p.num_stages = stages;
  p.stage_stride = (int)stride;
  p.act_off = (int)(header + (size_t)stages * stride);
  p.part_off = (int)(p.act_off + act_bytes);
  p.kc_blocks = kc_blocks;
  int per_group = ((kc_blocks < nblk ? 2 : 4) * di->sm_count + n_groups - 1) / n_groups;
  const int max_per = (int)((n + R - 1) / R);
  if (per_group > max_per) per_group = max_per;
  if (per_group < 1) per_group = 1;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kLaunchFailure;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(mma_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin) != cudaSuccess)
      return kLaunchFailure;
    attr_set[dev] = true;
  }
  const size_t smem = header + (size_t)stages * stride + act_bytes + part_bytes;
  const cudaError_t e = launch(mma_q4k_kernel, dim3((unsigned)per_group, (unsigned)n_groups), dim3(kDecodeThreads), smem, stream, p);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- small batches on the integer tensor cores (mma_batch.cuh): Q4_K, Q5_K, Q6_K, Q8_0; k a multiple of 256
template <class F, int MT>
cudaError_t launch_mma_batch(const MmaBatchParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  static bool attr_set[64] = {};
  auto kern = mma_batch_kernel<F, MT>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    DeviceInfo* di;
    if (!device_info(&di)) return cudaErrorInvalidDevice;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch(kern, grid, dim3(kMbThreads), smem, stream, p);
}

template <class F>
int32_t mma_batch_fmt(int n_groups, int64_t n, int64_t k, const void* w, const ActPlanes& act, const int* offsets, int fixed_rows,
                      const int* out_rows, float* y, bool wide, cudaStream_t stream) {
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  const int nblk = (int)(k / 256);
  const int act_rows = wide ? 16 : 8;
  const size_t header = align_up(sizeof(MmaBatchHeader), 128);
  const size_t part_bytes = (size_t)kMbConsumerWarps * (wide ? 2 : 1) * 128 * sizeof(float);
  const size_t total = (size_t)di->max_smem_optin;
  // k in as few sweeps as shared memory allows: the activation rows of one sweep plus at least two (preferably four) stages of 16 weight rows
  MmaBatchParams p;
  const int R = 16;
  int kc_blocks = 0, stages = 0;
  size_t stride = 0, act_bytes = 0;
  int wstride = 0;
  // fewest sweeps over k first; within that, at least three stages (two at the very least)
  int rpc = 1;
  for (int chunks = 1; chunks <= 64 && !kc_blocks; ++chunks) {
    const int kc = (nblk + chunks - 1) / chunks;
    const size_t ab = (size_t)mb_act_layout<F>(kc, act_rows).bytes;
    // whole rows staged: consecutive rows travel in one bulk copy (2 per copy; 4 for short rows)
    rpc = chunks == 1 ? (g_opt.dbg_mb_rpc ? (int)g_opt.dbg_mb_rpc : (nblk * F::kBytes256 <= 1536 ? 4 : 2)) : 1;
    // a staged copy: its bytes widened to 16-byte boundaries, placed so that consecutive copies are 16 bytes apart modulo 128
    const int ws = (int)align_up((size_t)(rpc - 1) * nblk * F::kBytes256 + (size_t)kc * F::kBytes256 + 32, 128) + 16;
    const size_t st = align_up((size_t)(R / rpc) * ws, 128);
    const int min_stages = chunks < 4 ? 3 : 2;
    if (header + ab + part_bytes + (size_t)min_stages * st <= total) {
      kc_blocks = kc, act_bytes = ab, wstride = ws, stride = st;
      stages = (int)((total - header - ab - part_bytes) / st);
    }
  }
  if (!kc_blocks) return kNotSupported;
  if (stages > kMbMaxStages) stages = kMbMaxStages;
  if (g_opt.dbg_max_stages && stages > g_opt.dbg_max_stages) stages = (int)g_opt.dbg_max_stages;
  p.w = (const uint8_t*)w;
  p.act = act;
  p.offsets = offsets;
  p.fixed_rows = fixed_rows;
  p.out_rows = out_rows;
  p.y = y;
  p.n = (int)n;
  p.k = (int)k;
  p.row_bytes = nblk * F::kBytes256;
  p.group_bytes = n * (int64_t)p.row_bytes;
  p.total_bytes = (int64_t)n_groups * p.group_bytes;
  p.num_stages = stages;
  // (never more groups than stages: a group must not wait for a slot's next phase before the slot's first use)
  p.n_wgroups = stages >= 4 ? 4 : stages >= 2 ? 2 : 1;
  if (g_opt.dbg_mb_groups && g_opt.dbg_mb_groups <= p.n_wgroups) p.n_wgroups = (int)g_opt.dbg_mb_groups;
  p.stage_stride = (int)stride;
  p.wstride = wstride;
  p.rows_per_copy = rpc;
  p.act_off = (int)(header + (size_t)stages * stride);
  p.part_off = (int)(p.act_off + act_bytes);
  p.kc_blocks = kc_blocks;
  const int n_tiles = (int)((n + 15) / 16);
  int per_group = (di->sm_count + n_groups - 1) / n_groups;
  if (n_groups > 1) per_group = (2 * di->sm_count + n_groups - 1) / n_groups;
  if (g_opt.decode_grid > 0) per_group = (int)g_opt.decode_grid;
  const int max_per = n_tiles;
  if (per_group > max_per) per_group = max_per;
  if (per_group < 1) per_group = 1;
  const size_t smem = header + (size_t)stages * stride + act_bytes + part_bytes;
  const dim3 grid((unsigned)per_group, (unsigned)n_groups);
  const cudaError_t e = wide ? launch_mma_batch<F, 2>(p, grid, smem, stream) : launch_mma_batch<F, 1>(p, grid, smem, stream);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// kNotSupported when the format or shape has no plan here (the caller falls back)
int32_t mma_batch_impl(int type, int n_groups, int64_t n, int64_t k, const void* w, const ActPlanes& act, const int* offsets,
                       int fixed_rows, const int* out_rows, float* y, bool wide, cudaStream_t stream) {
  if (k % 256 || k > (1 << 20) || n > (1 << 24) || n_groups > 65535) return kNotSupported;
  switch (type) {
    case kQ4K: return mma_batch_fmt<MbQ4K>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    case kQ5K: return mma_batch_fmt<MbQ5K>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    case kQ6K: return mma_batch_fmt<MbQ6K>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    case kQ8_0: return mma_batch_fmt<MbQ8_0>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    case kQ4_0: return mma_batch_fmt<MbQ4_0>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    case kQ5_0: return mma_batch_fmt<MbQ5_0>(n_groups, n, k, w, act, offsets, fixed_rows, out_rows, y, wide, stream);
    default: return kNotSupported;
  }
}

// Any m_total through the decode kernels: activation rows are taken kDecodeMaxM at a time, each
// chunk streaming the weights once. Exactly the integer arithmetic of the small-M path.
int32_t decode_chunked(int type, int64_t m_total, int64_t n, int64_t k, const void* w, void* packed_act, float* y,
                       cudaStream_t stream) {
  const ActPlanes all = act_planes(packed_act, type, m_total, k);
  // (Q4_0 / Q5_0 have no register-resident one-row kernel: their single rows take this path too, measured 11.9 against
  // 14.3 us on the generic kernel for 4096 -> 11008)
  if ((m_total >= g_opt.dbg_mb_min_m || type == kQ4_0 || type == kQ5_0) && g_opt.decode_kernel == 0 && g_opt.moe_kernel == 0) {
    // a few rows: one pass over the weights on the integer tensor cores (up to 16 rows per pass)
    const int32_t st = mma_batch_impl(type, 1, n, k, w, all, nullptr, (int)m_total, nullptr, y, m_total > 8, stream);
    if (st != kNotSupported) return st;
  }
  // (when k is so large that the tensor-core kernel sweeps it in chunks, two-row dp4a passes stay ahead up to 5 rows)
  const bool mma_chunked = k / 256 > 16;
  if (type == kQ4K && m_total > (mma_chunked ? 5 : 2) && g_opt.decode_kernel == 0 && g_opt.moe_kernel != 1 && n <= (1 << 24)) {
    // a few rows of Q4_K: one pass over the weights on the integer tensor cores (16 rows per pass)
    const int32_t st = moe_mma_impl(1, n, k, w, all, nullptr, (int)m_total, nullptr, y, stream);
    if (st != kNotSupported) return st;
  }
  const int abe = block_elems(act_type_for(type));
  // Two rows at a time through the register-resident kernel beats sixteen at a time through the generic
  // one when the matrix fits in L2 (every pass after the first streams from there).
  const bool regs_ok = g_opt.decode_kernel != 1 && (type == kQ4K || type == kQ5K || type == kQ6K || (type == kQ8_0 && k % 128 == 0)) &&
                       (k / 128 + 7) / 8 <= 64 && m_total > 2;
  const int64_t step = regs_ok ? 2 : kDecodeMaxM;
  for (int64_t m0 = 0; m0 < m_total; m0 += step) {
    const int64_t mc = m_total - m0 < step ? m_total - m0 : step;
    ActPlanes a;
    a.qs = all.qs + m0 * k;
    a.d = all.d + m0 * (k / abe);
    a.bsums = all.bsums ? all.bsums + m0 * (k / 16) : nullptr;
    const int32_t st = decode_impl(type, mc, n, k, w, a, y + m0 * n, stream);
    if (st != kOk) return st;
  }
  return kOk;
}

// ---- block -> float dequantization (dequantize.cuh)
// out_type: kF32, kF16, kBF16, or the tensor-core path's operands: kF16Sat (f16 with finite overflow saturated) and
// kTf32 (f32 rounded to tf32)
constexpr int kF16Sat = -16, kTf32Out = -32;
int32_t dequantize_impl(int ggml_type, int64_t numel, const void* blocks, void* y, int out_type, cudaStream_t stream) {
  const int be = block_elems(ggml_type);
  if (be == 0) return kNotSupported;
  if (numel < 0 || numel % be) return kInvalidProblem;
  if (out_type != kF32 && out_type != kF16 && out_type != kBF16 && out_type != kF16Sat && out_type != kTf32Out) return kNotSupported;
  if (numel == 0) return kOk;
  if (!blocks || !y) return kInvalidProblem;
  const size_t in_align = (ggml_type == kQ4K || ggml_type == kQ5K) ? 16 : (ggml_type == kQ8K ? 4 : 2);
  if (!aligned(blocks, in_align) || !aligned(y, (out_type == kF32 || out_type == kTf32Out) ? 4 : 2)) return kMisaligned;
  const int64_t nb = numel / be;
  const uint8_t* w = (const uint8_t*)blocks;
  int64_t units;
  switch (ggml_type) {
    case kQ4K: case kQ5K: units = nb * 8; break;
    case kQ6K: units = nb * 16; break;
    case kQ8_0: units = nb * 4; break;
    case kQ4_0: case kQ4_1: case kQ5_0: case kQ5_1: units = nb * 4; break;
    case kQ8K: case kQ2K: case kQ3K: units = nb * 64; break;
    default: return kNotSupported;
  }
  const dim3 block(256), grid((unsigned)((units + 255) / 256));
#define FQ_DEQ(KERNEL)                                                                        \
  do {                                                                                        \
    if (out_type == kF32)                                                                     \
      KERNEL<float><<<grid, block, 0, stream>>>(w, units, (float*)y);                         \
    else if (out_type == kF16)                                                                \
      KERNEL<__half><<<grid, block, 0, stream>>>(w, units, (__half*)y);                       \
    else if (out_type == kF16Sat)                                                             \
      KERNEL<half_sat><<<grid, block, 0, stream>>>(w, units, (half_sat*)y);                   \
    else if (out_type == kTf32Out)                                                            \
      KERNEL<f32_tf32><<<grid, block, 0, stream>>>(w, units, (f32_tf32*)y);                   \
    else                                                                                      \
      KERNEL<__nv_bfloat16><<<grid, block, 0, stream>>>(w, units, (__nv_bfloat16*)y);         \
  } while (0)
  switch (ggml_type) {
    case kQ4K: FQ_DEQ(dequant_q4k_kernel); break;
    case kQ5K: FQ_DEQ(dequant_q5k_kernel); break;
    case kQ6K: FQ_DEQ(dequant_q6k_kernel); break;
    case kQ8_0: FQ_DEQ(dequant_q8_0_kernel); break;
    case kQ4_0: FQ_DEQ(dequant_q4_0_kernel); break;
#define FQ_DEQ_L(L, FIVE, MIN)                                                                                  \
  do {                                                                                                          \
    if (out_type == kF32)                                                                                       \
      dequant_legacy32_kernel<float, L, FIVE, MIN><<<grid, block, 0, stream>>>(w, units, (float*)y);            \
    else if (out_type == kF16)                                                                                  \
      dequant_legacy32_kernel<__half, L, FIVE, MIN><<<grid, block, 0, stream>>>(w, units, (__half*)y);          \
    else if (out_type == kF16Sat)                                                                               \
      dequant_legacy32_kernel<half_sat, L, FIVE, MIN><<<grid, block, 0, stream>>>(w, units, (half_sat*)y);      \
    else if (out_type == kTf32Out)                                                                              \
      dequant_legacy32_kernel<f32_tf32, L, FIVE, MIN><<<grid, block, 0, stream>>>(w, units, (f32_tf32*)y);      \
    else                                                                                                        \
      dequant_legacy32_kernel<__nv_bfloat16, L, FIVE, MIN><<<grid, block, 0, stream>>>(w, units, (__nv_bfloat16*)y); \
  } while (0)
    case kQ4_1: FQ_DEQ_L(Q4_1L, false, true); break;
    case kQ5_0: FQ_DEQ_L(Q5_0L, true, false); break;
    case kQ5_1: FQ_DEQ_L(Q5_1L, true, true); break;
#undef FQ_DEQ_L
    case kQ8K: FQ_DEQ(dequant_q8k_kernel); break;
    case kQ2K: FQ_DEQ(dequant_q2k_kernel); break;
    case kQ3K: FQ_DEQ(dequant_q3k_kernel); break;
  }
#undef FQ_DEQ
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailure;
}


// ---- tensor-core path (prefill.cuh)
// Formats with a dequantizing stage of their own inside the GEMM kernel ...
bool prefill_native_type(int type) { return type == kQ4K || type == kQ6K || type == kQ8_0; }
// ... and those that reach it through a slab of rows dequantized into the operand type by their stand-alone kernels
bool prefill_slab_type(int type) {
  return type == kQ4_0 || type == kQ4_1 || type == kQ5_0 || type == kQ5_1 || type == kQ2K || type == kQ3K || type == kQ5K;
}
bool prefill_available(int type, int64_t m, int64_t n, int64_t k) {
  (void)n;
  int64_t max_m = g_opt.decode_max_m;
  if (max_m == 0) {
    // The library's choice: 16 rows; 64 where the integer tensor-core kernel applies (16 rows per pass over the weights,
    // the later passes from L2) - still faster there than the bf16 GEMM, and the reference's own arithmetic.
    max_m = 16;
    if ((prefill_native_type(type) || type == kQ5K) && g_opt.decode_kernel == 0 && g_opt.moe_kernel == 0 && k % 256 == 0) max_m = 64;
  }
  return (prefill_native_type(type) || prefill_slab_type(type)) && m > max_m && k % kPfTileK == 0 && k <= (1 << 20);
}
// Whether a tensor-core problem goes through a slab: always, unless the caller asked for the one-kernel form of the
// three formats that have in-kernel stages. Measured on 4096 -> 11008, slab against one kernel: Q4_K 59 / 61 us at 128
// rows, 102 / 122 at 512, 232 / 306 at 2048; Q6_K 60 / 124 at 128, 110 / 258 at 512 - the GEMM fed by tensor-map copies
// alone runs near 900 TFLOP/s, which the dequantizing threads of the one-kernel form do not sustain.
bool prefill_uses_slab(int type, int64_t m) {
  (void)m;
  return prefill_slab_type(type) || !g_opt.prefill_one_kernel;
}
// Rows of the dequantized slab: the whole matrix when it fits 128 MiB, else as many 128-row tiles as do
int64_t prefill_slab_rows(int64_t n, int64_t k) {
  const int64_t esz = g_opt.prefill_tf32 ? 4 : 2;
  const int64_t budget = g_opt.dbg_slab_kb ? g_opt.dbg_slab_kb << 10 : (int64_t)128 << 20;
  int64_t rows = budget / (k * esz) / kPfTileN * kPfTileN;
  if (rows < kPfTileN) rows = kPfTileN;
  return rows < n ? rows : n;
}
// the activations in the operand type, then (f16 operands) one unscale factor per row, then the slab
size_t prefill_x_bytes(int64_t m, int64_t k) {
  return align_up((size_t)m * k * (g_opt.prefill_tf32 ? 4 : 2), 256) + align_up((size_t)m * 4, 256);
}
size_t prefill_workspace_bytes(int type, int64_t m, int64_t n, int64_t k) {
  size_t b = prefill_x_bytes(m, k);
  if (prefill_uses_slab(type, m)) b += align_up((size_t)prefill_slab_rows(n, k) * k * (g_opt.prefill_tf32 ? 4 : 2), 256);
  return b;
}

// tensor map of a row-major [rows][K] matrix in the operand type (the activations; weights dequantized into a slab):
// boxes of 128 bytes x tile_m rows, 128-byte swizzle, zero fill
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
bool make_x_map(const void* xb, int64_t m, int64_t k, int tile_m, bool f32, bool f16, CUtensorMap* map) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn)
      return false;
    encode = (EncodeTiledFn)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
  const cuuint64_t strides[1] = {(cuuint64_t)k * (f32 ? 4 : 2)};
  const cuuint32_t box[2] = {(cuuint32_t)(f32 ? 32 : kPfTileK), (cuuint32_t)tile_m};  // 128 bytes x tile_m rows
  const cuuint32_t estr[2] = {1, 1};
  return encode(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xb), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class Fmt, int kTileM, bool kTf32, bool kMulti, bool kF16>
cudaError_t launch_prefill_m(const PrefillParams& p, const void* xb, cudaStream_t stream) {
  constexpr size_t smem = 1024 + (size_t)kPfStages * (kPfTileN * 128 + kTileM * 128) + sizeof(PrefillSmem) + 64;
  static bool attr_set[64] = {};
  auto kern = prefill_gemm_kernel<Fmt, kTileM, kTf32, kMulti, kF16>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  CUtensorMap xmap;
  if (!make_x_map(xb, p.M, p.K, kTileM, kTf32, kF16, &xmap)) return cudaErrorUnknown;
  const dim3 grid((unsigned)((p.N + kPfTileN - 1) / kPfTileN), (unsigned)((p.M + kTileM - 1) / kTileM));
  kern<<<grid, kPfThreads, smem, stream>>>(p, xmap);
  return cudaGetLastError();
}

template <class Fmt, int kTileM, bool kTf32 = false, bool kF16 = false>
cudaError_t launch_prefill(const PrefillParams& p, const void* xb, cudaStream_t stream) {
  return p.n_dst > 1 ? launch_prefill_m<Fmt, kTileM, kTf32, true, kF16>(p, xb, stream)
                     : launch_prefill_m<Fmt, kTileM, kTf32, false, kF16>(p, xb, stream);
}

template <int kTileM, int kStages, bool kTf32, bool kF16, bool kMulti>
cudaError_t launch_plain_gemm_t(PlainGemmParams p, const void* xb, const void* w, int sm_count, cudaStream_t stream) {
  constexpr size_t smem = 1024 + (size_t)kStages * (kPfTileN * 128 + kTileM * 128) + kPgEpilogueWarps * 32 * 36 * 4 +
                          sizeof(PlainGemmSmem<kTileM, kStages>) + 64;
  static bool attr_set[64] = {};
  auto kern = plain_gemm_kernel<kTileM, kStages, kTf32, kF16, kMulti>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  CUtensorMap xmap, wmap;
  if (!make_x_map(xb, p.M, p.K, kTileM, kTf32, kF16, &xmap)) return cudaErrorUnknown;
  if (!make_x_map(w, p.N, p.K, kPfTileN, kTf32, kF16, &wmap)) return cudaErrorUnknown;
  // Work items: whole tiles for the full rounds of thread blocks; the tiles of a last, partly filled round are cut along M
  // into 2 or 4 pieces (at least 64 activation rows each) while the pieces still fit one round.
  const int tiles_n = (p.N + kPfTileN - 1) / kPfTileN;
  p.tiles_m = (p.M + kTileM - 1) / kTileM;
  const int64_t tiles = (int64_t)tiles_n * p.tiles_m;
  const int64_t rounds = tiles / sm_count, rest = tiles % sm_count;
  int split = 0;
  constexpr int kMaxSplit = kTileM == 256 ? 2 : 1;
  if (rest && !g_opt.dbg_no_split)
    while (split < kMaxSplit && (rest << (split + 1)) <= sm_count) ++split;
  const int64_t whole = split ? rounds * sm_count : tiles;
  const int64_t items = whole + ((tiles - whole) << split);
  if (items > INT32_MAX) return cudaErrorInvalidValue;
  p.whole_tiles = (int)whole;
  p.split_log2 = split;
  p.n_items = (int)items;
  const unsigned grid = (unsigned)(items < sm_count ? items : sm_count);
  kern<<<grid, kPgThreads, smem, stream>>>(p, xmap, wmap);
  return cudaGetLastError();
}

// type < 0: `w` is a slab of rows already in the operand type (plain_gemm.cuh); else GGUF blocks dequantized inside the
// kernel (prefill.cuh). The activations are in the workspace
int32_t prefill_gemm(int type, int64_t m, int64_t n, int64_t k, const void* w, float* const* y_dst, int n_dst, int64_t ldy,
                     int64_t n_off, void* workspace, cudaStream_t stream) {
  const bool tf32 = g_opt.prefill_tf32 != 0, f16 = !tf32 && !g_opt.prefill_bf16;
  const void* xb = workspace;
  const float* unscale = (const float*)((const uint8_t*)workspace + align_up((size_t)m * k * (tf32 ? 4 : 2), 256));
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  if (type < 0) {
    PlainGemmParams g;
    for (int q = 0; q < 8; ++q) g.y[q] = q < n_dst ? y_dst[q] : nullptr;
    g.n_dst = n_dst, g.ldy = (int)ldy, g.n_off = (int)n_off;
    g.M = (int)m, g.N = (int)n, g.K = (int)k;
    g.row_unscale = f16 ? unscale : nullptr;
    cudaError_t e;
    const bool multi = n_dst > 1, narrow = m <= 128;
#define FQ_PLAIN(TF32, F16)                                                                                             \
  e = narrow ? (multi ? launch_plain_gemm_t<128, 6, TF32, F16, true>(g, xb, w, di->sm_count, stream)                    \
                      : launch_plain_gemm_t<128, 6, TF32, F16, false>(g, xb, w, di->sm_count, stream))                  \
             : (multi ? launch_plain_gemm_t<256, 4, TF32, F16, true>(g, xb, w, di->sm_count, stream)                    \
                      : launch_plain_gemm_t<256, 4, TF32, F16, false>(g, xb, w, di->sm_count, stream))
    if (tf32)
      FQ_PLAIN(true, false);
    else if (f16)
      FQ_PLAIN(false, true);
    else
      FQ_PLAIN(false, false);
#undef FQ_PLAIN
    return e == cudaSuccess ? kOk : kLaunchFailure;
  }
  PrefillParams p;
  p.row_unscale = f16 ? unscale : nullptr;
  p.w = (const uint8_t*)w;
  for (int q = 0; q < 8; ++q) p.y[q] = q < n_dst ? y_dst[q] : nullptr;
  p.n_dst = n_dst;
  p.ldy = (int)ldy;
  p.n_off = (int)n_off;
  p.M = (int)m;
  p.N = (int)n;
  p.K = (int)k;
  p.row_bytes = type < 0 ? (int)(k * (tf32 ? 4 : 2)) : (int)(k / block_elems(type) * block_bytes(type));
  cudaError_t e;
  // the wide tile halves the weight dequantization per flop, but only pays once it still fills the SMs
  const bool wide = m > 128 && ((n + kPfTileN - 1) / kPfTileN) * ((m + 255) / 256) >= di->sm_count;
#define FQ_PREFILL(FMT)                                                                                                   \
  e = tf32  ? (wide ? launch_prefill<FMT, 256, true>(p, xb, stream) : launch_prefill<FMT, 128, true>(p, xb, stream))      \
      : f16 ? (wide ? launch_prefill<FMT, 256, false, true>(p, xb, stream)                                                \
                    : launch_prefill<FMT, 128, false, true>(p, xb, stream))                                               \
            : (wide ? launch_prefill<FMT, 256>(p, xb, stream) : launch_prefill<FMT, 128>(p, xb, stream))
  switch (type) {
    case kQ4K: FQ_PREFILL(Q4KPrefill); break;
    case kQ6K: FQ_PREFILL(Q6KPrefill); break;
    case kQ8_0: FQ_PREFILL(Q8_0Prefill); break;
    default: return kNotSupported;
  }
#undef FQ_PREFILL
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// y_dst / n_dst / ldy / n_off: see PrefillParams; the plain call passes one destination of width n
int32_t prefill_impl(int type, int64_t m, int64_t n, int64_t k, const void* w, const float* x, float* const* y_dst, int n_dst,
                     int64_t ldy, int64_t n_off, void* workspace, cudaStream_t stream, bool one_kernel = false) {
  const bool tf32 = g_opt.prefill_tf32 != 0, f16 = !tf32 && !g_opt.prefill_bf16;
  void* xb = workspace;  // the activations in the tensor cores' operand type: f16 (rows scaled), bf16, or f32 rounded to tf32
  float* unscale = (float*)((uint8_t*)workspace + align_up((size_t)m * k * (tf32 ? 4 : 2), 256));
  const int64_t n4 = m * k / 4;
  if (tf32)
    f32_to_tf32_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(x, n4, (float*)xb);
  else if (f16)
    f32_to_f16_rows_kernel<<<(unsigned)m, 256, 0, stream>>>(x, (int)k, (__half*)xb, unscale);
  else
    f32_to_bf16_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(x, n4, (__nv_bfloat16*)xb);
  if (cudaGetLastError() != cudaSuccess) return kLaunchFailure;
  if (one_kernel || !prefill_uses_slab(type, m)) return prefill_gemm(type, m, n, k, w, y_dst, n_dst, ldy, n_off, workspace, stream);
  // Dequantize a slab of rows into the operand type (the reference's to_float values in f32, then one rounding), multiply
  // it, take the next slab. Kernels on one stream, so the slab is reused.
  uint8_t* slab = (uint8_t*)workspace + prefill_x_bytes(m, k);
  const int64_t slab_rows = prefill_slab_rows(n, k);
  const int64_t row_bytes = k / block_elems(type) * block_bytes(type);
  const int out_type = tf32 ? kTf32Out : f16 ? kF16Sat : (int)kBF16;
  for (int64_t r0 = 0; r0 < n; r0 += slab_rows) {
    const int64_t rows = n - r0 < slab_rows ? n - r0 : slab_rows;
    int32_t st = dequantize_impl(type, rows * k, (const uint8_t*)w + r0 * row_bytes, slab, out_type, stream);
    if (st != kOk) return st;
    st = prefill_gemm(-1, m, rows, k, slab, y_dst, n_dst, ldy, n_off + r0, workspace, stream);
    if (st != kOk) return st;
  }
  return kOk;
}

int32_t check_problem(int type, int64_t m, int64_t n, int64_t k) {
  if (!supported_weight(type)) return kNotSupported;
  if (m < 0 || n < 0 || k <= 0) return kInvalidProblem;
  if (k % block_elems(type)) return kInvalidProblem;  // every reference entry rejects this (byte_kernels.rs:4768-4773)
  if (k > (1 << 24) || n > ((int64_t)1 << 31)) return kNotSupported;
  return kOk;
}

}  // namespace
}  // namespace fq

using namespace fq;

extern "C" {

const char* fuelq_status_string(int32_t status) {
  switch (status) {
    case kOk: return "success";
    case kMisaligned: return "misaligned operand (16-byte alignment required)";
    case kInvalidProblem: return "invalid problem (non-positive size, k not a multiple of the block size, or null operand)";
    case kNotSupported: return "not supported (type or shape outside what the kernels implement)";
    case kWorkspace: return "workspace too small or null when required";
    case kLaunchFailure: return "internal kernel error (CUDA launch failure)";
    default: return "unknown status code";
  }
}

int32_t fuelq_block_elems(int32_t t) { return block_elems(t); }
int32_t fuelq_block_bytes(int32_t t) { return block_bytes(t); }

int32_t fuelq_set_option(int32_t key, int64_t value) {
  switch (key) {
    case FUELQ_OPT_PDL: g_opt.pdl = value ? 1 : 0; return kOk;
    case FUELQ_OPT_DECODE_MAX_M:
      if (value < 0) return kInvalidProblem;
      g_opt.decode_max_m = value;
      return kOk;
    case FUELQ_OPT_DECODE_GRID:
      if (value < 0 || value > 65535) return kInvalidProblem;
      g_opt.decode_grid = value;
      return kOk;
    case FUELQ_OPT_DECODE_KERNEL:
      if (value < 0 || value > 2) return kInvalidProblem;
      g_opt.decode_kernel = value;
      return kOk;
    // keys >= 100: development switches for tuning runs (stage size, ring depth, warp groups, which write-back form ...);
    // not part of the contract, every default is what measured best
    case 102: g_opt.dbg_stage_kb = value; return kOk;
    case 103: g_opt.dbg_max_stages = value; return kOk;
    case 104: g_opt.dbg_smem_kb = value; return kOk;
    case 105: g_opt.dbg_depth = value; return kOk;
    case 106: g_opt.dbg_pre = value; return kOk;
    case 107: g_opt.moe_kernel = value; return kOk;
    case 111: g_opt.dbg_mb_groups = value; return kOk;
    case 112: g_opt.dbg_mb_min_m = value; return kOk;
    case 113: g_opt.dbg_mb_rpc = value; return kOk;
    case 114: g_opt.dbg_host_wb = value; return kOk;
    case 115: g_opt.dbg_host_early = value; return kOk;
    case 116: g_opt.dbg_slab_kb = value > 0 ? value : 0; return kOk;
    case 117: g_opt.dbg_no_split = value; return kOk;
    case FUELQ_OPT_L2_PREFETCH: g_opt.l2_prefetch = value ? 1 : 0; return kOk;
    case FUELQ_OPT_FUSED_QUANT: g_opt.fused_quant = value ? 1 : 0; return kOk;
    case FUELQ_OPT_PREFILL_TF32: g_opt.prefill_tf32 = value ? 1 : 0; return kOk;
    case FUELQ_OPT_PREFILL_BF16: g_opt.prefill_bf16 = value ? 1 : 0; return kOk;
    case FUELQ_OPT_PREFILL_ONE_KERNEL: g_opt.prefill_one_kernel = value ? 1 : 0; return kOk;
    case FUELQ_OPT_PEER_WAIT_MS:
      if (value < 1 || value > 60000) return kInvalidProblem;
      g_opt.peer_wait_ms = value;
      return kOk;
    default: return kInvalidProblem;
  }
}

int64_t fuelq_get_option(int32_t key) {
  switch (key) {
    case FUELQ_OPT_PDL: return g_opt.pdl;
    case FUELQ_OPT_DECODE_MAX_M: return g_opt.decode_max_m;
    case FUELQ_OPT_DECODE_GRID: return g_opt.decode_grid;
    case FUELQ_OPT_DECODE_KERNEL: return g_opt.decode_kernel;
    case FUELQ_OPT_L2_PREFETCH: return g_opt.l2_prefetch;
    case FUELQ_OPT_FUSED_QUANT: return g_opt.fused_quant;
    case FUELQ_OPT_PEER_WAIT_MS: return g_opt.peer_wait_ms;
    case FUELQ_OPT_PREFILL_TF32: return g_opt.prefill_tf32;
    case FUELQ_OPT_PREFILL_BF16: return g_opt.prefill_bf16;
    case FUELQ_OPT_PREFILL_ONE_KERNEL: return g_opt.prefill_one_kernel;
    default: return -1;
  }
}

int32_t fuelq_device_error(int32_t* host_code_out, int32_t clear) {
  int code = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return kLaunchFailure;
  if (cudaMemcpyFromSymbol(&code, g_fq_dev_error, sizeof(int)) != cudaSuccess) return kLaunchFailure;
  if (clear && code) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_fq_dev_error, &zero, sizeof(int)) != cudaSuccess) return kLaunchFailure;
  }
  if (host_code_out) *host_code_out = code;
  return kOk;
}

int32_t fuelq_quantize_act(int32_t weight_type, int64_t m_total, int64_t k, const float* x, void* q8_blocks,
                           void* stream) {
  if (m_total > 0 && !q8_blocks) return kInvalidProblem;
  return quantize_act_impl(weight_type, m_total, k, x, q8_blocks, nullptr, (cudaStream_t)stream);
}

size_t fuelq_act_packed_bytes(int32_t weight_type, int64_t m_total, int64_t k) {
  if (!supported_weight(weight_type) || m_total < 0 || k <= 0) return 0;
  return act_packed_bytes(weight_type, m_total, k);
}

int32_t fuelq_quantize_act_packed(int32_t weight_type, int64_t m_total, int64_t k, const float* x, void* packed,
                                  size_t packed_bytes, void* stream) {
  if (!supported_weight(weight_type)) return kNotSupported;
  if (m_total > 0 && (!packed || packed_bytes < act_packed_bytes(weight_type, m_total, k))) return kWorkspace;
  if (packed && !aligned(packed, 16)) return kMisaligned;
  return quantize_act_impl(weight_type, m_total, k, x, nullptr, packed, (cudaStream_t)stream);
}

size_t fuelq_qmatmul_workspace_bytes(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k) {
  if (check_problem(ggml_type, m_total, n, k) != kOk) return 0;
  if (prefill_available(ggml_type, m_total, n, k)) return prefill_workspace_bytes(ggml_type, m_total, n, k);
  return act_packed_bytes(ggml_type, m_total, k);
}

int32_t fuelq_qmatmul_numerics(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k) {
  const int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return -st;
  if (!prefill_available(ggml_type, m_total, n, k)) return 0;
  return g_opt.prefill_tf32 ? FUELQ_NUMERICS_TF32 : g_opt.prefill_bf16 ? FUELQ_NUMERICS_BF16 : FUELQ_NUMERICS_F16;
}

int32_t fuelq_qmatmul_can_implement(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k) {
  const int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return st;
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  DecodePlan pl;
  return n == 0 ? kOk : plan_decode(ggml_type, n, k, *di, &pl);
}

int32_t fuelq_qmatmul_packed(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                             const void* packed_act, float* y, void* stream) {
  const int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return st;
  if (m_total == 0 || n == 0) return kOk;
  if (!w || !packed_act || !y) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(packed_act, 16) || !aligned(y, 4)) return kMisaligned;
  if (g_opt.l2_prefetch) {
    const int32_t sp = prefetch_impl(w, n * (k / block_elems(ggml_type)) * block_bytes(ggml_type), (cudaStream_t)stream);
    if (sp != kOk) return sp;
  }
  return decode_chunked(ggml_type, m_total, n, k, w, const_cast<void*>(packed_act), y, (cudaStream_t)stream);
}

static int32_t qmatmul_integer(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w, const float* x,
                               float* y, void* workspace, void* stream);

int32_t fuelq_qmatmul(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w, const float* x,
                      float* y, void* workspace, size_t workspace_bytes, void* stream) {
  int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return st;
  if (m_total == 0 || n == 0) return kOk;
  if (!w || !x || !y) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(x, 16) || !aligned(y, 4)) return kMisaligned;
  const size_t need = fuelq_qmatmul_workspace_bytes(ggml_type, m_total, n, k);
  if (!workspace || workspace_bytes < need) return kWorkspace;
  if (!aligned(workspace, 16)) return kMisaligned;
  if (prefill_available(ggml_type, m_total, n, k)) {
    if (m_total > (1 << 30) || n > (1 << 30)) return kNotSupported;
    float* const one[1] = {y};
    return prefill_impl(ggml_type, m_total, n, k, w, x, one, 1, n, 0, workspace, (cudaStream_t)stream);
  }
  return qmatmul_integer(ggml_type, m_total, n, k, w, x, y, workspace, stream);
}

// The integer kernels (the reference's arithmetic): activation blocks into the workspace, then the mat-vec kernels.
static int32_t qmatmul_integer(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w, const float* x,
                               float* y, void* workspace, void* stream) {
  int32_t st;
  if (g_opt.l2_prefetch) {
    st = prefetch_impl(w, n * (k / block_elems(ggml_type)) * block_bytes(ggml_type), (cudaStream_t)stream);
    if (st != kOk) return st;
  }
  // One row of a small matrix (a few microseconds of streaming): the separate quantizer launch is a large share of the
  // time, so the mat-vec's thread blocks quantize the row themselves, one block per SM (measured 5.4 against 6.0 us per
  // call for 4096 x 4096 Q4_K in a chain of launches; larger matrices measured faster with the two-kernel form).
  const bool small_one_row = m_total == 1 && (ggml_type == kQ4K || ggml_type == kQ6K) && g_opt.decode_grid == 0 &&
                             n * (k / 256) * block_bytes(ggml_type) <= (12 << 20);
  if (m_total <= 2 && (g_opt.fused_quant || small_one_row) && g_opt.decode_kernel != 1) {
    // one kernel: every thread block quantizes the activation rows itself while its weights stream in
    const ActPlanes none = {};
    st = decode_regs_impl(ggml_type, m_total, n, k, w, none, y, (cudaStream_t)stream, nullptr, x);
    if (st != kNotSupported) return st;
  }
  st = quantize_act_impl(ggml_type, m_total, k, x, nullptr, workspace, (cudaStream_t)stream);
  if (st != kOk) return st;
  return decode_chunked(ggml_type, m_total, n, k, w, workspace, y, (cudaStream_t)stream);
}

int32_t fuelq_qmatmul_sharded(int32_t ggml_type, int64_t m_total, int64_t n_local, int64_t k, const void* w_local,
                              const float* x, float* const* y_dst, int32_t n_dst, int64_t n_total, int64_t n_offset,
                              void* workspace, size_t workspace_bytes, void* stream) {
  const int32_t st = check_problem(ggml_type, m_total, n_local, k);
  if (st != kOk) return st;
  if (n_dst < 1 || n_dst > 8 || n_total <= 0 || n_offset < 0 || n_offset + n_local > n_total || n_total > (1 << 30) ||
      m_total * n_total > ((int64_t)1 << 40))
    return kInvalidProblem;
  if (m_total == 0 || n_local == 0) return kOk;
  if (!w_local || !x || !y_dst) return kInvalidProblem;
  for (int q = 0; q < n_dst; ++q)
    if (!y_dst[q]) return kInvalidProblem;
  if (!aligned(w_local, 16) || !aligned(x, 16)) return kMisaligned;
  if (!prefill_available(ggml_type, m_total, n_local, k)) return kNotSupported;  // the tensor-core path only
  if (m_total > (1 << 30)) return kNotSupported;
  if (!workspace || workspace_bytes < prefill_workspace_bytes(ggml_type, m_total, n_local, k)) return kWorkspace;
  if (!aligned(workspace, 16)) return kMisaligned;
  return prefill_impl(ggml_type, m_total, n_local, k, w_local, x, y_dst, n_dst, n_total, n_offset, workspace,
                      (cudaStream_t)stream);
}

size_t fuelq_qmatmul_host_workspace_bytes(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k) {
  if (check_problem(ggml_type, m_total, n, k) != kOk) return 0;
  return align_up((size_t)m_total * k * 4, 256) + align_up((size_t)m_total * n * 4, 256) +
         fuelq_qmatmul_workspace_bytes(ggml_type, m_total, n, k);
}

int32_t fuelq_qmatmul_host(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                           const float* x_host, float* y_host, void* workspace, size_t workspace_bytes,
                           void* stream_v) {
  const int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return st;
  if (m_total == 0 || n == 0) return kOk;
  if (!w || !x_host || !y_host) return kInvalidProblem;
  if (!workspace || workspace_bytes < fuelq_qmatmul_host_workspace_bytes(ggml_type, m_total, n, k)) return kWorkspace;
  if (!aligned(workspace, 256)) return kMisaligned;
  cudaStream_t stream = (cudaStream_t)stream_v;
  uint8_t* p = (uint8_t*)workspace;
  float* x_dev = (float*)p;
  p += align_up((size_t)m_total * k * 4, 256);
  float* y_dev = (float*)p;
  p += align_up((size_t)m_total * n * 4, 256);
  // Small activations held in page-locked, device-mapped host memory (cudaHostAlloc, cudaHostRegister with the
  // mapped flag, a framework's pinned tensors): the quantizing kernel reads x in place over PCIe and a small kernel
  // writes y in place, so the chain is three kernels on one stream with no copy-engine hand-off in between.
  const size_t xb = (size_t)m_total * k * 4, yb = (size_t)m_total * n * 4;
  if (!prefill_available(ggml_type, m_total, n, k) && xb <= (256u << 10) && yb <= (1u << 20)) {
    const float* xm = (const float*)mapped_alias(x_host);
    float* ym = (float*)mapped_alias(y_host);
    if (xm && ym && aligned(xm, 16) && aligned(ym, 4)) {
      int32_t s1 = kOk;
      if (g_opt.l2_prefetch)
        s1 = prefetch_impl(w, n * (k / block_elems(ggml_type)) * block_bytes(ggml_type), stream);
      unsigned* done = (unsigned*)x_dev;  // the staging area for x is free on this path: its first word counts thread blocks
      if (s1 == kOk) s1 = quantize_act_impl(ggml_type, m_total, k, xm, nullptr, p, stream, done, g_opt.dbg_host_early != 0);
      if (s1 != kOk) return s1;
      // One row in plain launches: the mat-vec kernel's last thread block writes y to the host buffer itself (one launch
      // fewer). With programmatic dependent launch the separate write-back kernel measured faster: it is resident
      // before the mat-vec ends, and sixteen thread blocks share the copy.
      const bool wb_inside = g_opt.dbg_host_wb == 2 || (g_opt.dbg_host_wb == 0 && !g_opt.pdl);
      if (m_total == 1 && wb_inside && g_opt.decode_kernel != 1) {
        s1 = decode_regs_impl(ggml_type, 1, n, k, w, act_planes(p, ggml_type, 1, k), y_dev, stream, nullptr, nullptr, ym, done);
        if (s1 != kNotSupported) return s1;
      }
      s1 = decode_chunked(ggml_type, m_total, n, k, w, p, y_dev, stream);
      if (s1 != kOk) return s1;
      const long long words = (long long)m_total * n;
      const unsigned grid = (unsigned)std::min<long long>((words / 4 + 255) / 256 + 1, 16);
      const cudaError_t e = launch(copy_out_f32_kernel, dim3(grid), dim3(256), 0, stream, (const float*)y_dev, ym, words,
                                   aligned(ym, 16) ? 1 : 0);
      return e == cudaSuccess ? kOk : kLaunchFailure;
    }
  }
  if (cudaMemcpyAsync(x_dev, x_host, xb, cudaMemcpyHostToDevice, stream) != cudaSuccess) return kLaunchFailure;
  const int32_t s2 = fuelq_qmatmul(ggml_type, m_total, n, k, w, x_dev, y_dev, p,
                                   workspace_bytes - (size_t)(p - (uint8_t*)workspace), stream_v);
  if (s2 != kOk) return s2;
  if (cudaMemcpyAsync(y_host, y_dev, yb, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return kLaunchFailure;
  return kOk;
}

// ---- mat-vec for callers that cannot allocate -------------------------------------------------
// Some hosts of this library may not call cudaMalloc at all: code running inside a captured or
// latency-critical region whose memory was fixed at start-up, plug-in sandboxes that are handed
// device pointers but no allocator, or a process whose memory pool is owned by another runtime.
// For them the activation scratch lives in the library image itself: a fixed device array that
// every GPU loading the library carries until the process exits.
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB: e.g. m_total * k up to ~900k elements
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

size_t fuelq_static_scratch_bytes(void) { return kStaticScratchBytes; }

int32_t fuelq_qmatmul_static_scratch(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                                     const float* x, float* y, void* stream) {
  const int32_t st = check_problem(ggml_type, m_total, n, k);
  if (st != kOk) return st;
  if (m_total == 0 || n == 0) return kOk;
  // Sizes beyond the built-in scratch are refused, never truncated. A tensor-core problem whose activations fit but
  // whose slab of dequantized rows does not runs without a slab: Q4_K / Q6_K / Q8_0 dequantized inside the GEMM kernel
  // (the same arithmetic class), the other formats on the integer kernels if their activation blocks fit.
  int fallback = 0;
  if (fuelq_qmatmul_workspace_bytes(ggml_type, m_total, n, k) > kStaticScratchBytes) {
    if (!prefill_available(ggml_type, m_total, n, k)) return kWorkspace;
    if (prefill_native_type(ggml_type) && prefill_x_bytes(m_total, k) <= kStaticScratchBytes && m_total <= (1 << 30) && n <= (1 << 30))
      fallback = 1;
    else if (act_packed_bytes(ggml_type, m_total, k) <= kStaticScratchBytes)
      fallback = 2;
    else
      return kWorkspace;
  }
  // In host code the array's name is only a handle; the device address has to be asked for, once
  // per device, with that device current.
  static void* scratch_addr[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kLaunchFailure;
  if (!scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return kLaunchFailure;
    scratch_addr[dev] = p;
  }
  // every plane of the scratch is written by the activation-quantization kernel before the
  // mat-vec reads it, so nothing in it needs clearing between calls
  if (fallback) {
    if (!w || !x || !y) return kInvalidProblem;
    if (!aligned(w, 16) || !aligned(x, 16) || !aligned(y, 4)) return kMisaligned;
    if (fallback == 2) return qmatmul_integer(ggml_type, m_total, n, k, w, x, y, scratch_addr[dev], stream);
    float* const one[1] = {y};
    return prefill_impl(ggml_type, m_total, n, k, w, x, one, 1, n, 0, scratch_addr[dev], (cudaStream_t)stream, true);
  }
  return fuelq_qmatmul(ggml_type, m_total, n, k, w, x, y, scratch_addr[dev], kStaticScratchBytes, stream);
}

int32_t fuelq_prefetch_weights(const void* w, int64_t bytes, void* stream) {
  if (bytes < 0) return kInvalidProblem;
  return prefetch_impl(w, bytes, (cudaStream_t)stream);
}

int32_t fuelq_quantize_weights(int32_t ggml_type, int64_t numel, const float* x, void* blocks, void* stream_v) {
  if (!supported_weight(ggml_type)) return kNotSupported;
  const int be = block_elems(ggml_type);
  if (numel < 0 || numel % be) return kInvalidProblem;
  if (numel == 0) return kOk;
  if (!x || !blocks) return kInvalidProblem;
  if (!aligned(x, 16) || !aligned(blocks, (ggml_type == kQ4K || ggml_type == kQ5K || ggml_type == kQ2K) ? 4 : 2)) return kMisaligned;
  cudaStream_t stream = (cudaStream_t)stream_v;
  const int64_t nb = numel / be;
  uint8_t* out = (uint8_t*)blocks;
  switch (ggml_type) {
    case kQ8_0: quantize_w_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ4_0: quantize_w_q4_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ4_1: quantize_w_legacy32_kernel<Q4_1L, false, true><<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ5_0: quantize_w_legacy32_kernel<Q5_0L, true, false><<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ5_1: quantize_w_legacy32_kernel<Q5_1L, true, true><<<(unsigned)((nb + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ2K: quantize_w_q2k_kernel<<<(unsigned)((nb * 16 + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ3K: quantize_w_q3k_kernel<<<(unsigned)((nb * 16 + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ4K: quantize_w_q4k_kernel<false><<<(unsigned)((nb * 8 + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ5K: quantize_w_q4k_kernel<true><<<(unsigned)((nb * 8 + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    case kQ6K: quantize_w_q6k_kernel<<<(unsigned)((nb * 16 + 127) / 128), 128, 0, stream>>>(x, nb, out); break;
    default: return kNotSupported;
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- f32 glue of a LLaMA-style decode step (llama_glue.cuh) -----------------------------------------
int32_t fuelq_embed_rows(int32_t ggml_type, const void* table, int64_t k, const int32_t* ids, int64_t n_ids, float* out,
                         void* stream) {
  if (ggml_type != kQ4K && ggml_type != kF32) return kNotSupported;
  if (k <= 0 || k % 256 || n_ids < 0) return kInvalidProblem;
  if (n_ids == 0) return kOk;
  if (!table || !ids || !out) return kInvalidProblem;
  if (!aligned(table, 16) || !aligned(out, ggml_type == kF32 ? 16 : 4)) return kMisaligned;
  if (ggml_type == kF32) {  // a table the loader already dequantized (any other on-disk format)
    const cudaError_t e = launch(embed_f32_kernel, dim3((unsigned)n_ids), dim3(256), 0, (cudaStream_t)stream, (const float*)table,
                                 (int)k, (const int*)ids, out);
    return e == cudaSuccess ? kOk : kLaunchFailure;
  }
  const cudaError_t e = launch(embed_q4k_kernel, dim3((unsigned)n_ids), dim3(256), 0, (cudaStream_t)stream,
                               (const uint8_t*)table, (int)(k / 256 * 144), (int)k, (const int*)ids, out);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_add_rmsnorm(float* x, const float* delta, const float* gain, float* out, int64_t rows, int64_t dim, float eps,
                          void* stream) {
  if (rows < 0 || dim <= 0 || dim % 256 || dim > 8192) return kInvalidProblem;
  if (rows == 0) return kOk;
  if (!x || !gain || !out) return kInvalidProblem;
  if (!aligned(x, 16) || !aligned(gain, 16) || (delta && !aligned(delta, 16)) || !aligned(out, 16)) return kMisaligned;
  const cudaError_t e = launch(add_rmsnorm_kernel<false>, dim3((unsigned)rows), dim3((unsigned)(dim / 256 * 32)), 0,
                               (cudaStream_t)stream, x, delta, gain, out, (int)dim, eps, (int8_t*)nullptr, (float*)nullptr,
                               (int16_t*)nullptr);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_rope_store(float* q, const float* k, const float* v, float* kcache, float* vcache, const float* cos_table,
                         const float* sin_table, const int32_t* pos, int32_t n_heads, int32_t n_kv, int32_t head_dim,
                         int32_t max_seq, void* stream) {
  if (n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || head_dim % 2 || max_seq <= 0) return kInvalidProblem;
  if (!q || !k || !v || !kcache || !vcache || !cos_table || !sin_table || !pos) return kInvalidProblem;
  const cudaError_t e = launch(rope_store_kernel, dim3((unsigned)(n_heads + n_kv)), dim3(128), 0, (cudaStream_t)stream, q, k, v,
                               kcache, vcache, cos_table, sin_table, (const int*)pos, (int)n_heads, (int)n_kv, (int)head_dim,
                               (int)max_seq);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

namespace {
// null `rope`: q is rotated and the caches are up to date; otherwise the attention kernel does both itself
bool make_attn_rope(const fuelq_rope* rope, AttnRope* out) {
  *out = AttnRope{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (!rope) return true;
  if (!rope->k || !rope->v || !rope->cos_table || !rope->sin_table || !rope->kcache || !rope->vcache) return false;
  if (!aligned(rope->k, 16) || !aligned(rope->v, 16) || !aligned(rope->cos_table, 16) || !aligned(rope->sin_table, 16) ||
      !aligned(rope->kcache, 16) || !aligned(rope->vcache, 16))
    return false;
  *out = AttnRope{rope->k, rope->v, rope->cos_table, rope->sin_table, rope->kcache, rope->vcache};
  return true;
}
}  // namespace

size_t fuelq_attn_decode_workspace_bytes(int32_t n_heads) {
  return n_heads > 0 ? (size_t)n_heads * kAttnSplits * kAttnPartStride * sizeof(float) : 0;
}

int32_t fuelq_attn_decode(const float* q, const float* kcache, const float* vcache, float* out, const int32_t* pos,
                          int32_t n_heads, int32_t n_kv, int32_t head_dim, int32_t max_seq, float scale, void* workspace,
                          size_t workspace_bytes, const fuelq_rope* rope, void* stream) {
  if (head_dim != 128) return kNotSupported;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || max_seq <= 0 || max_seq > 8192) return kInvalidProblem;
  if (!q || !kcache || !vcache || !out || !pos) return kInvalidProblem;
  if (!workspace || workspace_bytes < fuelq_attn_decode_workspace_bytes(n_heads)) return kWorkspace;
  if (!aligned(q, 16) || !aligned(kcache, 16) || !aligned(vcache, 16) || !aligned(workspace, 16)) return kMisaligned;
  AttnRope ar;
  if (!make_attn_rope(rope, &ar)) return kInvalidProblem;
  cudaError_t e = launch(attn_partial_kernel, dim3((unsigned)n_heads, kAttnSplits), dim3(256), 0, (cudaStream_t)stream, q,
                         kcache, vcache, (float*)workspace, (const int*)pos, (int)n_heads, (int)n_kv, (int)max_seq, scale, ar);
  if (e != cudaSuccess) return kLaunchFailure;
  e = launch(attn_combine_kernel, dim3((unsigned)n_heads), dim3(128), 0, (cudaStream_t)stream, (const float*)workspace, out);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- fused producers for the single-GPU step: the same values as the plain call followed by
// fuelq_quantize_act_packed (weight type Q4K/Q6K, m = 1), written straight into the packed planes
int32_t fuelq_add_rmsnorm_q8k(float* x, const float* delta, const float* gain, int64_t dim, float eps, void* packed,
                              size_t packed_bytes, void* stream) {
  if (dim <= 0 || dim % 256 || dim > 8192) return kInvalidProblem;
  if (!x || !gain) return kInvalidProblem;
  if (!packed || packed_bytes < act_packed_bytes(kQ4K, 1, dim)) return kWorkspace;
  if (!aligned(x, 16) || !aligned(gain, 16) || (delta && !aligned(delta, 16)) || !aligned(packed, 16)) return kMisaligned;
  const ActPlanes a = act_planes(packed, kQ4K, 1, dim);
  const cudaError_t e = launch(add_rmsnorm_kernel<true>, dim3(1), dim3((unsigned)(dim / 256 * 32)), 0, (cudaStream_t)stream, x,
                               delta, gain, (float*)nullptr, (int)dim, eps, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_swiglu_q8k(const float* gate, const float* up, int64_t n, void* packed, size_t packed_bytes, void* stream) {
  if (n <= 0 || n % 256) return kInvalidProblem;
  if (!gate || !up) return kInvalidProblem;
  if (!packed || packed_bytes < act_packed_bytes(kQ4K, 1, n)) return kWorkspace;
  if (!aligned(gate, 16) || !aligned(up, 16) || !aligned(packed, 16)) return kMisaligned;
  const ActPlanes a = act_planes(packed, kQ4K, 1, n);
  const int64_t nb = n / 256;
  const cudaError_t e = launch(swiglu_q8k_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, gate, up,
                               nb, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_attn_decode_q8k(const float* q, const float* kcache, const float* vcache, const int32_t* pos, int32_t n_heads,
                              int32_t n_kv, int32_t head_dim, int32_t max_seq, float scale, void* workspace,
                              size_t workspace_bytes, void* packed, size_t packed_bytes, const fuelq_rope* rope, void* stream) {
  if (head_dim != 128) return kNotSupported;
  if (n_heads <= 0 || n_heads % 2 || n_kv <= 0 || n_heads % n_kv || max_seq <= 0 || max_seq > 8192) return kInvalidProblem;
  if (!q || !kcache || !vcache || !pos) return kInvalidProblem;
  if (!workspace || workspace_bytes < fuelq_attn_decode_workspace_bytes(n_heads)) return kWorkspace;
  if (!packed || packed_bytes < act_packed_bytes(kQ4K, 1, (int64_t)n_heads * 128)) return kWorkspace;
  if (!aligned(q, 16) || !aligned(kcache, 16) || !aligned(vcache, 16) || !aligned(workspace, 16) || !aligned(packed, 16))
    return kMisaligned;
  AttnRope ar;
  if (!make_attn_rope(rope, &ar)) return kInvalidProblem;
  cudaError_t e = launch(attn_partial_kernel, dim3((unsigned)n_heads, kAttnSplits), dim3(256), 0, (cudaStream_t)stream, q,
                         kcache, vcache, (float*)workspace, (const int*)pos, (int)n_heads, (int)n_kv, (int)max_seq, scale, ar);
  if (e != cudaSuccess) return kLaunchFailure;
  const ActPlanes a = act_planes(packed, kQ4K, 1, (int64_t)n_heads * 128);
  e = launch(attn_combine_q8k_kernel, dim3((unsigned)(n_heads / 2)), dim3(32), 0, (cudaStream_t)stream,
             (const float*)workspace, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_swiglu(const float* gate, const float* up, float* out, int64_t n, void* stream) {
  if (n < 0) return kInvalidProblem;
  if (n == 0) return kOk;
  if (!gate || !up || !out) return kInvalidProblem;
  const cudaError_t e = launch(swiglu_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, gate, up,
                               out, (int64_t)n);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_argmax_last(const float* x, int64_t n, int32_t* out_index, void* stream) {
  if (n <= 0 || n > (1 << 30)) return kInvalidProblem;
  if (!x || !out_index) return kInvalidProblem;
  const cudaError_t e = launch(argmax_last_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, x, (int)n, (int*)out_index);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- mixture-of-experts block (moe.cuh)
int32_t fuelq_moe_route(const float* logits, int64_t n_tokens, int32_t n_experts, int32_t top_k, int32_t* topk_ids,
                        float* topk_weights, void* stream) {
  if (n_tokens < 0 || n_experts <= 0 || n_experts > 1024 || top_k <= 0 || top_k > kMoeMaxTopK || top_k > n_experts)
    return kInvalidProblem;
  if (n_tokens == 0) return kOk;
  if (n_tokens > (1 << 24)) return kNotSupported;
  if (!logits || !topk_ids || !topk_weights) return kInvalidProblem;
  const cudaError_t e = launch(moe_route_kernel, dim3((unsigned)((n_tokens + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
                               logits, (int)n_tokens, (int)n_experts, (int)top_k, (int*)topk_ids, topk_weights);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_bucket(const int32_t* topk_ids, int64_t n_pairs, int32_t n_experts, int32_t* sorted_ids,
                         int32_t* expert_offsets, void* stream) {
  if (n_pairs < 0 || n_pairs > (1 << 24) || n_experts <= 0 || n_experts > 8192) return kInvalidProblem;
  if (!expert_offsets || (n_pairs > 0 && (!topk_ids || !sorted_ids))) return kInvalidProblem;
  // per-chunk count table in shared memory when it fits (config 5: 64 chunks x 128 experts = 32 KB)
  const size_t table = ((size_t)((n_pairs + 31) / 32) * n_experts + n_experts + 1) * sizeof(int);
  if (n_pairs > 0 && table <= 160 * 1024) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      if (cudaFuncSetAttribute(moe_bucket_chunks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
        return kLaunchFailure;
      attr_set[dev] = true;
    }
    const cudaError_t e = launch(moe_bucket_chunks_kernel, dim3(1), dim3(1024), table, (cudaStream_t)stream, (const int*)topk_ids,
                                 (int)n_pairs, (int)n_experts, (int*)sorted_ids, (int*)expert_offsets);
    return e == cudaSuccess ? kOk : kLaunchFailure;
  }
  const int in_smem = (size_t)(n_experts + 1 + n_pairs) * sizeof(int) <= 48 * 1024 ? 1 : 0;  // default dynamic limit
  const size_t bsm = (size_t)(n_experts + 1 + (in_smem ? n_pairs : 0)) * sizeof(int);
  const cudaError_t e = launch(moe_bucket_kernel, dim3(1), dim3(1024), bsm,
                               (cudaStream_t)stream, (const int*)topk_ids, (int)n_pairs, (int)n_experts, (int*)sorted_ids,
                               (int*)expert_offsets, in_smem);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_quantize_rows(const float* x, int64_t k, const int32_t* row_ids, int32_t divisor, int64_t n_rows,
                                void* packed, size_t packed_bytes, void* stream) {
  if (k <= 0 || k % 256 || k > (1 << 24) || divisor <= 0 || n_rows < 0) return kInvalidProblem;
  if (n_rows == 0) return kOk;
  if (!x || !row_ids || !packed) return kInvalidProblem;
  if (packed_bytes < act_packed_bytes(kQ4K, n_rows, k)) return kWorkspace;
  if (!aligned(x, 16) || !aligned(packed, 16)) return kMisaligned;
  const ActPlanes a = act_planes(packed, kQ4K, n_rows, k);
  const int64_t nb = n_rows * (k / 256);
  const cudaError_t e = launch(moe_gather_quantize_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, x,
                               (int)k, (const int*)row_ids, (int)divisor, nb, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_swiglu_quantize(const float* gate_up, int64_t f, int64_t n_rows, void* packed, size_t packed_bytes,
                                  void* stream) {
  if (f <= 0 || f % 256 || f > (1 << 24) || n_rows < 0) return kInvalidProblem;
  if (n_rows == 0) return kOk;
  if (!gate_up || !packed) return kInvalidProblem;
  if (packed_bytes < act_packed_bytes(kQ4K, n_rows, f)) return kWorkspace;
  if (!aligned(gate_up, 16) || !aligned(packed, 16)) return kMisaligned;
  const ActPlanes a = act_planes(packed, kQ4K, n_rows, f);
  const int64_t nb = n_rows * (f / 256);
  const cudaError_t e = launch(moe_swiglu_quantize_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
                               gate_up, (int)f, nb, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

extern "C++" {
namespace {
template <class Fmt>
cudaError_t launch_moe(const MoeParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  static bool attr_set[64] = {};
  auto kern = moe_decode_kernel<Fmt>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!attr_set[dev]) {
    DeviceInfo* di;
    if (!device_info(&di)) return cudaErrorInvalidDevice;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, di->max_smem_optin);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return launch(kern, grid, dim3(kDecodeThreads), smem, stream, p);
}
}  // namespace
}  // extern "C++"

int32_t fuelq_moe_qmatmul(int32_t ggml_type, int32_t n_experts, int64_t n, int64_t k, const void* w, const void* packed_act,
                          int64_t n_rows, const int32_t* expert_offsets, const int32_t* out_rows, float* y, void* stream) {
  if (ggml_type != kQ4K && ggml_type != kQ6K) return kNotSupported;
  if (n_experts <= 0 || n_experts > 65535 || n <= 0 || n > (1 << 24) || k <= 0 || k % 256 || k > (1 << 24) || n_rows < 0)
    return kInvalidProblem;
  if (n_rows == 0) return kOk;
  if (!w || !packed_act || !expert_offsets || !y) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(packed_act, 16)) return kMisaligned;
  if ((g_opt.moe_kernel == 0 && ggml_type != kQ4K) || g_opt.moe_kernel == 3) {
    const int32_t sm = mma_batch_impl(ggml_type, n_experts, n, k, w, act_planes(const_cast<void*>(packed_act), ggml_type, n_rows, k),
                                      (const int*)expert_offsets, 0, (const int*)out_rows, y, true, (cudaStream_t)stream);
    if (sm != kNotSupported) return sm;
  }
  if (ggml_type == kQ4K && (g_opt.moe_kernel == 0 || g_opt.moe_kernel == 2)) {
    const int32_t sm = moe_mma_impl(n_experts, n, k, w, act_planes(const_cast<void*>(packed_act), ggml_type, n_rows, k),
                                    (const int*)expert_offsets, 0, (const int*)out_rows, y, (cudaStream_t)stream);
    if (sm != kNotSupported) return sm;
  }
  DeviceInfo* di;
  if (!device_info(&di)) return kLaunchFailure;
  MoeParams p;
  p.row_bytes = (int)(k / 256 * block_bytes(ggml_type));
  if (p.row_bytes % 16) return kNotSupported;  // rows are bulk-copied whole: Q6_K needs k a multiple of 2048
  p.w = (const uint8_t*)w;
  p.act = act_planes(const_cast<void*>(packed_act), ggml_type, n_rows, k);
  p.offsets = (const int*)expert_offsets;
  p.out_rows = (const int*)out_rows;
  p.y = y;
  p.n = (int)n;
  p.k = (int)k;
  p.expert_bytes = n * (int64_t)p.row_bytes;
  p.units_per_row = (int)(k / 256) * (ggml_type == kQ4K ? Q4KDecode::kUnitsPerBlock : Q6KDecode::kUnitsPerBlock);
  const size_t header = align_up(sizeof(MoeSmemHeader), 128);
  // shared memory per thread block (two per SM): activation rows of one pass, then the ring of weight stages
  int act_rows = (int)((40 * 1024) / (k + k / 8 + k / 64 + 64)) / kMoeMT * kMoeMT;
  if (act_rows > 32) act_rows = 32;
  if (act_rows < kMoeMT) return kNotSupported;
  const size_t act_bytes = align_up(act_packed_bytes(kQ4K, act_rows, k), 128);
  const size_t per_cta = ((size_t)di->max_smem_optin + 1024) / 2 - 1024 - 512;
  if (header + act_bytes + 8192 > per_cta) return kNotSupported;
  const size_t budget = per_cta - header - act_bytes;
  int R = (24 * 1024) / p.row_bytes;
  if (R > 64) R = 64;
  if (R >= kDecodeConsumerWarps) R = R / kDecodeConsumerWarps * kDecodeConsumerWarps;
  if (R < 1) return kNotSupported;
  p.rows_per_stage = R;
  p.stage_stride = (int)align_up((size_t)R * p.row_bytes, 128);
  int stages = (int)(budget / p.stage_stride);
  if (stages < 2) return kNotSupported;
  if (stages > kDecodeMaxStages) stages = kDecodeMaxStages;
  p.num_stages = stages;
  p.act_rows = act_rows;
  p.act_smem_off = (int)(header + (size_t)stages * p.stage_stride);
  // enough thread blocks per expert to fill the GPU a few times over, never more than one per stage of rows
  int per_expert = (4 * di->sm_count + n_experts - 1) / n_experts;
  const int max_per = (int)((n + R - 1) / R);
  if (per_expert > max_per) per_expert = max_per;
  if (per_expert < 1) per_expert = 1;
  const size_t smem = header + (size_t)stages * p.stage_stride + act_bytes;
  const dim3 grid((unsigned)per_expert, (unsigned)n_experts);
  const cudaError_t e = ggml_type == kQ4K ? launch_moe<Q4KDecode>(p, grid, smem, (cudaStream_t)stream)
                                          : launch_moe<Q6KDecode>(p, grid, smem, (cudaStream_t)stream);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

namespace {
int32_t check_ep(int64_t hidden, int64_t n_pairs, int32_t experts_per_rank, int32_t world, int64_t capacity) {
  if (hidden <= 0 || hidden % 4 || hidden > (1 << 24) || n_pairs < 0 || experts_per_rank <= 0 || world < 1 || world > 64 ||
      capacity < 1 || capacity > hidden || n_pairs > capacity)
    return kInvalidProblem;
  return kOk;
}
}  // namespace

int32_t fuelq_moe_ep_pack(const float* x, int64_t hidden, const int32_t* sorted_ids, const int32_t* expert_offsets,
                          const int32_t* topk_ids, int32_t top_k, int64_t n_pairs, int32_t experts_per_rank, int32_t world,
                          int64_t capacity, float* send, void* stream) {
  const int32_t st = check_ep(hidden, n_pairs, experts_per_rank, world, capacity);
  if (st != kOk) return st;
  if (top_k <= 0 || !x || !sorted_ids || !expert_offsets || !topk_ids || !send) return kInvalidProblem;
  if (!aligned(x, 16) || !aligned(send, 16)) return kMisaligned;
  const cudaError_t e = launch(moe_ep_pack_kernel, dim3((unsigned)(n_pairs + world)), dim3(128), 0, (cudaStream_t)stream, x,
                               (int)hidden, (const int*)sorted_ids, (const int*)expert_offsets, (const int*)topk_ids, (int)top_k,
                               (int)n_pairs, (int)experts_per_rank, (int)world, (int)capacity, send);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_ep_local_ids(const float* recv, int64_t hidden, int64_t capacity, int32_t world, int32_t first_expert,
                               int32_t* local_ids, void* stream) {
  const int32_t st = check_ep(hidden, 0, 1, world, capacity);
  if (st != kOk) return st;
  if (!recv || !local_ids || first_expert < 0) return kInvalidProblem;
  if (!aligned(recv, 16)) return kMisaligned;
  const int64_t slots = (int64_t)world * (capacity + 1);
  const cudaError_t e = launch(moe_ep_local_ids_kernel, dim3((unsigned)((slots + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                               recv, (int)hidden, (int)capacity, (int)world, (int)first_expert, (int*)local_ids);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_ep_unpack(const float* y_back, int64_t hidden, const int32_t* sorted_ids, const int32_t* expert_offsets,
                            int64_t n_pairs, int32_t experts_per_rank, int32_t world, int64_t capacity, float* y_pairs,
                            void* stream) {
  const int32_t st = check_ep(hidden, n_pairs, experts_per_rank, world, capacity);
  if (st != kOk) return st;
  if (n_pairs == 0) return kOk;
  if (!y_back || !sorted_ids || !expert_offsets || !y_pairs) return kInvalidProblem;
  if (!aligned(y_back, 16) || !aligned(y_pairs, 16)) return kMisaligned;
  const cudaError_t e = launch(moe_ep_unpack_kernel, dim3((unsigned)n_pairs), dim3(128), 0, (cudaStream_t)stream, y_back,
                               (int)hidden, (const int*)sorted_ids, (const int*)expert_offsets, (int)n_pairs, (int)experts_per_rank,
                               (int)world, (int)capacity, y_pairs);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_moe_combine(const float* y_pairs, const int32_t* topk_ids, const float* topk_weights, int64_t n_tokens,
                          int32_t top_k, int64_t n, float* out, void* stream) {
  if (n_tokens < 0 || n_tokens > (1 << 24) || top_k <= 0 || top_k > kMoeMaxTopK || n <= 0 || n > (1 << 24))
    return kInvalidProblem;
  if (n_tokens == 0) return kOk;
  if (!y_pairs || !topk_ids || !topk_weights || !out) return kInvalidProblem;
  const cudaError_t e = launch(moe_combine_kernel, dim3((unsigned)n_tokens), dim3(256), 0, (cudaStream_t)stream, y_pairs,
                               (const int*)topk_ids, topk_weights, (int)top_k, (int)n, out);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

// ---- tensor-parallel decode over peer-mapped memory (peer.cuh)
namespace {
int32_t make_peer_ctx(const fuelq_peers* peers, int32_t wait_seq, int32_t push_seq, PeerCtx* c) {
  if (!peers || peers->world < 1 || peers->world > kPeerMaxWorld || peers->rank < 0 || peers->rank >= peers->world)
    return kInvalidProblem;
  if (wait_seq >= kPeerMaxSeq || push_seq >= kPeerMaxSeq) return kInvalidProblem;
  if (!peers->epoch) return kInvalidProblem;
  c->world = peers->world;
  c->rank = peers->rank;
  c->wait_seq = wait_seq < 0 ? -1 : wait_seq;
  c->push_seq = push_seq < 0 ? -1 : push_seq;
  c->epoch = peers->epoch;
  c->wait_ns = (unsigned long long)g_opt.peer_wait_ms * 1000000ull;
  return kOk;
}
}  // namespace

size_t fuelq_peer_vec_bytes(int64_t n) { return n > 0 ? (size_t)n * 8 : 0; }

int32_t fuelq_ipc_alloc(size_t bytes, void** dev_ptr, void* handle64) {
  if (!dev_ptr || !handle64 || bytes == 0) return kInvalidProblem;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return kLaunchFailure;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
      cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, p) != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return kLaunchFailure;
  }
  *dev_ptr = p;
  return kOk;
}
int32_t fuelq_ipc_open(const void* handle64, void** dev_ptr) {
  if (!handle64 || !dev_ptr) return kInvalidProblem;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  if (cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return kLaunchFailure;
  }
  return kOk;
}
int32_t fuelq_ipc_close(void* dev_ptr) {
  if (!dev_ptr) return kOk;
  return cudaIpcCloseMemHandle(dev_ptr) == cudaSuccess ? kOk : kLaunchFailure;
}
int32_t fuelq_ipc_free(void* dev_ptr) {
  if (!dev_ptr) return kOk;
  return cudaFree(dev_ptr) == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_qmatmul_packed_peer(int32_t ggml_type, int64_t k, int64_t n_local, const void* w, const void* act,
                                  void* const* dst, int64_t dst_offset, const fuelq_peers* peers, int32_t push_seq,
                                  void* stream) {
  const int32_t st = check_problem(ggml_type, 1, n_local, k);
  if (st != kOk) return st;
  if (n_local == 0 || dst_offset < 0) return kInvalidProblem;  // every rank contributes to an exchange point
  if (!w || !act || !dst) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(act, 16)) return kMisaligned;
  DecodeRegsPeer g;
  const int32_t sc = make_peer_ctx(peers, -1, push_seq, &g.ctx);
  if (sc != kOk) return sc;
  if (g.ctx.push_seq < 0) return kInvalidProblem;
  for (int q = 0; q < kPeerMaxWorld; ++q) {
    g.dst[q] = nullptr;
    if (q >= g.ctx.world) continue;
    if (!dst[q]) return kInvalidProblem;
    if (!aligned(dst[q], 16)) return kMisaligned;
    g.dst[q] = (uint2*)dst[q] + dst_offset;
  }
  const ActPlanes planes = act_planes(const_cast<void*>(act), ggml_type, 1, k);
  return decode_regs_impl(ggml_type, 1, n_local, k, w, planes, nullptr, (cudaStream_t)stream, &g);
}

int32_t fuelq_qmatmul_packed_tree(int32_t ggml_type, int64_t n, int64_t k, const void* w, const void* packed_act, float* y,
                                  int32_t n_leaves, const int32_t* leaf_blocks, void* stream) {
  const int32_t st = check_problem(ggml_type, 1, n, k);
  if (st != kOk) return st;
  if (n == 0) return kOk;
  if (!w || !packed_act || !y) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(packed_act, 16) || !aligned(y, 4)) return kMisaligned;
  return decode_tree_impl(ggml_type, n, k, w, act_planes(const_cast<void*>(packed_act), ggml_type, 1, k), y, n_leaves, leaf_blocks,
                          nullptr, (cudaStream_t)stream);
}

int32_t fuelq_qmatmul_packed_tree_peer(int32_t ggml_type, int64_t n, int64_t k, const void* w, const void* packed_act,
                                       void* const* dst, int64_t dst_offset, const fuelq_peers* peers, int32_t push_seq,
                                       int32_t n_leaves, const int32_t* leaf_blocks, void* stream) {
  const int32_t st = check_problem(ggml_type, 1, n, k);
  if (st != kOk) return st;
  if (n == 0 || dst_offset < 0) return kInvalidProblem;
  if (!w || !packed_act || !dst) return kInvalidProblem;
  if (!aligned(w, 16) || !aligned(packed_act, 16)) return kMisaligned;
  DecodeRegsPeer g;
  const int32_t sc = make_peer_ctx(peers, -1, push_seq, &g.ctx);
  if (sc != kOk) return sc;
  if (g.ctx.push_seq < 0) return kInvalidProblem;
  for (int q = 0; q < kPeerMaxWorld; ++q) {
    g.dst[q] = nullptr;
    if (q >= g.ctx.world) continue;
    if (!dst[q]) return kInvalidProblem;
    if (!aligned(dst[q], 16)) return kMisaligned;
    g.dst[q] = (uint2*)dst[q] + dst_offset;
  }
  return decode_tree_impl(ggml_type, n, k, w, act_planes(const_cast<void*>(packed_act), ggml_type, 1, k), nullptr, n_leaves,
                          leaf_blocks, &g, (cudaStream_t)stream);
}

int32_t fuelq_add_rmsnorm_q8k_parts(float* x, const float* parts, int32_t n_parts, const float* gain, int64_t dim, float eps,
                                    void* packed, size_t packed_bytes, void* stream) {
  if (dim <= 0 || dim % 256 || dim > 8192) return kInvalidProblem;
  if (n_parts != 1 && n_parts != 2 && n_parts != 4 && n_parts != 8) return kInvalidProblem;
  if (!x || !gain || !parts) return kInvalidProblem;
  if (!packed || packed_bytes < act_packed_bytes(kQ4K, 1, dim)) return kWorkspace;
  if (!aligned(x, 16) || !aligned(gain, 16) || !aligned(parts, 16) || !aligned(packed, 16)) return kMisaligned;
  const ActPlanes a = act_planes(packed, kQ4K, 1, dim);
  const cudaError_t e = launch(add_rmsnorm_q8k_parts_kernel, dim3(1), dim3((unsigned)(dim / 256 * 32)), 0, (cudaStream_t)stream, x,
                               parts, (int)n_parts, gain, (int)dim, eps, (int8_t*)a.qs, (float*)a.d, (int16_t*)a.bsums);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_add_rmsnorm_q8k_peer(float* x, const void* delta, int32_t n_parts, const float* gain, int64_t dim, float eps,
                                   void* packed, size_t packed_bytes, const fuelq_peers* peers, int32_t wait_seq, void* stream) {
  if (dim <= 0 || dim % 256 || dim > 8192) return kInvalidProblem;
  if (!x || !gain) return kInvalidProblem;
  if (!packed || packed_bytes < act_packed_bytes(kQ4K, 1, dim)) return kWorkspace;
  if (!aligned(x, 16) || !aligned(gain, 16) || (delta && !aligned(delta, 16)) || !aligned(packed, 16)) return kMisaligned;
  PeerCtx c;
  const int32_t sc = make_peer_ctx(peers, wait_seq, -1, &c);
  if (sc != kOk) return sc;
  if ((delta != nullptr) != (c.wait_seq >= 0)) return kInvalidProblem;
  if (delta && n_parts != 1 && n_parts != 2 && n_parts != 4 && n_parts != 8) return kInvalidProblem;
  const ActPlanes a = act_planes(packed, kQ4K, 1, dim);
  const cudaError_t e = launch(add_rmsnorm_q8k_peer_kernel, dim3(1), dim3((unsigned)(dim / 256 * 32)), 0, (cudaStream_t)stream,
                               x, (const uint2*)delta, (int)(delta ? n_parts : 0), gain, (int)dim, eps, (int8_t*)a.qs, (float*)a.d,
                               (int16_t*)a.bsums, c);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_rowpar_reduce(const void* own_parts, int32_t n_parts, int64_t n, float* y, const fuelq_peers* peers,
                            int32_t wait_seq, void* stream) {
  if (n <= 0 || n % 4 || n > (1 << 24)) return kInvalidProblem;
  if (n_parts != 1 && n_parts != 2 && n_parts != 4 && n_parts != 8) return kInvalidProblem;
  if (!own_parts || !y) return kInvalidProblem;
  if (!aligned(own_parts, 16) || !aligned(y, 16)) return kMisaligned;
  PeerCtx c;
  const int32_t sc = make_peer_ctx(peers, wait_seq, -1, &c);
  if (sc != kOk) return sc;
  if (c.wait_seq < 0) return kInvalidProblem;
  const cudaError_t e = launch(rowpar_reduce_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                               (const uint2*)own_parts, (int)n_parts, (int)n, y, c);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_argmax_last_peer(const void* x, int64_t n, int32_t* out_index, const fuelq_peers* peers, int32_t wait_seq,
                               uint32_t* epoch, void* stream) {
  if (n <= 0 || n % 2 || n > (1 << 30)) return kInvalidProblem;
  if (!x || !out_index || !epoch) return kInvalidProblem;
  if (!aligned(x, 16)) return kMisaligned;
  PeerCtx c;
  const int32_t sc = make_peer_ctx(peers, wait_seq, -1, &c);
  if (sc != kOk) return sc;
  if (epoch != c.epoch || c.wait_seq < 0) return kInvalidProblem;
  const cudaError_t e = launch(argmax_last_peer_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, (const float*)x, (int)n,
                               (int*)out_index, c, epoch);
  return e == cudaSuccess ? kOk : kLaunchFailure;
}

int32_t fuelq_dequantize(int32_t ggml_type, int64_t numel, const void* blocks, void* y, int32_t out_type,
                         void* stream_v) {
  if (out_type != kF32 && out_type != kF16 && out_type != kBF16) return kNotSupported;
  return dequantize_impl(ggml_type, numel, blocks, y, out_type, (cudaStream_t)stream_v);
}

}  // extern "C"
