/* fuelq — B200 (sm_100a) kernels for fuel's GGUF k-quant matrix multiply.
 *
 * C ABI of libfuelq.so: the symbols a fuel backend binds in place of the
 * quantized entries it gets today from its CUDA kernel provider. Conventions are
 * the ones fuel's FFI wrappers already assume (fuel-cuda-backend/src/quantized.rs:58-65,
 * 138-144; fuel-cuda-backend/src/baracuda/status.rs:5-12):
 *   - every entry returns an int32 status: 0 ok, 1 misaligned operand, 2 invalid
 *     problem, 3 not supported, 4 workspace too small or null, 5 launch failure;
 *   - all pointers are device pointers on the current device unless the name says
 *     host; weights are GGUF block bytes, row-major [n][k / block] ("one row per
 *     output feature"), activations and outputs contiguous row-major f32;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call
 *     returns without synchronizing; nothing is allocated; outputs and workspace
 *     are caller-owned.
 */
#ifndef FUELQ_H_
#define FUELQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FUELQ_OK 0
#define FUELQ_MISALIGNED 1
#define FUELQ_INVALID_PROBLEM 2
#define FUELQ_NOT_SUPPORTED 3
#define FUELQ_WORKSPACE 4
#define FUELQ_LAUNCH_FAILURE 5

/* GGUF type ids (fuel-ir/src/quantized.rs:35-75, GgmlDType::to_u32). */
#define FUELQ_TYPE_F32 0
#define FUELQ_TYPE_F16 1
#define FUELQ_TYPE_Q4_0 2
#define FUELQ_TYPE_Q4_1 3 /* Q4_1, Q5_0, Q5_1: mat-vec at every batch size through the exact-integer decode kernel, */
#define FUELQ_TYPE_Q5_0 6 /* dequantize, and the weight quantizer; Q4_1 / Q5_1 take Q8_1 activation blocks          */
#define FUELQ_TYPE_Q5_1 7
#define FUELQ_TYPE_Q8_0 8
#define FUELQ_TYPE_Q8_1 9 /* activation blocks only (the dot-product partner of Q4_1 / Q5_1) */
#define FUELQ_TYPE_Q2K 10 /* Q2_K, Q3_K: mat-vec at every batch size through the exact-integer decode kernel, dequantize, quantizer */
#define FUELQ_TYPE_Q3K 11
#define FUELQ_TYPE_Q4K 12
#define FUELQ_TYPE_Q5K 13 /* mat-vec (every batch size through the exact-integer decode kernels), dequantize, weight quantizer */
#define FUELQ_TYPE_Q6K 14
#define FUELQ_TYPE_Q8K 15
#define FUELQ_TYPE_BF16 30

/* Text for a status code (fuel-cuda-backend/src/baracuda/status.rs:37-48, status_reason). */
const char* fuelq_status_string(int32_t status);

/* Elements / bytes per block (fuel-ir/src/quantized.rs:77-103, GgmlDType::block_size / type_size).
 * 0 for a type this library does not handle. */
int32_t fuelq_block_elems(int32_t ggml_type);
int32_t fuelq_block_bytes(int32_t ggml_type);

/* Options. key: */
#define FUELQ_OPT_PDL 1          /* 1: launch kernels with programmatic dependent launch so a kernel's weight
                                    prefetch overlaps its predecessor's tail (default 0) */
#define FUELQ_OPT_DECODE_MAX_M 2 /* largest m_total routed to the integer kernels; above it the tensor-core GEMM runs
                                    (every block format, k a multiple of 64). 0 (default) = the library's choice: 16,
                                    and 64 for Q4_K / Q5_K / Q6_K / Q8_0 with k a multiple of 256 (the integer tensor-core
                                    kernel, 16 rows per pass over the weights, is still the faster of the two there).
                                    Any positive value is taken as given */
#define FUELQ_OPT_DECODE_GRID 3  /* CTAs for the decode kernel; 0 = two per SM (default) */
#define FUELQ_OPT_DECODE_KERNEL 4 /* 0 = pick per problem (default); 1 = generic decode kernel (activations read
                                    through L1, any M <= 16); 2 = register-resident kernel only (M <= 2) */
#define FUELQ_OPT_L2_PREFETCH 5   /* 1: every mat-vec call first enqueues a small kernel that streams its weight
                                    matrix from HBM into L2; with FUELQ_OPT_PDL it runs beside the preceding
                                    kernels, so the transfer overlaps their work (default 0) */
#define FUELQ_OPT_FUSED_QUANT 6   /* 1: fuelq_qmatmul with m_total <= 2 and Q4_K / Q6_K weights runs as ONE kernel
                                    whose thread blocks quantize the activation rows themselves (same bytes as
                                    fuelq_quantize_act). 0 (default): the library's choice - one kernel for one row
                                    of a small matrix (up to 12 MiB of blocks), else quantize kernel, then mat-vec
                                    kernel, which measured faster in a chain of launches (the small kernel overlaps
                                    the previous mat-vec's tail). Same bits either way */
#define FUELQ_OPT_PEER_WAIT_MS 7  /* deadline, in milliseconds, of the exchange polls in the fuelq_*_peer kernels (default
                                    4000, 1..60000): a kernel whose peer never delivers records device error 6 after
                                    this long and carries on, so the context stays usable */
#define FUELQ_OPT_PREFILL_TF32 8  /* 1: the tensor-core path (m_total above the integer crossover) multiplies in tf32
                                    instead of 16-bit operands: weights dequantized to f32 and rounded to tf32,
                                    activations rounded to tf32, f32 accumulation. Half the MMA rate, twice the
                                    workspace (4 bytes per activation; ask fuelq_qmatmul_workspace_bytes after
                                    setting it); the same 10 mantissa bits as the default f16 operands (default 0) */
#define FUELQ_OPT_PREFILL_BF16 9  /* 1: the tensor-core path's 16-bit operands are bf16 (7 mantissa bits: results about
                                    2.5e-3 from the exact dequantized product). 0 (default): f16 (10 mantissa bits,
                                    about 4e-4, same MMA rate): weights dequantized straight to f16 (finite values
                                    saturate at +-65504, far beyond any GGUF weight), every activation row scaled
                                    by a power of two into f16's range and the result row scaled back, both exact */
#define FUELQ_OPT_PREFILL_ONE_KERNEL 10 /* The tensor-core path takes the weights as a slab of rows dequantized into the
                                    operand type by the stand-alone dequantizing kernels (the slab, at most 128 MiB,
                                    is part of the workspace fuelq_qmatmul_workspace_bytes reports) and multiplies
                                    slab by slab; both operands then reach the tensor cores by tensor-map copies.
                                    1: Q4_K / Q6_K / Q8_0 are instead dequantized inside the GEMM kernel - no slab
                                    in the workspace, measured slower above ~100 rows (Q4_K 4096 -> 14336 at 2048
                                    rows: 575 against 746 TFLOP/s). Same operand values either way for Q6_K and
                                    Q8_0; Q4_K's in-kernel form fuses d*sc*q - dmin*m into one rounding where the
                                    slab form has the reference's two (default 0) */
int32_t fuelq_set_option(int32_t key, int64_t value);
int64_t fuelq_get_option(int32_t key);

/* Reads (and, if `clear`, resets) the device-side error word set by a kernel whose
 * bounded wait expired. Synchronizes the device. 0 = no error recorded. */
int32_t fuelq_device_error(int32_t* host_code_out, int32_t clear);

/* Activation quantization to the weight format's dot-product partner: Q8_K blocks for Q2K / Q3K / Q4K / Q5K / Q6K
 * weights, Q8_1 blocks for Q4_1 / Q5_1, Q8_0 blocks otherwise - the first half of the reference's matmul
 * (fuel-quantized/src/k_quants.rs:2303-2313; BlockQ8K::from_float :2230-2267, BlockQ8_1::from_float :728-757,
 * BlockQ8_0::from_float :629-658). Output bytes are identical to the reference's.
 * x: f32 [m_total, k]; q8_blocks: m_total * k / block * block_bytes bytes, 4-byte aligned. */
int32_t fuelq_quantize_act(int32_t weight_type, int64_t m_total, int64_t k, const float* x, void* q8_blocks,
                           void* stream);

/* Same numbers in the plane-split layout the mat-vec kernels read (int8 plane, f32 scale
 * plane, int16 block-sum plane). Lets several projections of one input (Q/K/V, gate/up)
 * share one quantization — the reference re-quantizes per call (k_quants.rs:2303-2313). */
size_t fuelq_act_packed_bytes(int32_t weight_type, int64_t m_total, int64_t k);
int32_t fuelq_quantize_act_packed(int32_t weight_type, int64_t m_total, int64_t k, const float* x, void* packed,
                                  size_t packed_bytes, void* stream);

/* Workspace needed by fuelq_qmatmul for this problem (the FFI contract the reference
 * follows passes (workspace, workspace_bytes) on every call, quantized.rs:193-195). */
size_t fuelq_qmatmul_workspace_bytes(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k);

/* Which arithmetic fuelq_qmatmul uses for this problem under the current options. The reference's CPU path
 * (fuel_quantized::matmul, k_quants.rs:2284-2331) has ONE arithmetic for every batch size: activations
 * re-quantized to 8-bit blocks, exact integer dot products per sub-block, f32 block sums. This library keeps that
 * arithmetic up to the crossover batch size and multiplies dequantized weights with f16 (or bf16, tf32) activations
 * on the tensor cores above it, so RESULTS CHANGE CLASS AT THE CROSSOVER: integer results sit within f32
 * summation order (~1e-6) of the reference's, tensor-core results differ from them by the activation
 * quantization the reference applies and this path does not (up to ~2e-2 of the largest output) and from the
 * exact dequantized product by ~4e-4 (f16, the default, and tf32) or ~2.5e-3 (bf16). Callers that need the reference's numbers at any
 * batch size raise FUELQ_OPT_DECODE_MAX_M. Returns one of the values below, or a negative status (-FUELQ_...). */
#define FUELQ_NUMERICS_INTEGER 0 /* the reference's arithmetic */
#define FUELQ_NUMERICS_BF16 1
#define FUELQ_NUMERICS_TF32 2
#define FUELQ_NUMERICS_F16 3
int32_t fuelq_qmatmul_numerics(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k);

/* 0 if fuelq_qmatmul handles (type, m_total, n, k), else the status it would return. */
int32_t fuelq_qmatmul_can_implement(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k);

/* y[m_total, n] = x[m_total, k] * W[n, k]^T with W in GGUF blocks — QMatMul::forward /
 * DynQuantizedStorage::fwd (fuel-backend-contract/src/quantized.rs:72-80), i.e.
 * fuel_quantized::matmul (k_quants.rs:2284-2331) and the CUDA entry it replaces,
 * baracuda_kernels_mmvq_<fmt>_batched_run (fuel-cuda-backend/src/quantized.rs:138-231).
 * Up to the crossover (FUELQ_OPT_DECODE_MAX_M) it quantizes x and runs the integer decode kernels; above it the
 * tensor-core path (activations converted to the operand type, weights dequantized into a slab of the workspace, one
 * GEMM per slab). Weight formats: Q4_K, Q6_K, Q8_0, Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K and Q5_K on both paths; the
 * tensor-core path needs k to be a multiple of 64 (other k stay on the integer kernels at any m_total).
 * w must be 16-byte aligned, x and y 16-byte aligned. */
int32_t fuelq_qmatmul(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w, const float* x,
                      float* y, void* workspace, size_t workspace_bytes, void* stream);

/* fuelq_qmatmul for callers holding HOST activations: copies x_host to the device, runs the
 * product and copies y back, all enqueued on `stream` (pinned host memory keeps it
 * asynchronous); the caller synchronizes the stream before reading y_host. This is the
 * shape of the reference's eager CUDA forward, which stages small host arrays and reads
 * results back around every call (fuel-cuda-backend/src/quantized.rs:170-231), without
 * its per-call allocations and device synchronize. On the integer path, when both host buffers
 * are page-locked and mapped into the device's address space (cudaHostAlloc, cudaHostRegister
 * with the mapped flag) and small (x <= 256 KiB, y <= 1 MiB), no copy is enqueued at all: the
 * quantizing kernel reads x in place and a small kernel writes y in place, same bits either way.
 * x_host must hold its final contents when the call is made: it is read at some time between the
 * call and the completion of the enqueued work, not necessarily after earlier work of the stream.
 * workspace: device, 256-byte aligned, fuelq_qmatmul_host_workspace_bytes() bytes. */
size_t fuelq_qmatmul_host_workspace_bytes(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k);
int32_t fuelq_qmatmul_host(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                           const float* x_host, float* y_host, void* workspace, size_t workspace_bytes,
                           void* stream);

/* fuelq_qmatmul without a workspace argument, for callers that are not able to allocate device
 * memory (no counterpart in the reference, whose CUDA forward allocates on every call,
 * fuel-cuda-backend/src/quantized.rs:193-198): a plug-in that receives device pointers but owns no
 * allocator, or code whose memory was fixed before it started. The activation scratch is a 1 MiB
 * array built into the library and resident on every GPU that loads it until the process ends.
 *  - problems whose activation blocks need more than fuelq_static_scratch_bytes() are refused with
 *    status 4 (roughly m_total * k > 900 000 elements); nothing is truncated;
 *  - the first call on each device also does the set-up (it looks up the array's device address);
 *    that first call should come before any stream capture begins;
 *  - all calls share the one array: two calls whose kernels may run at the same time on the GPU
 *    (different streams, or different host threads) would overwrite each other's activations. Keep
 *    them on one stream. Nothing in the array has to be cleared between calls.
 * Results are bit-identical to fuelq_qmatmul, except for tensor-core problems (fuelq_qmatmul_numerics != 0) whose
 * activations fit the array but whose slab of dequantized weight rows does not: those run without a slab - Q4_K,
 * Q6_K and Q8_0 as under FUELQ_OPT_PREFILL_ONE_KERNEL (same arithmetic class), the other formats on the integer
 * kernels (the reference's arithmetic). Calls no allocation routine of any kind. */
size_t fuelq_static_scratch_bytes(void);
int32_t fuelq_qmatmul_static_scratch(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                                     const float* x, float* y, void* stream);

/* Streams `bytes` of a weight buffer from HBM into L2 ahead of the call that will read it (no
 * reference counterpart: the reference has no notion of cache residency; the nearest thing is its
 * transfer-cost model, fuel-hardware/src/transfer_cost.rs). Purely a hint: results never depend on it. */
int32_t fuelq_prefetch_weights(const void* w, int64_t bytes, void* stream);

/* The mat-vec alone, on activations already quantized by fuelq_quantize_act_packed. */
int32_t fuelq_qmatmul_packed(int32_t ggml_type, int64_t m_total, int64_t n, int64_t k, const void* w,
                             const void* packed_act, float* y, void* stream);

/* f32 -> GGUF blocks on the device, byte-identical to the reference's host quantizers
 * (GgmlType::from_float: Q8_0 k_quants.rs:629-658, Q4_0 :199-235, Q4_1 :315-351, Q5_0 :424-460, Q5_1 :535-575,
 * Q4_K :1470-1528 and Q5_K :1732-1887 with make_qkx1_quants utils.rs:229-286, Q6_K :2005-2075 with make_qx_quants
 * utils.rs:62-191, Q2_K :836-895, Q3_K :1135-1216 with make_q3_quants utils.rs:289-354). The importance-matrix
 * quantizers are not built.
 * This is DynQuantizedStorage::quantize (fuel-backend-contract/src/quantized.rs:34-35); the
 * reference's CUDA backend does it on the CPU and uploads (fuel-cuda-backend/src/quantized.rs:389-412).
 * x: f32 [numel] device, 16-byte aligned; numel a multiple of the block size. */
int32_t fuelq_quantize_weights(int32_t ggml_type, int64_t numel, const float* x, void* blocks, void* stream);

/* Blocks -> floats: DynQuantizedStorage::dequantize / dequantize_f16
 * (fuel-backend-contract/src/quantized.rs:56-62), GgmlType::to_float; replaces
 * baracuda_kernels_dequantize_<fmt>_run (fuel-cuda-backend/src/quantized.rs:58-105).
 * out_type: FUELQ_TYPE_F32, _F16 or _BF16. numel a multiple of the block size. */
int32_t fuelq_dequantize(int32_t ggml_type, int64_t numel, const void* blocks, void* y, int32_t out_type,
                         void* stream);

/* ---- callers of the hot path: f32 glue of a LLaMA-style decode step, batch 1 -------------------------
 * What the reference's model code runs between its quantized linears (fuel-core/src/lazy.rs:7363-7447).
 * All device pointers; `pos` points at the current position on the device so a step can be replayed
 * from a CUDA graph. */

/* token ids -> rows of an embedding table [vocab][k]: ggml_type 12 = Q4_K blocks, dequantized on the fly
 * (the synthetic 7B-architecture workload quantizes its embeddings); 0 = f32, which is how the reference keeps
 * every embedding table after loading (fuel-core/src/lazy.rs:8626-8636, lazy_quantized_llama.rs:287). */
int32_t fuelq_embed_rows(int32_t ggml_type, const void* table, int64_t k, const int32_t* ids, int64_t n_ids, float* out,
                         void* stream);
/* x += delta (delta may be null), then out = x / sqrt(mean(x^2) + eps) * gain, per row
 * (rms_norm_last_dim_f32, fuel-cpu-backend/src/byte_kernels.rs:2339-2367 + the affine gain of lazy.rs:10330-10347).
 * dim a multiple of 256, at most 8192; pointers 16-byte aligned. */
int32_t fuelq_add_rmsnorm(float* x, const float* delta, const float* gain, float* out, int64_t rows, int64_t dim, float eps,
                          void* stream);
/* rotate-half RoPE of q [n_heads][hd] (in place) and k [n_kv][hd] at position *pos, then store the rotated k
 * and v into caches [n_kv][max_seq][hd] (rope_f32, byte_kernels.rs:1885-1960; cache layout lazy.rs:8578-8700). */
int32_t fuelq_rope_store(float* q, const float* k, const float* v, float* kcache, float* vcache, const float* cos_table,
                         const float* sin_table, const int32_t* pos, int32_t n_heads, int32_t n_kv, int32_t head_dim,
                         int32_t max_seq, void* stream);
/* out[h] = softmax(q[h] . K[kv(h)][0..*pos]^T * scale) . V, max-subtracted softmax (byte_kernels.rs:2259-2305). head_dim 128. */
/* Optional fusion of fuelq_rope_store into the attention call: with a non-null `rope`, q arrives unrotated, the current
 * token's k and v are read from rope->k / rope->v (k rotated on the fly), and the call appends them to the caches
 * itself - same values as fuelq_rope_store followed by the call with rope = NULL, one launch fewer. */
typedef struct fuelq_rope {
  const float* k;         /* [n_kv][head_dim], unrotated */
  const float* v;         /* [n_kv][head_dim] */
  const float* cos_table; /* [max_seq][head_dim] */
  const float* sin_table;
  float* kcache;          /* the caches passed to the call, writable */
  float* vcache;
} fuelq_rope;
size_t fuelq_attn_decode_workspace_bytes(int32_t n_heads);
int32_t fuelq_attn_decode(const float* q, const float* kcache, const float* vcache, float* out, const int32_t* pos,
                          int32_t n_heads, int32_t n_kv, int32_t head_dim, int32_t max_seq, float scale, void* workspace,
                          size_t workspace_bytes, const fuelq_rope* rope, void* stream);
/* Fused forms for a single-GPU step: the plain call followed by fuelq_quantize_act_packed (k-quant weights,
 * m = 1), written straight into the packed planes with the same bytes, one launch instead of two.
 * dim / n multiples of 256. */
int32_t fuelq_add_rmsnorm_q8k(float* x, const float* delta, const float* gain, int64_t dim, float eps, void* packed,
                              size_t packed_bytes, void* stream);
int32_t fuelq_swiglu_q8k(const float* gate, const float* up, int64_t n, void* packed, size_t packed_bytes, void* stream);
int32_t fuelq_attn_decode_q8k(const float* q, const float* kcache, const float* vcache, const int32_t* pos, int32_t n_heads,
                              int32_t n_kv, int32_t head_dim, int32_t max_seq, float scale, void* workspace,
                              size_t workspace_bytes, void* packed, size_t packed_bytes, const fuelq_rope* rope, void* stream);
/* Column-sharded form of fuelq_qmatmul for the tensor-core path (m_total above the integer crossover): this GPU
 * holds rows [n_offset, n_offset + n_local) of the weight matrix and computes those columns of Y; the kernel's
 * epilogue stores each output tile into EVERY destination y_dst[q] (an [m_total][n_total] matrix: this GPU's own, and
 * the other GPUs' mapped with fuelq_ipc_open), so when all GPUs' calls have completed every GPU holds the full Y - the
 * all-gather of the shards happens inside the kernel, as plain NVLink stores overlapped with the remaining tiles. The
 * reference has no multi-GPU form (fuel-core/src/quantized/mod.rs:854-868). The caller orders "all calls completed"
 * itself (stream sync + a process barrier, or an event per peer). Workspace: fuelq_qmatmul_workspace_bytes(type,
 * m_total, n_local, k). */
int32_t fuelq_qmatmul_sharded(int32_t ggml_type, int64_t m_total, int64_t n_local, int64_t k, const void* w_local,
                              const float* x, float* const* y_dst, int32_t n_dst, int64_t n_total, int64_t n_offset,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ---- Mixture-of-experts block with quantized experts (the grouped / indexed quantized mat-vec).
 * Replaces the slot the reference leaves empty (indexed_moe_forward, fuel-backend-contract/src/quantized.rs:29-103;
 * the CUDA implementation was retired and its grouped kernel is only named: fuel-cuda-backend/src/quantized.rs:292-304)
 * and follows the reference's sparse MoE forward for everything around it (fuel-core/src/lazy_nn/moe.rs:92-127,
 * 296-348): K rounds of first-maximum argmax with the picked logit lowered by 1e30, softmax over the picked logits,
 * experts visited in ascending id, rows inside an expert in ascending token order, a token's result accumulated as
 * ((0 + w_a*y_a) + w_b*y_b) + ... over its experts in ascending id. A "pair" is token * top_k + slot.
 * All calls are stream-ordered, allocate nothing and read the routing on the device (no host round trip). */
/* logits [n_tokens][n_experts] -> topk_ids, topk_weights [n_tokens][top_k]; n_experts <= 1024, top_k <= 16 */
int32_t fuelq_moe_route(const float* logits, int64_t n_tokens, int32_t n_experts, int32_t top_k, int32_t* topk_ids,
                        float* topk_weights, void* stream);
/* pairs sorted by expert (ascending pair id inside an expert) -> sorted_ids [n_pairs], expert_offsets [n_experts + 1] */
int32_t fuelq_moe_bucket(const int32_t* topk_ids, int64_t n_pairs, int32_t n_experts, int32_t* sorted_ids,
                         int32_t* expert_offsets, void* stream);
/* sorted row i <- Q8_K( x[row_ids[i] / divisor] ), packed as fuelq_quantize_act_packed lays out n_rows rows;
 * divisor = top_k gathers a token's row for each of its pairs, divisor = 1 gathers per pair */
int32_t fuelq_moe_quantize_rows(const float* x, int64_t k, const int32_t* row_ids, int32_t divisor, int64_t n_rows,
                                void* packed, size_t packed_bytes, void* stream);
/* rows [gate | up] of width 2f -> Q8_K( silu(gate) * up ), same packed layout (f a multiple of 256) */
int32_t fuelq_moe_swiglu_quantize(const float* gate_up, int64_t f, int64_t n_rows, void* packed, size_t packed_bytes,
                                  void* stream);
/* y[out_rows[i] or i][0..n) = W[e] . act row i for every sorted row i of every expert e (rows
 * expert_offsets[e] .. expert_offsets[e+1]); w is [n_experts][n][k] GGUF blocks, Q4_K or Q6_K, each row a multiple of
 * 16 bytes. An expert's matrix is streamed once, and not at all when it has no rows. */
int32_t fuelq_moe_qmatmul(int32_t ggml_type, int32_t n_experts, int64_t n, int64_t k, const void* w, const void* packed_act,
                          int64_t n_rows, const int32_t* expert_offsets, const int32_t* out_rows, float* y, void* stream);
/* out[t] = sum over the token's pairs, in ascending expert id, of topk_weights[pair] * y_pairs[pair] */
int32_t fuelq_moe_combine(const float* y_pairs, const int32_t* topk_ids, const float* topk_weights, int64_t n_tokens,
                          int32_t top_k, int64_t n, float* out, void* stream);

/* Expert parallelism inside one node, fixed sizes, nothing read on the host (fuel_b200/moe.py: QMoeExpertParallel). A
 * (source, destination) pair of ranks owns a chunk of capacity + 1 rows of `hidden` floats in the send / receive buffers
 * [world][capacity + 1][hidden]: the rows for that destination sorted by expert, then one row with their expert ids
 * as int32 (-1 = unused); capacity <= hidden. fuelq_moe_ep_pack fills the send buffer from the bucketed pairs of the
 * local tokens (expert_offsets over ALL experts, experts_per_rank consecutive experts per rank); after the
 * all-to-all, fuelq_moe_ep_local_ids turns the received id rows into one local expert id per slot (what
 * fuelq_moe_bucket takes; the slot index is the row index in the receive buffer); after the local experts and the
 * all-to-all back, fuelq_moe_ep_unpack moves every result row from its slot to its pair's row of y_pairs. */
int32_t fuelq_moe_ep_pack(const float* x, int64_t hidden, const int32_t* sorted_ids, const int32_t* expert_offsets,
                          const int32_t* topk_ids, int32_t top_k, int64_t n_pairs, int32_t experts_per_rank, int32_t world,
                          int64_t capacity, float* send, void* stream);
int32_t fuelq_moe_ep_local_ids(const float* recv, int64_t hidden, int64_t capacity, int32_t world, int32_t first_expert,
                               int32_t* local_ids, void* stream);
int32_t fuelq_moe_ep_unpack(const float* y_back, int64_t hidden, const int32_t* sorted_ids, const int32_t* expert_offsets,
                            int64_t n_pairs, int32_t experts_per_rank, int32_t world, int64_t capacity, float* y_pairs,
                            void* stream);

/* ---- Tensor-parallel decode step over peer-mapped memory.
 * The reference's quantized mat-vec runs on one device (fuel-core/src/quantized/mod.rs:854-868); these entry points are
 * how the 7B decode of the benchmark is split over the GPUs of one node, in the shape of the reference's tensor-parallel
 * layers (fuel-parallel/src/tensor_parallel.rs:283-343): column-parallel layers split by output rows, row-parallel layers
 * by k with their partial results summed by one fixed tree (see fuelq_qmatmul_packed_tree below), so the result has the
 * same bits for any GPU count. The slices are exchanged inside the producing and
 * consuming kernels: every 32-bit word that crosses GPUs is stored as an 8-byte pair {word, stamp} with one
 * store, straight into a destination buffer on every rank over NVLink; the consumer re-reads the pairs it
 * needs from its own buffer until all carry the expected stamp (with a deadline of a few seconds, after which
 * it records device error 6 and carries on). No fences, flags, collectives or multicast. A step has a fixed
 * list of exchange points numbered seq = 0 .. FUELQ_PEER_MAX_SEQ-1, each used once per step; the stamp is
 * epoch * FUELQ_PEER_MAX_SEQ + seq + 1, `epoch` counting steps on the device (advanced by
 * fuelq_argmax_last_peer), so a captured CUDA graph replays without changes. Destination buffers must start
 * zeroed, come from fuelq_ipc_alloc and are mapped into the other processes with fuelq_ipc_open. A buffer
 * may serve several exchange points of a step only if every rank must have consumed the earlier contents
 * before any rank can produce the later ones. All ranks issue the same sequence of calls. */
#define FUELQ_PEER_MAX_WORLD 8
#define FUELQ_PEER_MAX_SEQ 1024
typedef struct fuelq_peers {
  int32_t world, rank;
  const uint32_t* epoch; /* device word on this rank, starts at 0 */
} fuelq_peers;
/* bytes of a destination buffer for n f32 words */
size_t fuelq_peer_vec_bytes(int64_t n);
/* zeroed device memory that other processes of this node can map: handle64 receives 64 opaque bytes */
int32_t fuelq_ipc_alloc(size_t bytes, void** dev_ptr, void* handle64);
int32_t fuelq_ipc_open(const void* handle64, void** dev_ptr);
int32_t fuelq_ipc_close(void* dev_ptr);
int32_t fuelq_ipc_free(void* dev_ptr);
/* Column-parallel layer: y_local = W_local . act (m = 1, integer path; W_local is this rank's band of output rows),
 * stored as stamped pairs of push_seq at word dst_offset of the vector buffer dst[q] of every rank q. `act` is this
 * rank's packed planes of the whole input vector (fuelq_quantize_act_packed layout; Q4_K / Q6_K / Q8_0). */
int32_t fuelq_qmatmul_packed_peer(int32_t ggml_type, int64_t k, int64_t n_local, const void* w, const void* act,
                                  void* const* dst, int64_t dst_offset, const fuelq_peers* peers, int32_t push_seq,
                                  void* stream);
/* fuelq_add_rmsnorm_q8k whose delta is the sum of n_parts (1, 2, 4 or 8) partial vectors filled through wait_seq:
 * `delta` is a vector buffer of n_parts * dim words, part q at word q * dim (null and -1: no delta). The parts
 * are added pairwise, ((p0 + p1) + (p2 + p3)) + ..., the top levels of the tree fuelq_qmatmul_packed_tree sums by. */
int32_t fuelq_add_rmsnorm_q8k_peer(float* x, const void* delta, int32_t n_parts, const float* gain, int64_t dim, float eps,
                                   void* packed, size_t packed_bytes, const fuelq_peers* peers, int32_t wait_seq, void* stream);
/* The same with the parts as plain f32 vectors [n_parts][dim] in this GPU's memory (after a library all-gather). */
int32_t fuelq_add_rmsnorm_q8k_parts(float* x, const float* parts, int32_t n_parts, const float* gain, int64_t dim, float eps,
                                    void* packed, size_t packed_bytes, void* stream);

/* ---- Row-parallel layers: y = W . act with W cut along k (the reference's RowParallel::forward is a local matmul
 * followed by an all-reduce, fuel-parallel/src/tensor_parallel.rs:321-343, its sum folded in rank order,
 * fuel-parallel/src/device_group.rs:100-118). Here the sum over k follows ONE fixed tree at every GPU count: the k axis
 * of the whole layer is cut into eight leaves (ranges of whole 256-element blocks), a leaf is summed in an order of its
 * own, and leaves are added pairwise, ((l0 + l1) + (l2 + l3)) + ((l4 + l5) + (l6 + l7)). A GPU holds an aligned group of
 * 8 / world leaves, so its mat-vec yields a complete subtree, and adding the GPUs' results pairwise in rank order
 * (fuelq_add_rmsnorm_q8k_peer / _parts) finishes the same tree: the result has the same bits on 1, 2, 4 or 8 GPUs.
 * m = 1; Q4_K / Q6_K; w is this GPU's slab [n][k] (its k columns of every row, contiguous); leaf_blocks[l] is the
 * number of 256-element blocks of its leaf l (n_leaves = 1, 2, 4 or 8; at most 16 blocks per leaf). */
int32_t fuelq_qmatmul_packed_tree(int32_t ggml_type, int64_t n, int64_t k, const void* w, const void* packed_act, float* y,
                                  int32_t n_leaves, const int32_t* leaf_blocks, void* stream);
/* The same, the n results stored as stamped pairs of push_seq at word dst_offset of the vector buffer dst[q] of every rank q
 * (a rank of a row-parallel layer passes dst_offset = rank * n: part `rank` of the consumer's delta). */
int32_t fuelq_qmatmul_packed_tree_peer(int32_t ggml_type, int64_t n, int64_t k, const void* w, const void* packed_act,
                                       void* const* dst, int64_t dst_offset, const fuelq_peers* peers, int32_t push_seq,
                                       int32_t n_leaves, const int32_t* leaf_blocks, void* stream);
/* The all-reduce of a row-parallel layer by itself (the reference's RowParallel::forward ends in one,
 * fuel-parallel/src/tensor_parallel.rs:321-343): y[0..n) = ((p0 + p1) + (p2 + p3)) + ... over the n_parts (1, 2, 4 or 8)
 * partial vectors that the ranks' fuelq_qmatmul_packed_tree_peer calls stored into this rank's buffer own_parts through
 * exchange point wait_seq (part q at word q * n). The same value fuelq_add_rmsnorm_q8k_peer adds to the residual, for a
 * caller whose next op is something else; the same bits on every rank and at every GPU count. n a multiple of 4. */
int32_t fuelq_rowpar_reduce(const void* own_parts, int32_t n_parts, int64_t n, float* y, const fuelq_peers* peers,
                            int32_t wait_seq, void* stream);
/* fuelq_argmax_last over a vector buffer of n (even) words filled through wait_seq; then *epoch += 1
 * (epoch must be peers->epoch) */
int32_t fuelq_argmax_last_peer(const void* x, int64_t n, int32_t* out_index, const fuelq_peers* peers, int32_t wait_seq,
                               uint32_t* epoch, void* stream);
/* out = silu(gate) * up */
int32_t fuelq_swiglu(const float* gate, const float* up, float* out, int64_t n, void* stream);
/* index of the LAST maximum of x[0..n) (LogitsProcessor argmax: max_by + total_cmp,
 * fuel-transformers/src/generation/mod.rs:84-93). */
int32_t fuelq_argmax_last(const float* x, int64_t n, int32_t* out_index, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FUELQ_H_ */
