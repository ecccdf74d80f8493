//! Raw bindings of `libfuelq.so`. One declaration per symbol of `include/fuelq.h`, `include/fuelq_host.h`,
//! `include/fuelq_seam.h` and `include/fuelq_gguf.h` that the `fuelq` crate uses. Every entry returns an `i32`
//! status with the meaning fuel's CUDA FFI wrappers already map
//! (`fuel-cuda-backend/src/baracuda/status.rs:5-12`): 0 ok, 1 misaligned, 2 invalid problem, 3 not supported,
//! 4 workspace, 5 launch failure. `ggml_type` is `GgmlDType::to_u32()` (`fuel-ir/src/quantized.rs:57-75`);
//! `stream` is a `cudaStream_t`.
#![allow(non_camel_case_types)]

use std::ffi::{c_char, c_int, c_void};

pub const FUELQ_OK: i32 = 0;
pub const FUELQ_OPT_PDL: i32 = 1;
pub const FUELQ_OPT_DECODE_MAX_M: i32 = 2;
pub const FUELQ_OPT_PREFILL_TF32: i32 = 8;
pub const FUELQ_OPT_PREFILL_BF16: i32 = 9;
pub const FUELQ_OPT_PREFILL_ONE_KERNEL: i32 = 10;
pub const FUELQ_NUMERICS_INTEGER: i32 = 0;
pub const FUELQ_NUMERICS_BF16: i32 = 1;
pub const FUELQ_NUMERICS_TF32: i32 = 2;
pub const FUELQ_NUMERICS_F16: i32 = 3;

/// The handshake envelope, `fuel_kernel_seam_announce::SeamHello` field for field (56 bytes).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct fuelq_seam_hello_t {
    pub magic: u32,
    pub envelope_version: u8,
    pub reserved: [u8; 3],
    pub profiles_len: u16,
    pub profiles: [u16; 16],
    pub reserved1: [u8; 6],
    pub capabilities: u64,
}
const _: () = assert!(std::mem::size_of::<fuelq_seam_hello_t>() == 56);

#[repr(C)]
pub struct FuelqGguf {
    _opaque: [u8; 0],
}

#[repr(C)]
pub struct fuelq_gguf_tensor {
    pub name: *const c_char,
    pub ggml_type: i32,
    pub n_dims: i32,
    pub dims: [i64; 8],
    pub offset: u64,
    pub nbytes: u64,
    pub data: *const c_void,
}

unsafe extern "C" {
    pub fn fuelq_seam_hello(out: *mut fuelq_seam_hello_t) -> c_int;

    pub fn fuelq_status_string(status: i32) -> *const c_char;
    pub fn fuelq_block_elems(ggml_type: i32) -> i32;
    pub fn fuelq_block_bytes(ggml_type: i32) -> i32;
    pub fn fuelq_set_option(key: i32, value: i64) -> i32;
    pub fn fuelq_get_option(key: i32) -> i64;
    pub fn fuelq_device_error(host_code_out: *mut i32, clear: i32) -> i32;

    pub fn fuelq_qmatmul_workspace_bytes(ggml_type: i32, m_total: i64, n: i64, k: i64) -> usize;
    pub fn fuelq_qmatmul_can_implement(ggml_type: i32, m_total: i64, n: i64, k: i64) -> i32;
    pub fn fuelq_qmatmul_numerics(ggml_type: i32, m_total: i64, n: i64, k: i64) -> i32;
    pub fn fuelq_qmatmul(
        ggml_type: i32, m_total: i64, n: i64, k: i64, w: *const c_void, x: *const f32, y: *mut f32,
        workspace: *mut c_void, workspace_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_quantize_act(
        weight_type: i32, m_total: i64, k: i64, x: *const f32, q8_blocks: *mut c_void, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_quantize_weights(
        ggml_type: i32, numel: i64, x: *const f32, blocks: *mut c_void, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_dequantize(
        ggml_type: i32, numel: i64, blocks: *const c_void, y: *mut c_void, out_type: i32, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_prefetch_weights(w: *const c_void, bytes: i64, stream: *mut c_void) -> i32;

    // mixture-of-experts block: the body of DynQuantizedStorage::indexed_moe_forward
    pub fn fuelq_moe_route(
        logits: *const f32, n_tokens: i64, n_experts: i32, top_k: i32, topk_ids: *mut i32, topk_weights: *mut f32,
        stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_moe_bucket(
        topk_ids: *const i32, n_pairs: i64, n_experts: i32, sorted_ids: *mut i32, expert_offsets: *mut i32,
        stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_moe_quantize_rows(
        x: *const f32, k: i64, row_ids: *const i32, divisor: i32, n_rows: i64, packed: *mut c_void,
        packed_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_moe_swiglu_quantize(
        gate_up: *const f32, f: i64, n_rows: i64, packed: *mut c_void, packed_bytes: usize, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_moe_qmatmul(
        ggml_type: i32, n_experts: i32, n: i64, k: i64, w: *const c_void, packed_act: *const c_void, n_rows: i64,
        expert_offsets: *const i32, out_rows: *const i32, y: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn fuelq_moe_combine(
        y_pairs: *const f32, topk_ids: *const i32, topk_weights: *const f32, n_tokens: i64, top_k: i32, n: i64,
        out: *mut f32, stream: *mut c_void,
    ) -> i32;

    // GGUF reader
    pub fn fuelq_last_error() -> *const c_char;
    pub fn fuelq_gguf_open(path: *const c_char, out: *mut *mut FuelqGguf) -> i32;
    pub fn fuelq_gguf_close(g: *mut FuelqGguf) -> i32;
    pub fn fuelq_gguf_find_tensor(g: *const FuelqGguf, name: *const c_char) -> i64;
    pub fn fuelq_gguf_tensor_at(g: *const FuelqGguf, index: i64, out: *mut fuelq_gguf_tensor) -> i32;
    pub fn fuelq_gguf_load_tensor(
        g: *const FuelqGguf, index: i64, byte_offset: u64, nbytes: u64, device_dst: *mut c_void, stream: *mut c_void,
    ) -> i32;
}
