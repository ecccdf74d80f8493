//! Link registry for `contracts/qmatmul.fkc.md`: each contract's `entry_point` string resolves here to a
//! `KernelRef` (`fuel-dispatch/src/kernel.rs:168-173`); an entry the importer cannot find is its typed
//! `EntryPointUnresolved` error, not a panic. All three share one body: the block format comes from
//! `OpParams::QMatMul::quant_type`, as in the CPU wrapper (`fuel-dispatch/src/dispatch.rs:1630-1718`).

use std::ffi::c_void;
use std::sync::{Arc, RwLock};

use fuel_dispatch::kernel::{KernelRef, OpParams, Storage};
use fuel_graph::QuantType;
use fuel_ir::{DType, Error, GgmlDType, Layout, Result};

use crate::check;

pub static ENTRY_POINTS: &[(&str, KernelRef)] = &[
    ("fuelq::kernel_ref::qmatmul_q4k_f32", qmatmul_f32_b200),
    ("fuelq::kernel_ref::qmatmul_q6k_f32", qmatmul_f32_b200),
    ("fuelq::kernel_ref::qmatmul_q8_0_f32", qmatmul_f32_b200),
];

fn ggml_of(q: QuantType) -> Result<GgmlDType> {
    Ok(match q {
        QuantType::Q4_0 => GgmlDType::Q4_0,
        QuantType::Q8_0 => GgmlDType::Q8_0,
        QuantType::Q4_K_M => GgmlDType::Q4K,
        QuantType::Q5K => GgmlDType::Q5K,
        QuantType::Q6K => GgmlDType::Q6K,
        other => return Err(Error::Msg(format!("qmatmul (B200): {other:?} has no kernel in this provider")).bt()),
    })
}

/// `(OpKind::QMatMul, [F32, U32, F32], BackendId::Cuda)`. Inputs: activations (F32), weight blocks (U32- or
/// U8-typed byte buffer). Output: pre-allocated by the executor; the workspace comes from the device's
/// stream-ordered pool. Everything is enqueued on the device's stream; nothing synchronizes.
pub fn qmatmul_f32_b200(
    inputs: &[Arc<RwLock<Storage>>],
    outputs: &mut [Arc<RwLock<Storage>>],
    _layouts: &[Layout],
    params: &OpParams,
) -> Result<()> {
    if inputs.len() != 2 || outputs.len() != 1 {
        return Err(Error::Msg(format!("qmatmul wrapper expects 2 inputs and 1 output, got {} and {}", inputs.len(), outputs.len())).bt());
    }
    let (quant_type, batch_count, m, n, k) = match params {
        OpParams::QMatMul { quant_type, batch_count, m, n, k } => (*quant_type, *batch_count, *m, *n, *k),
        other => return Err(Error::Msg(format!("qmatmul wrapper expects OpParams::QMatMul, got {other:?}")).bt()),
    };
    let t = ggml_of(quant_type)?.to_u32() as i32;
    let act = inputs[0].read().map_err(|_| Error::Msg("qmatmul: poisoned activation lock".into()).bt())?;
    let w = inputs[1].read().map_err(|_| Error::Msg("qmatmul: poisoned weight lock".into()).bt())?;
    if w.dtype != DType::U32 && w.dtype != DType::U8 {
        return Err(Error::Msg(format!("qmatmul: weight bytes must be U32- or U8-typed, got {:?}", w.dtype)).bt());
    }
    let mut out = outputs[0].write().map_err(|_| Error::Msg("qmatmul: poisoned output lock".into()).bt())?;
    let (dev, act_ptr) = fuel_dispatch::cuda::device_ptr(&act)?;
    let (_, w_ptr) = fuel_dispatch::cuda::device_ptr(&w)?;
    let (_, out_ptr) = fuel_dispatch::cuda::device_ptr_mut(&mut out)?;
    let m_total = (batch_count * m) as i64;
    let ws_bytes = unsafe { fuelq_sys::fuelq_qmatmul_workspace_bytes(t, m_total, n as i64, k as i64) };
    let ws = unsafe { dev.alloc::<u8>(ws_bytes.max(16))? };
    let st = unsafe {
        fuelq_sys::fuelq_qmatmul(t, m_total, n as i64, k as i64, w_ptr as *const c_void, act_ptr as *const f32,
                                 out_ptr as *mut f32, ws.as_raw().0 as *mut c_void, ws_bytes,
                                 dev.stream().as_raw() as *mut c_void)
    };
    check(st, "fuelq_qmatmul")
}
