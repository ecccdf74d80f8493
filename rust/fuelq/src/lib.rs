//! fuel's quantized-kernel provider for B200, over `libfuelq.so`.
//!
//! What fuel's backend contract asks of a provider, and where it is here:
//!  * storage: [`QB200Storage`] implements `DynQuantizedStorage`
//!    (`fuel-backend-contract/src/quantized.rs:29-103`) — the type `QCudaStorage` is today
//!    (`fuel-cuda-backend/src/quantized.rs:306-697`), with `fwd`, `dequantize*` and `quantize` enqueued
//!    on the device stream through the C ABI instead of staged through the host;
//!  * constructors: [`B200Device`] implements `QuantizedDeviceKernels` (`quantized.rs:108-120`);
//!  * lazy graph: [`fkc::ENTRY_POINTS`] maps the `entry_point` strings of `contracts/qmatmul.fkc.md` to
//!    `KernelRef`s for `(OpKind::QMatMul, [F32, U32, F32], BackendId::Cuda)`;
//!  * handshake: [`seam::negotiate_with_provider`];
//!  * the eager façade the reference removed: [`QTensor`], [`QMatMul`], `impl Module for QMatMul`.
//!
//! Not compiled where this repository is built (no Rust toolchain there); `fuel_b200/csrc/host.hpp` is
//! the same logic in C++, compiled and tested.

pub mod fkc;
pub mod seam;

use std::any::Any;
use std::borrow::Cow;
use std::ffi::c_void;
use std::sync::Arc;

use fuel_backend_contract::dyn_backend::{DynBackendDevice, DynBackendStorage};
use fuel_backend_contract::quantized::{DynQuantizedStorage, QuantizedDeviceKernels};
use fuel_cuda_backend::{CudaDevice, CudaStorage, CudaStorageSlice};
use fuel_ir::{bail, Error, GgmlDType, Layout, Result, Shape};
use fuelq_sys as sys;

/// Maps a libfuelq status to fuel's error type; the codes are the ones
/// `fuel-cuda-backend/src/baracuda/status.rs:22-48` names.
pub(crate) fn check(status: i32, op: &'static str) -> Result<()> {
    if status == sys::FUELQ_OK {
        return Ok(());
    }
    let reason = unsafe { std::ffi::CStr::from_ptr(sys::fuelq_status_string(status)) }.to_string_lossy();
    Err(Error::Msg(format!("{op}: status {status} ({reason})")).bt())
}

fn ggml(t: GgmlDType) -> i32 {
    t.to_u32() as i32
}

/// Quantized weight blocks on one B200, exactly the GGUF bytes, plus the device they live on.
#[derive(Debug)]
pub struct QB200Storage {
    data: fuel_cuda_backend::CudaSlice<u8>,
    len: usize,
    dtype: GgmlDType,
    device: CudaDevice,
}

impl QB200Storage {
    pub fn zeros(device: &CudaDevice, elem_count: usize, dtype: GgmlDType) -> Result<Self> {
        if elem_count % dtype.block_size() != 0 {
            bail!("qzeros: {elem_count} elements is not a whole number of {dtype:?} blocks")
        }
        let len = elem_count / dtype.block_size() * dtype.type_size();
        Ok(Self { data: device.alloc_zeros::<u8>(len.max(16))?, len, dtype, device: device.clone() })
    }

    /// `QuantizedDeviceKernels::load_quantized`: GGUF bytes from the host, unchanged
    /// (`fuel-cuda-backend/src/quantized.rs:593-609` without the row padding, which these kernels do not need).
    pub fn from_host_blocks(device: &CudaDevice, dtype: GgmlDType, bytes: &[u8]) -> Result<Self> {
        if bytes.len() % dtype.type_size() != 0 {
            bail!("load_quantized: {} bytes is not a whole number of {dtype:?} blocks", bytes.len())
        }
        let mut data = unsafe { device.alloc::<u8>(bytes.len().max(16))? };
        device.memcpy_htod(bytes, &mut data.slice_mut(0..bytes.len()))?;
        Ok(Self { data, len: bytes.len(), dtype, device: device.clone() })
    }

    fn raw(&self) -> *const c_void {
        self.data.as_raw().0 as *const c_void
    }

    fn stream(&self) -> *mut c_void {
        self.device.stream().as_raw() as *mut c_void
    }

    /// f32 on the device -> blocks, on the device (byte-identical to `from_float` on the host, which is what
    /// `QCudaStorage::quantize` runs after copying the tensor down, `quantized.rs:414-420`).
    fn quantize_device(&mut self, src: &CudaStorage) -> Result<()> {
        let x = match &src.slice {
            CudaStorageSlice::F32(d) => d,
            _ => bail!("only f32 can be quantized"),
        };
        let numel = x.len();
        if numel / self.dtype.block_size() * self.dtype.type_size() != self.len {
            bail!("quantize: {numel} elements do not fill a {:?} storage of {} bytes", self.dtype, self.len)
        }
        let st = unsafe {
            sys::fuelq_quantize_weights(ggml(self.dtype), numel as i64, x.as_raw().0 as *const f32,
                                        self.data.as_raw().0 as *mut c_void, self.stream())
        };
        check(st, "fuelq_quantize_weights")
    }

    fn dequantize_to(&self, elem_count: usize, out_type: i32) -> Result<CudaStorage> {
        if elem_count / self.dtype.block_size() * self.dtype.type_size() != self.len {
            bail!("dequantize: {elem_count} elements do not match a storage of {} bytes", self.len)
        }
        let (dst, ptr) = self.device.alloc_storage(elem_count, if out_type == 0 { fuel_ir::DType::F32 } else { fuel_ir::DType::F16 })?;
        let st = unsafe { sys::fuelq_dequantize(ggml(self.dtype), elem_count as i64, self.raw(), ptr, out_type, self.stream()) };
        check(st, "fuelq_dequantize")?;
        Ok(dst)
    }

    /// `QMatMul::forward`: `[.., k] -> [.., n]` (`fuel-cuda-backend/src/quantized.rs:452-473`).
    pub fn fwd_cuda(&self, self_shape: &Shape, input: &CudaStorage, layout: &Layout) -> Result<(CudaStorage, Shape)> {
        let (n, k) = self_shape.dims2()?;
        let dims = layout.shape().dims();
        if dims.len() < 2 || *dims.last().unwrap() != k {
            bail!("input tensor {layout:?} incompatible with {self_shape:?}")
        }
        let x = match &input.slice {
            CudaStorageSlice::F32(d) => d,
            _ => bail!("quantized-matmul: activations must be f32"),
        };
        let (o1, o2) = layout.contiguous_offsets().ok_or(Error::RequiresContiguous { op: "quantized-matmul" })?;
        let m = (o2 - o1) / k;
        let t = ggml(self.dtype);
        let ws_bytes = unsafe { sys::fuelq_qmatmul_workspace_bytes(t, m as i64, n as i64, k as i64) };
        // both allocations are stream-ordered pool allocations: no host synchronization anywhere in the call
        let ws = unsafe { self.device.alloc::<u8>(ws_bytes.max(16))? };
        let dst = unsafe { self.device.alloc::<f32>(m * n)? };
        let st = unsafe {
            sys::fuelq_qmatmul(t, m as i64, n as i64, k as i64, self.raw(),
                               (x.as_raw().0 as *const f32).add(o1), dst.as_raw().0 as *mut f32,
                               ws.as_raw().0 as *mut c_void, ws_bytes, self.stream())
        };
        check(st, "fuelq_qmatmul")?;
        let mut out_shape = dims.to_vec();
        out_shape.pop();
        out_shape.push(n);
        Ok((CudaStorage::wrap_cuda_slice(dst, self.device.clone()), out_shape.into()))
    }
}

impl DynQuantizedStorage for QB200Storage {
    fn dtype(&self) -> GgmlDType {
        self.dtype
    }
    fn block_size(&self) -> usize {
        self.dtype.block_size()
    }
    fn storage_size_in_bytes(&self) -> usize {
        self.len
    }
    fn quantize(&mut self, src: &dyn DynBackendStorage) -> Result<()> {
        let cuda = src.as_any().downcast_ref::<CudaStorage>()
            .ok_or_else(|| Error::Msg("quantize: expected cuda storage".into()).bt())?;
        self.quantize_device(cuda)
    }
    fn quantize_imatrix(&mut self, _src: &dyn DynBackendStorage, _w: &[f32], _n_per_row: usize) -> Result<()> {
        // importance-matrix quantizers are not on the device; status 3 in the C ABI
        Err(Error::Msg("quantize_imatrix: not supported by the B200 provider".into()).bt())
    }
    fn quantize_onto(&mut self, src: &dyn DynBackendStorage) -> Result<()> {
        let cpu = src.as_any().downcast_ref::<fuel_cpu_backend::CpuStorage>()
            .ok_or_else(|| Error::Msg("quantize_onto: expected cpu storage".into()).bt())?;
        let staged = self.device.storage_from_cpu_storage(&cpu.0)?;
        self.quantize_device(&staged)
    }
    fn quantize_imatrix_onto(&mut self, _src: &dyn DynBackendStorage, _w: &[f32], _n_per_row: usize) -> Result<()> {
        Err(Error::Msg("quantize_imatrix_onto: not supported by the B200 provider".into()).bt())
    }
    fn dequantize(&self, elem_count: usize) -> Result<Box<dyn DynBackendStorage>> {
        Ok(Box::new(self.dequantize_to(elem_count, 0)?))
    }
    fn dequantize_f16(&self, elem_count: usize) -> Result<Box<dyn DynBackendStorage>> {
        Ok(Box::new(self.dequantize_to(elem_count, 1)?))
    }
    fn data(&self) -> Result<Cow<'_, [u8]>> {
        // the original block bytes, as the reference returns them (quantized.rs:475-480)
        Ok(Cow::Owned(self.device.clone_dtoh(&self.data.slice(0..self.len))?))
    }
    fn device_ptr(&self) -> Result<*const u8> {
        Ok(self.raw() as *const u8)
    }
    fn fwd(&self, self_shape: &Shape, input: &dyn DynBackendStorage, layout: &Layout)
        -> Result<(Box<dyn DynBackendStorage>, Shape)> {
        let cuda = input.as_any().downcast_ref::<CudaStorage>()
            .ok_or_else(|| Error::Msg("qmatmul: expected cuda storage".into()).bt())?;
        let (s, sh) = self.fwd_cuda(self_shape, cuda, layout)?;
        Ok((Box::new(s), sh))
    }
    fn as_any(&self) -> &dyn Any {
        self
    }
    fn device_arc_dyn(&self) -> Arc<dyn DynBackendDevice> {
        Arc::new(self.device.clone())
    }
}

/// The device handle through which fuel-core asks for quantized storage.
#[derive(Clone, Debug)]
pub struct B200Device(pub CudaDevice);

impl std::ops::Deref for B200Device {
    type Target = CudaDevice;
    fn deref(&self) -> &CudaDevice {
        &self.0
    }
}

impl B200Device {
    pub fn qzeros(&self, elem_count: usize, dtype: GgmlDType) -> Result<Box<dyn DynQuantizedStorage>> {
        Ok(Box::new(QB200Storage::zeros(&self.0, elem_count, dtype)?))
    }
    pub fn load_quantized(&self, dtype: GgmlDType, data: Cow<'_, [u8]>) -> Result<Box<dyn DynQuantizedStorage>> {
        Ok(Box::new(QB200Storage::from_host_blocks(&self.0, dtype, &data)?))
    }
}
// `impl QuantizedDeviceKernels for B200Device` forwards to the two methods above; it needs
// `B200Device: DynBackendDevice`, which is the same forwarding over `CudaDevice`'s own impl.

// ---------------------------------------------------------------- the eager façade
/// A quantized weight tensor: storage + its `[n, k]` shape (the type fuel-core removed,
/// `fuel-core/src/quantized/mod.rs:14-24`).
#[derive(Debug)]
pub struct QTensor {
    storage: Box<dyn DynQuantizedStorage>,
    shape: Shape,
}

impl QTensor {
    pub fn new(storage: Box<dyn DynQuantizedStorage>, shape: impl Into<Shape>) -> Result<Self> {
        let shape = shape.into();
        let (n, k) = shape.dims2()?;
        if k % storage.block_size() != 0
            || n * (k / storage.block_size()) * storage.dtype().type_size() != storage.storage_size_in_bytes()
        {
            bail!("QTensor: shape {shape:?} does not match {} bytes of {:?}", storage.storage_size_in_bytes(), storage.dtype())
        }
        Ok(Self { storage, shape })
    }
    pub fn dtype(&self) -> GgmlDType {
        self.storage.dtype()
    }
    pub fn shape(&self) -> &Shape {
        &self.shape
    }
    pub fn storage(&self) -> &dyn DynQuantizedStorage {
        self.storage.as_ref()
    }
}

/// `xs @ W^T` for a quantized `W` (`QMatMul::forward` is `DynQuantizedStorage::fwd`,
/// `fuel-backend-contract/src/quantized.rs:72-80`).
#[derive(Debug)]
pub struct QMatMul {
    weight: Arc<QTensor>,
}

impl QMatMul {
    pub fn from_qtensor(weight: QTensor) -> Self {
        Self { weight: Arc::new(weight) }
    }
    pub fn from_arc(weight: Arc<QTensor>) -> Self {
        Self { weight }
    }
    /// Storage-level forward: returns the output storage and its shape.
    pub fn forward_storage(&self, input: &dyn DynBackendStorage, layout: &Layout)
        -> Result<(Box<dyn DynBackendStorage>, Shape)> {
        self.weight.storage.fwd(&self.weight.shape, input, layout)
    }
}

/// fuel's layer trait: one tensor in, one tensor out.
pub trait Module {
    type Tensor;
    fn forward(&self, xs: &Self::Tensor) -> Result<Self::Tensor>;
}

/// A device tensor as the eager API sees it: storage, layout.
pub struct EagerTensor {
    pub storage: Box<dyn DynBackendStorage>,
    pub layout: Layout,
}

impl Module for QMatMul {
    type Tensor = EagerTensor;
    fn forward(&self, xs: &EagerTensor) -> Result<EagerTensor> {
        let (storage, shape) = self.forward_storage(xs.storage.as_ref(), &xs.layout)?;
        Ok(EagerTensor { storage, layout: Layout::contiguous(shape) })
    }
}
