"""QTensor / QMatMul — the reference's quantized-tensor facade, bound to the native host layer.

Mirrors the eager API the reference's models were written against (`QTensor::quantize`,
`QTensor::dequantize`, `QMatMul::from_qtensor`, `Module::forward`; what survives of it in
the reference is `DynQuantizedStorage`, fuel-backend-contract/src/quantized.rs:29-103).
Each object wraps a handle to fuel_b200/csrc/host.hpp's C++ types through the C entry points
of include/fuelq_host.h; torch only supplies device tensors for inputs and outputs.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .ggml import GgmlDType

_L = _lib.lib
_OUT_TYPES = {torch.float32: GgmlDType.F32, torch.float16: GgmlDType.F16, torch.bfloat16: GgmlDType.BF16}


def _check(status: int, op: str) -> None:
    if status != _lib.OK:
        raise _lib.FuelqError(op, status, _L.fuelq_last_error().decode() or _lib.status_string(status))


class QTensor:
    """A [n, k] weight held on the device as GGUF blocks."""

    def __init__(self, handle: int, device: torch.device):
        self._h = ctypes.c_void_p(handle)
        self.device = device
        t, n, k, nbytes, ptr = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_size_t(), ctypes.c_void_p()
        _check(_L.fuelq_qtensor_info(self._h, ctypes.byref(t), ctypes.byref(n), ctypes.byref(k), ctypes.byref(nbytes),
                                     ctypes.byref(ptr)), "qtensor_info")
        self._dtype = GgmlDType(t.value)
        self._shape = (n.value, k.value)
        self._nbytes = nbytes.value
        self._ptr = ptr.value or 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            _L.fuelq_qtensor_free(h)

    # ---- constructors
    @classmethod
    def quantize(cls, src, dtype: GgmlDType, device: torch.device | str = "cuda") -> "QTensor":
        """f32 [n, k] (torch CUDA tensor, torch CPU tensor or numpy array) -> blocks."""
        device = torch.device(device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if isinstance(src, torch.Tensor) and src.is_cuda:
            if src.dtype != torch.float32:
                raise ValueError("only f32 can be quantized")
            src = src.contiguous()
            n, k = src.reshape(-1, src.shape[-1]).shape
            ptr, on_dev = src.data_ptr(), 1
        else:
            src = np.ascontiguousarray(src.numpy() if isinstance(src, torch.Tensor) else src, dtype=np.float32)
            n, k = src.reshape(-1, src.shape[-1]).shape
            ptr, on_dev = src.ctypes.data, 0
        out = ctypes.c_void_p()
        with torch.cuda.device(idx):
            stream = torch.cuda.current_stream().cuda_stream
            _check(_L.fuelq_qtensor_quantize(idx, stream, int(dtype), n, k, ptr, on_dev, ctypes.byref(out)), "QTensor.quantize")
            torch.cuda.current_stream().synchronize()
        return cls(out.value, torch.device("cuda", idx))

    @classmethod
    def from_blocks(cls, blocks, dtype: GgmlDType, shape, device: torch.device | str = "cuda") -> "QTensor":
        """Pre-quantized GGUF bytes (numpy uint8) -> device weight (QuantizedDeviceKernels::load_quantized)."""
        device = torch.device(device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        n, k = shape
        out = ctypes.c_void_p()
        with torch.cuda.device(idx):
            stream = torch.cuda.current_stream().cuda_stream
            _check(_L.fuelq_qtensor_load(idx, stream, int(dtype), n, k, blocks.ctypes.data, blocks.size, ctypes.byref(out)),
                   "QTensor.from_blocks")
        return cls(out.value, torch.device("cuda", idx))

    # ---- accessors (DynQuantizedStorage)
    def dtype(self) -> GgmlDType:
        return self._dtype

    def shape(self):
        return self._shape

    def rank(self) -> int:
        return 2

    def block_size(self) -> int:
        return self._dtype.block_size()

    def storage_size_in_bytes(self) -> int:
        return self._nbytes

    def device_ptr(self) -> int:
        return self._ptr

    def data(self) -> np.ndarray:
        out = np.empty(self._nbytes, dtype=np.uint8)
        _check(_L.fuelq_qtensor_data(self._h, out.ctypes.data, out.size), "QTensor.data")
        return out

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.empty(self._shape, dtype=dtype, device=self.device)
        with torch.cuda.device(self.device):
            _check(_L.fuelq_qtensor_dequantize(self._h, out.data_ptr(), int(_OUT_TYPES[dtype])), "QTensor.dequantize")
        return out

    def dequantize_f16(self) -> torch.Tensor:
        return self.dequantize(torch.float16)


class QMatMul:
    """Module: forward(xs) = xs . W^T (QMatMul::forward == DynQuantizedStorage::fwd)."""

    def __init__(self, w: QTensor):
        self.w = w

    @classmethod
    def from_qtensor(cls, w: QTensor) -> "QMatMul":
        return cls(w)

    def forward(self, xs):
        n, k = self.w.shape()
        if isinstance(xs, np.ndarray) or (isinstance(xs, torch.Tensor) and not xs.is_cuda):
            x = np.ascontiguousarray(xs.numpy() if isinstance(xs, torch.Tensor) else xs, dtype=np.float32)
            if x.ndim < 2:
                raise _lib.FuelqError("QMatMul.forward", _lib.INVALID_PROBLEM, "input tensor has only one dimension")
            if x.shape[-1] != k:
                raise _lib.FuelqError("QMatMul.forward", _lib.INVALID_PROBLEM, "input tensor incompatible with the weight shape")
            y = np.empty((*x.shape[:-1], n), dtype=np.float32)
            with torch.cuda.device(self.w.device):
                _check(_L.fuelq_qmatmul_forward_host(self.w._h, x.ctypes.data, x.size // k, y.ctypes.data), "QMatMul.forward")
            return torch.from_numpy(y) if isinstance(xs, torch.Tensor) else y
        if xs.dtype != torch.float32:
            raise _lib.FuelqError("QMatMul.forward", _lib.NOT_SUPPORTED, "Expected f32")
        if not xs.is_contiguous():
            raise _lib.FuelqError("QMatMul.forward", _lib.INVALID_PROBLEM, "input tensor is not contiguous")
        if xs.dim() < 2:
            raise _lib.FuelqError("QMatMul.forward", _lib.INVALID_PROBLEM, "input tensor has only one dimension")
        if xs.shape[-1] != k:
            raise _lib.FuelqError("QMatMul.forward", _lib.INVALID_PROBLEM, "input tensor incompatible with the weight shape")
        y = torch.empty(*xs.shape[:-1], n, dtype=torch.float32, device=xs.device)
        with torch.cuda.device(xs.device):
            _check(_L.fuelq_qmatmul_forward(self.w._h, xs.data_ptr(), xs.numel() // k, y.data_ptr()), "QMatMul.forward")
        return y

    __call__ = forward
