"""Kernel-level entry points on torch CUDA tensors.

torch supplies device memory and the current stream only; every operation is one
call into libfuelq.so through the C ABI of include/fuelq.h. Function names follow
the reference's quantized storage API (fuel-backend-contract/src/quantized.rs:29-103).
"""
from __future__ import annotations

import torch

from . import _lib
from .ggml import GgmlDType

_L = _lib.lib
_OUT_TYPES = {torch.float32: GgmlDType.F32, torch.float16: GgmlDType.F16, torch.bfloat16: GgmlDType.BF16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")  # fuel-cpu-backend/src/quantized.rs:96-98


def storage_bytes(dtype: GgmlDType, elem_count: int) -> int:
    bs = dtype.block_size()
    if elem_count % bs:
        raise ValueError(f"{elem_count} elements is not a multiple of the {dtype.name} block size {bs}")
    return elem_count // bs * dtype.type_size()


def quantize_act(weight_dtype: GgmlDType, x: torch.Tensor) -> torch.Tensor:
    """Rows of x [.., k] -> the reference's Q8_K / Q8_1 / Q8_0 activation blocks (uint8 stream)."""
    _need_cuda(x, "x")
    k = x.shape[-1]
    m = x.numel() // k
    act = (GgmlDType.Q8K if weight_dtype in (GgmlDType.Q2K, GgmlDType.Q3K, GgmlDType.Q4K, GgmlDType.Q5K, GgmlDType.Q6K)
           else GgmlDType.Q8_1 if weight_dtype in (GgmlDType.Q4_1, GgmlDType.Q5_1) else GgmlDType.Q8_0)
    if k % act.block_size():
        _lib.check(_lib.INVALID_PROBLEM, "quantize_act")
    out = torch.empty(storage_bytes(act, m * k), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_L.fuelq_quantize_act(int(weight_dtype), m, k, x.data_ptr(), out.data_ptr(), _stream()),
                   "fuelq_quantize_act")
    return out


def quantize_act_packed(weight_dtype: GgmlDType, x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x, "x")
    k = x.shape[-1]
    m = x.numel() // k
    nbytes = _L.fuelq_act_packed_bytes(int(weight_dtype), m, k)
    out = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_L.fuelq_quantize_act_packed(int(weight_dtype), m, k, x.data_ptr(), out.data_ptr(), nbytes,
                                                _stream()), "fuelq_quantize_act_packed")
    return out


def qmatmul(dtype: GgmlDType, w_blocks: torch.Tensor, n: int, x: torch.Tensor,
            out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """y[.., n] = x[.., k] . W[n, k]^T, W as GGUF blocks (uint8 stream of n rows)."""
    _need_cuda(x, "x")
    _need_cuda(w_blocks, "w_blocks")
    if x.dtype != torch.float32:
        raise ValueError("activations must be float32")
    k = x.shape[-1]
    m = x.numel() // k if k else 0
    if k % dtype.block_size() == 0 and w_blocks.numel() != storage_bytes(dtype, n * k):
        raise ValueError(f"weight bytes={w_blocks.numel()} doesn't match n={n} x k={k} {dtype.name}")
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=torch.float32, device=x.device)
    ws_bytes = _L.fuelq_qmatmul_workspace_bytes(int(dtype), m, n, k)
    if workspace is None:
        workspace = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_L.fuelq_qmatmul(int(dtype), m, n, k, w_blocks.data_ptr(), x.data_ptr(), out.data_ptr(),
                                    workspace.data_ptr(), workspace.numel(), _stream()), "fuelq_qmatmul")
    return out


def qmatmul_host(dtype: GgmlDType, w_blocks: torch.Tensor, n: int, x_host: torch.Tensor,
                 out_host: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """qmatmul for HOST activations and a HOST result (CPU tensors; pinned ones keep the call asynchronous and, when
    small, are read and written in place by the kernels). Enqueued on the current stream of the weights' device;
    synchronize that stream before reading the result."""
    _need_cuda(w_blocks, "w_blocks")
    if x_host.is_cuda or x_host.dtype != torch.float32 or not x_host.is_contiguous():
        raise ValueError("x_host must be a contiguous float32 CPU tensor")
    k = x_host.shape[-1]
    m = x_host.numel() // k if k else 0
    if out_host is None:
        out_host = torch.empty(*x_host.shape[:-1], n, dtype=torch.float32, pin_memory=x_host.is_pinned())
    ws_bytes = _L.fuelq_qmatmul_host_workspace_bytes(int(dtype), m, n, k)
    if workspace is None:
        workspace = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=w_blocks.device)
    with torch.cuda.device(w_blocks.device):
        _lib.check(_L.fuelq_qmatmul_host(int(dtype), m, n, k, w_blocks.data_ptr(), x_host.data_ptr(), out_host.data_ptr(),
                                         workspace.data_ptr(), workspace.numel(), _stream()), "fuelq_qmatmul_host")
    return out_host


def qmatmul_packed(dtype: GgmlDType, w_blocks: torch.Tensor, n: int, k: int, m: int, packed_act: torch.Tensor,
                   out: torch.Tensor) -> torch.Tensor:
    with torch.cuda.device(out.device):
        _lib.check(_L.fuelq_qmatmul_packed(int(dtype), m, n, k, w_blocks.data_ptr(), packed_act.data_ptr(),
                                           out.data_ptr(), _stream()), "fuelq_qmatmul_packed")
    return out


def quantize_weights(dtype: GgmlDType, w: torch.Tensor) -> torch.Tensor:
    """f32 weights (any shape, row length a multiple of the block) -> GGUF block bytes, on the device."""
    _need_cuda(w, "w")
    if w.dtype != torch.float32:
        raise ValueError("only f32 can be quantized")  # fuel-cuda-backend/src/quantized.rs:414-418
    out = torch.empty(storage_bytes(dtype, w.numel()), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        _lib.check(_L.fuelq_quantize_weights(int(dtype), w.numel(), w.data_ptr(), out.data_ptr(), _stream()),
                   "fuelq_quantize_weights")
    return out


def dequantize(dtype: GgmlDType, blocks: torch.Tensor, elem_count: int,
               out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    _need_cuda(blocks, "blocks")
    out = torch.empty(elem_count, dtype=out_dtype, device=blocks.device)
    with torch.cuda.device(blocks.device):
        _lib.check(_L.fuelq_dequantize(int(dtype), elem_count, blocks.data_ptr(), out.data_ptr(),
                                       int(_OUT_TYPES[out_dtype]), _stream()), "fuelq_dequantize")
    return out


def device_error(clear: bool = True) -> int:
    import ctypes
    code = ctypes.c_int32(0)
    _lib.check(_L.fuelq_device_error(ctypes.byref(code), 1 if clear else 0), "fuelq_device_error")
    return code.value
