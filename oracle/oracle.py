"""TEST INFRASTRUCTURE — ctypes front for the CPU restatement in this folder.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this
module; nothing in the shipped package does. The arithmetic lives in the C++
files beside it (each function cites the reference lines it follows); this file
only moves numpy arrays across the boundary.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfuelq_oracle.so")

Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2K, Q3K, Q4K, Q5K, Q6K, Q8K = 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15  # GGUF ids, fuel-ir/src/quantized.rs:35-75
SCALAR, AVX2 = 0, 1

_lib = None


def build(force: bool = False) -> str:
    """Compile the restatement if the shared object is missing or stale."""
    srcs = [os.path.join(_HERE, f) for f in
            ("kquants_scalar.cpp", "kquants_avx2.cpp", "oracle_api.cpp", "blocks.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libfuelq_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, ci, vp, fp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)
        L.fq_oracle_block_elems.argtypes = [ci]
        L.fq_oracle_block_bytes.argtypes = [ci]
        L.fq_oracle_act_type.argtypes = [ci]
        L.fq_oracle_f32_to_f16.argtypes = [ctypes.c_float]
        L.fq_oracle_f32_to_f16.restype = ctypes.c_uint16
        L.fq_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.fq_oracle_f16_to_f32.restype = ctypes.c_float
        L.fq_oracle_quantize.argtypes = [ci, fp, i64, vp, ci]
        L.fq_oracle_dequantize.argtypes = [ci, vp, i64, fp, ci]
        L.fq_oracle_quantize_act.argtypes = [ci, fp, i64, i64, vp]
        L.fq_oracle_vec_dot.argtypes = [ci, ci, i64, vp, vp]
        L.fq_oracle_vec_dot.restype = ctypes.c_float
        L.fq_oracle_matmul.argtypes = [ci, ci, i64, i64, i64, fp, vp, fp, ci]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def block_elems(t: int) -> int:
    return lib().fq_oracle_block_elems(t)


def block_bytes(t: int) -> int:
    return lib().fq_oracle_block_bytes(t)


def act_type(t: int) -> int:
    return lib().fq_oracle_act_type(t)


def quantize(t: int, x, nthreads: int = 0) -> np.ndarray:
    """from_float over a flat f32 array -> uint8 block stream."""
    x = _f32(x).reshape(-1)
    be, bb = block_elems(t), block_bytes(t)
    assert be and x.size % be == 0, (t, x.size)
    out = np.zeros(x.size // be * bb, dtype=np.uint8)
    rc = lib().fq_oracle_quantize(t, _fp(x), x.size, out.ctypes.data, nthreads)
    assert rc == 0, rc
    return out


def dequantize(t: int, blocks: np.ndarray, nthreads: int = 0) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
    be, bb = block_elems(t), block_bytes(t)
    assert blocks.size % bb == 0
    n = blocks.size // bb * be
    out = np.empty(n, dtype=np.float32)
    rc = lib().fq_oracle_dequantize(t, blocks.ctypes.data, n, _fp(out), nthreads)
    assert rc == 0, rc
    return out


def quantize_act(weight_type: int, x) -> np.ndarray:
    """Rows of x [m, k] -> the dot-product partner blocks of `weight_type`."""
    x = _f32(x)
    m, k = x.reshape(-1, x.shape[-1]).shape
    at = act_type(weight_type)
    out = np.zeros(m * (k // block_elems(at)) * block_bytes(at), dtype=np.uint8)
    rc = lib().fq_oracle_quantize_act(weight_type, _fp(x), m, k, out.ctypes.data)
    assert rc == 0, rc
    return out


def vec_dot(t: int, order: int, k: int, w_blocks: np.ndarray, act_blocks: np.ndarray) -> float:
    return float(lib().fq_oracle_vec_dot(t, order, k, w_blocks.ctypes.data, act_blocks.ctypes.data))


def matmul(t: int, x, w_blocks: np.ndarray, n: int, order: int = SCALAR, nthreads: int = 0) -> np.ndarray:
    """y[m, n] = x[m, k] . W[n, k]^T through activation re-quantization, as the reference's matmul."""
    x = _f32(x)
    lead = x.shape[:-1]
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    m = x2.shape[0]
    w_blocks = np.ascontiguousarray(w_blocks, dtype=np.uint8).reshape(-1)
    assert w_blocks.size == n * (k // block_elems(t)) * block_bytes(t), (w_blocks.size, n, k)
    out = np.zeros((m, n), dtype=np.float32)
    rc = lib().fq_oracle_matmul(t, order, m, k, n, _fp(x2), w_blocks.ctypes.data, _fp(out), nthreads)
    assert rc == 0, rc
    return out.reshape(*lead, n)


def matmul_dequant_f64(t: int, x, w_blocks: np.ndarray, n: int) -> np.ndarray:
    """Float ground truth for the tensor-core path: exact dequantized weights, f64 accumulation."""
    x = _f32(x)
    k = x.shape[-1]
    w = dequantize(t, w_blocks).reshape(n, k).astype(np.float64)
    return (x.reshape(-1, k).astype(np.float64) @ w.T).reshape(*x.shape[:-1], n)


def max_threads() -> int:
    return lib().fq_oracle_max_threads()
