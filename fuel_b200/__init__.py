"""fuel_b200 — sm_100a kernels for fuel's GGUF k-quant matrix multiply, behind a C ABI.

The product is libfuelq.so (fuel_b200/csrc, include/fuelq.h). This package is the
thin Python binding used by the tests, the benchmark and multi-GPU orchestration.
"""
from .ggml import GgmlDType  # noqa: F401
