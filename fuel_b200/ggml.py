"""GGUF block-format tags — mirrors fuel-ir/src/quantized.rs:16-104 (GgmlDType)."""
from __future__ import annotations

import enum


class GgmlDType(enum.IntEnum):
    """Values are the GGUF on-disk ids (GgmlDType::to_u32)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 8
    Q4K = 12
    Q6K = 14
    Q8K = 15
    BF16 = 30

    @classmethod
    def from_u32(cls, u: int) -> "GgmlDType":
        try:
            return cls(u)
        except ValueError:
            raise ValueError(f"unknown dtype for tensor {u}") from None

    def to_u32(self) -> int:
        return int(self)

    def type_size(self) -> int:
        return _TYPE_SIZE[self]

    def block_size(self) -> int:
        return _BLOCK_SIZE[self]


_TYPE_SIZE = {GgmlDType.F32: 4, GgmlDType.F16: 2, GgmlDType.BF16: 2, GgmlDType.Q4_0: 18, GgmlDType.Q8_0: 34,
              GgmlDType.Q4K: 144, GgmlDType.Q6K: 210, GgmlDType.Q8K: 292}
_BLOCK_SIZE = {GgmlDType.F32: 1, GgmlDType.F16: 1, GgmlDType.BF16: 1, GgmlDType.Q4_0: 32, GgmlDType.Q8_0: 32,
               GgmlDType.Q4K: 256, GgmlDType.Q6K: 256, GgmlDType.Q8K: 256}
