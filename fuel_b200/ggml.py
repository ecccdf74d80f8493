"""GGUF block-format tags — mirrors fuel-ir/src/quantized.rs:16-104 (GgmlDType)."""
from __future__ import annotations

import enum


class GgmlDType(enum.IntEnum):
    """Values are the GGUF on-disk ids (GgmlDType::to_u32)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2K = 10
    Q3K = 11
    Q4K = 12
    Q5K = 13
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


_G = GgmlDType
_TYPE_SIZE = {_G.F32: 4, _G.F16: 2, _G.BF16: 2, _G.Q4_0: 18, _G.Q4_1: 20, _G.Q5_0: 22, _G.Q5_1: 24, _G.Q8_0: 34, _G.Q8_1: 36,
              _G.Q2K: 84, _G.Q3K: 110, _G.Q4K: 144, _G.Q5K: 176, _G.Q6K: 210, _G.Q8K: 292}
_BLOCK_SIZE = {t: (1 if t in (_G.F32, _G.F16, _G.BF16) else 256 if t.name.endswith("K") else 32) for t in _G}
