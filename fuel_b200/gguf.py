"""GGUF files: header, metadata and tensor bytes, through the library's reader (include/fuelq_gguf.h).

Mirrors the reference's `gguf_file::Content` (fuel-formats/src/gguf.rs:378-462): `GgufFile.metadata` and
`GgufFile.tensor_infos` are its two maps, `tensor_data_offset` its third field, `TensorInfo` its struct
(`ggml_dtype`, `shape` with the file's dimension list reversed, `offset`). Tensor bytes come out of the
read-only mapping either as a numpy view (host) or as a device tensor filled by one host-to-device copy of
exactly the requested rows — quantized tensors are never dequantized or repacked on the way.
"""
from __future__ import annotations

import ctypes
import dataclasses
import struct
from typing import Any

import numpy as np

from . import _lib
from .ggml import GgmlDType

_L = _lib.lib

(U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64) = range(13)
_NP = {U8: "<u1", I8: "<i1", U16: "<u2", I16: "<i2", U32: "<u4", I32: "<i4", F32: "<f4", BOOL: "<u1", U64: "<u8", I64: "<i8",
       F64: "<f8"}


class GgufError(ValueError):
    def __init__(self, status: int):
        super().__init__(_L.fuelq_last_error().decode(errors="replace"))
        self.status = status


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    """gguf.rs:62-66, plus the byte count the loaders derive (lazy_quantized_llama.rs:255-257)."""
    ggml_dtype: GgmlDType
    shape: tuple
    offset: int
    nbytes: int
    index: int

    def elem_count(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class GgufFile:
    def __init__(self, source):
        """`source`: a path, or the bytes of a whole file."""
        h = ctypes.c_void_p()
        if isinstance(source, (bytes, bytearray, memoryview)):
            self._image = bytes(source)  # kept alive: the reader does not copy it
            st = _L.fuelq_gguf_open_memory(self._image, len(self._image), ctypes.byref(h))
        else:
            self._image = None
            st = _L.fuelq_gguf_open(str(source).encode(), ctypes.byref(h))
        if st:
            raise GgufError(st)
        self._h = h
        self.version = _L.fuelq_gguf_version(h)
        self.alignment = _L.fuelq_gguf_alignment(h)
        self.tensor_data_offset = _L.fuelq_gguf_tensor_data_offset(h)
        self.metadata: dict[str, Any] = {}
        self.metadata_types: dict[str, int] = {}
        for i in range(_L.fuelq_gguf_meta_count(h)):
            v = _lib.GgufValue()
            self._check(_L.fuelq_gguf_meta_at(h, i, ctypes.byref(v)))
            key = v.key.decode(errors="replace")
            self.metadata[key] = self._value(i, v)
            self.metadata_types[key] = v.type
        self.tensor_infos: dict[str, TensorInfo] = {}
        for i in range(_L.fuelq_gguf_tensor_count(h)):
            t = _lib.GgufTensor()
            st = _L.fuelq_gguf_tensor_at(h, i, ctypes.byref(t))  # status 2 = the bytes lie outside the file; still listed
            if st and not t.name:
                raise GgufError(st)
            self.tensor_infos[t.name.decode(errors="replace")] = TensorInfo(
                GgmlDType.from_u32(t.ggml_type), tuple(t.dims[d] for d in range(t.n_dims)), t.offset, t.nbytes, i)

    # ---- lifetime
    def close(self) -> None:
        if getattr(self, "_h", None):
            _L.fuelq_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        self.close()

    def _check(self, st: int) -> None:
        if st:
            raise GgufError(st)

    def _value(self, index: int, v) -> Any:
        t = v.type
        if t in (F32, F64):
            return v.f
        if t == BOOL:
            return bool(v.i)
        if t == U64:
            return v.i & 0xFFFFFFFFFFFFFFFF
        if t == STRING:
            return ctypes.string_at(v.s, v.len).decode(errors="replace") if v.len else ""
        if t == ARRAY:
            if v.elem_type == STRING:
                out = []
                s, n = ctypes.c_void_p(), ctypes.c_uint64()
                for j in range(v.len):
                    self._check(_L.fuelq_gguf_meta_array_string(self._h, index, j, ctypes.byref(s), ctypes.byref(n)))
                    out.append(ctypes.string_at(s.value, n.value).decode(errors="replace") if n.value else "")
                return out
            if v.elem_type in _NP:
                dt = np.dtype(_NP[v.elem_type])
                raw = ctypes.string_at(v.array, v.len * dt.itemsize) if v.len else b""
                arr = np.frombuffer(raw, dtype=dt)
                return arr.astype(bool) if v.elem_type == BOOL else arr
            return None  # array of arrays: extent walked, contents not exposed
        return v.i

    # ---- tensors
    def tensor_info(self, name: str) -> TensorInfo:
        try:
            return self.tensor_infos[name]
        except KeyError:
            raise KeyError(f"gguf: missing tensor {name!r}") from None

    def tensor_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes, copied out of the mapping."""
        info = self.tensor_info(name)
        t = _lib.GgufTensor()
        self._check(_L.fuelq_gguf_tensor_at(self._h, info.index, ctypes.byref(t)))
        return np.frombuffer(ctypes.string_at(t.data, t.nbytes), dtype=np.uint8)

    def row_bytes(self, name: str) -> int:
        """Bytes of one row along the innermost dimension (whole blocks)."""
        info = self.tensor_info(name)
        k = info.shape[-1]
        if k % info.ggml_dtype.block_size():
            raise ValueError(f"gguf: tensor {name!r}: inner dimension {k} is not a whole number of blocks")
        return k // info.ggml_dtype.block_size() * info.ggml_dtype.type_size()

    def load(self, name: str, device, row_lo: int = 0, row_hi: int | None = None):
        """Rows [row_lo, row_hi) of a tensor (rows = all outer dimensions flattened) as a uint8 device tensor holding
        the file's bytes unchanged. One host-to-device copy straight from the mapping; returns after it completed."""
        import torch
        info = self.tensor_info(name)
        rb = self.row_bytes(name)
        rows = info.nbytes // rb if rb else 0
        row_hi = rows if row_hi is None else row_hi
        if not 0 <= row_lo <= row_hi <= rows:
            raise ValueError(f"gguf: rows [{row_lo}, {row_hi}) outside tensor {name!r} with {rows} rows")
        out = torch.empty((row_hi - row_lo) * rb, dtype=torch.uint8, device=device)
        with torch.cuda.device(out.device):
            st = torch.cuda.current_stream().cuda_stream
            self._check(_L.fuelq_gguf_load_tensor(self._h, info.index, row_lo * rb, (row_hi - row_lo) * rb, out.data_ptr(), st))
            torch.cuda.current_stream().synchronize()
        return out

    def load_f32(self, name: str, device):
        """The tensor as f32 on the device, shaped like the file says: f32 / f16 / bf16 converted, block formats
        through the library's dequantizer (the reference's `dequant_bytes_to_f32`, lazy_quantized_llama.rs:262-265)."""
        import torch
        from . import ops
        info = self.tensor_info(name)
        raw = self.load(name, device)
        dt = info.ggml_dtype
        if dt == GgmlDType.F32:
            out = raw.view(torch.float32)
        elif dt == GgmlDType.F16:
            out = raw.view(torch.float16).float()
        elif dt == GgmlDType.BF16:
            out = raw.view(torch.bfloat16).float()
        else:
            out = ops.dequantize(dt, raw, info.elem_count())
        return out.reshape(info.shape)


# ---- a writer, for producing files from tensors already in block form (tests, tools)
def _w_str(s: str, version: int) -> bytes:
    b = s.encode()
    return struct.pack("<I" if version == 1 else "<Q", len(b)) + b


_PACK = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _w_value(vtype: int, value, version: int) -> bytes:
    if vtype == STRING:
        return _w_str(value, version)
    if vtype == ARRAY:
        etype, items = value
        out = struct.pack("<I", etype) + struct.pack("<I" if version == 1 else "<Q", len(items))
        return out + b"".join(_w_value(etype, it, version) for it in items)
    return struct.pack(_PACK[vtype], value)


def write_gguf(path, metadata: list, tensors: list, version: int = 3, alignment: int | None = None) -> None:
    """Write a GGUF file. metadata: [(key, value_type, value)], an ARRAY value being (elem_type, [items]);
    tensors: [(name, GgmlDType, shape outermost-first, bytes-like)]. Layout as the reference reads it
    (gguf.rs:385-462): dimension lists are stored innermost-first, each tensor's data starts on a multiple of the
    alignment (`general.alignment` is added to the metadata when `alignment` is given, else 32 applies)."""
    assert version in (1, 2, 3)
    cnt = "<I" if version == 1 else "<Q"
    metadata = list(metadata)
    if alignment is not None:
        metadata.append(("general.alignment", U32, alignment))
    al = alignment or 32
    head = struct.pack("<II", 0x46554747, version) + struct.pack(cnt, len(tensors)) + struct.pack(cnt, len(metadata))
    for key, vtype, value in metadata:
        head += _w_str(key, version) + struct.pack("<I", vtype) + _w_value(vtype, value, version)
    offset, blobs = 0, []
    for name, dt, shape, data in tensors:
        data = bytes(data)
        head += _w_str(name, version) + struct.pack("<I", len(shape))
        for d in reversed(shape):
            head += struct.pack("<I" if version == 1 else "<Q", d)
        head += struct.pack("<IQ", int(dt), offset)
        blobs.append((offset, data))
        offset = (offset + len(data) + al - 1) // al * al
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((len(head) + al - 1) // al * al - len(head)))
        base = f.tell()
        for off, data in blobs:
            f.write(b"\0" * (base + off - f.tell()))
            f.write(data)
