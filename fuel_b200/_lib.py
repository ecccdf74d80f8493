"""ctypes binding of libfuelq.so (the C ABI declared in include/fuelq.h).

There is no fallback: if the shared library is missing or a symbol is absent the
import fails, and every call that returns a non-zero status raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfuelq.so")

OK, MISALIGNED, INVALID_PROBLEM, NOT_SUPPORTED, WORKSPACE, LAUNCH_FAILURE = range(6)
NUMERICS_INTEGER, NUMERICS_BF16, NUMERICS_TF32, NUMERICS_F16 = range(4)
OPT_PDL, OPT_DECODE_MAX_M, OPT_DECODE_GRID, OPT_DECODE_KERNEL, OPT_L2_PREFETCH, OPT_FUSED_QUANT, OPT_PEER_WAIT_MS, OPT_PREFILL_TF32, OPT_PREFILL_BF16, OPT_PREFILL_ONE_KERNEL = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10

_i32, _i64, _vp, _sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t

PEER_MAX_WORLD, PEER_MAX_SEQ = 8, 1024


class Peers(ctypes.Structure):
    """struct fuelq_peers of include/fuelq.h."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("epoch", ctypes.c_void_p)]


_pp = ctypes.POINTER(Peers)


class Rope(ctypes.Structure):
    """struct fuelq_rope of include/fuelq.h."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("k", "v", "cos_table", "sin_table", "kcache", "vcache")]


_rp = ctypes.POINTER(Rope)


class GgufTensor(ctypes.Structure):
    """struct fuelq_gguf_tensor of include/fuelq_gguf.h."""
    _fields_ = [("name", ctypes.c_char_p), ("ggml_type", ctypes.c_int32), ("n_dims", ctypes.c_int32),
                ("dims", ctypes.c_int64 * 8), ("offset", ctypes.c_uint64), ("nbytes", ctypes.c_uint64),
                ("data", ctypes.c_void_p)]


class GgufValue(ctypes.Structure):
    """struct fuelq_gguf_value of include/fuelq_gguf.h."""
    _fields_ = [("key", ctypes.c_char_p), ("type", ctypes.c_int32), ("elem_type", ctypes.c_int32),
                ("len", ctypes.c_uint64), ("i", ctypes.c_int64), ("f", ctypes.c_double), ("s", ctypes.c_void_p),
                ("array", ctypes.c_void_p)]


_u64 = ctypes.c_uint64

# name -> (restype, argtypes); must list every symbol include/fuelq.h declares
PROTOTYPES = {
    "fuelq_status_string": (ctypes.c_char_p, [_i32]),
    "fuelq_block_elems": (_i32, [_i32]),
    "fuelq_block_bytes": (_i32, [_i32]),
    "fuelq_set_option": (_i32, [_i32, _i64]),
    "fuelq_get_option": (_i64, [_i32]),
    "fuelq_device_error": (_i32, [ctypes.POINTER(_i32), _i32]),
    "fuelq_quantize_act": (_i32, [_i32, _i64, _i64, _vp, _vp, _vp]),
    "fuelq_act_packed_bytes": (_sz, [_i32, _i64, _i64]),
    "fuelq_quantize_act_packed": (_i32, [_i32, _i64, _i64, _vp, _vp, _sz, _vp]),
    "fuelq_qmatmul_workspace_bytes": (_sz, [_i32, _i64, _i64, _i64]),
    "fuelq_qmatmul_can_implement": (_i32, [_i32, _i64, _i64, _i64]),
    "fuelq_qmatmul_numerics": (_i32, [_i32, _i64, _i64, _i64]),
    "fuelq_qmatmul": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "fuelq_qmatmul_sharded": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _i64, _i64, _vp, _sz, _vp]),
    "fuelq_qmatmul_host_workspace_bytes": (_sz, [_i32, _i64, _i64, _i64]),
    "fuelq_qmatmul_host": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "fuelq_static_scratch_bytes": (_sz, []),
    "fuelq_qmatmul_static_scratch": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "fuelq_prefetch_weights": (_i32, [_vp, _i64, _vp]),
    "fuelq_qmatmul_packed": (_i32, [_i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "fuelq_quantize_weights": (_i32, [_i32, _i64, _vp, _vp, _vp]),
    "fuelq_dequantize": (_i32, [_i32, _i64, _vp, _vp, _i32, _vp]),
    "fuelq_embed_rows": (_i32, [_i32, _vp, _i64, _vp, _i64, _vp, _vp]),
    "fuelq_add_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, _vp]),
    "fuelq_rope_store": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "fuelq_attn_decode_workspace_bytes": (_sz, [_i32]),
    "fuelq_attn_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float, _vp, _sz, _rp, _vp]),
    "fuelq_add_rmsnorm_q8k": (_i32, [_vp, _vp, _vp, _i64, ctypes.c_float, _vp, _sz, _vp]),
    "fuelq_swiglu_q8k": (_i32, [_vp, _vp, _i64, _vp, _sz, _vp]),
    "fuelq_attn_decode_q8k": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float, _vp, _sz, _vp, _sz, _rp, _vp]),
    "fuelq_moe_route": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp]),
    "fuelq_moe_bucket": (_i32, [_vp, _i64, _i32, _vp, _vp, _vp]),
    "fuelq_moe_quantize_rows": (_i32, [_vp, _i64, _vp, _i32, _i64, _vp, _sz, _vp]),
    "fuelq_moe_swiglu_quantize": (_i32, [_vp, _i64, _i64, _vp, _sz, _vp]),
    "fuelq_moe_qmatmul": (_i32, [_i32, _i32, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "fuelq_moe_combine": (_i32, [_vp, _vp, _vp, _i64, _i32, _i64, _vp, _vp]),
    "fuelq_peer_vec_bytes": (_sz, [_i64]),
    "fuelq_ipc_alloc": (_i32, [_sz, ctypes.POINTER(_vp), _vp]),
    "fuelq_ipc_open": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "fuelq_ipc_close": (_i32, [_vp]),
    "fuelq_ipc_free": (_i32, [_vp]),
    "fuelq_qmatmul_packed_peer": (_i32, [_i32, _i64, _i64, _vp, _vp, _vp, _i64, _pp, _i32, _vp]),
    "fuelq_add_rmsnorm_q8k_peer": (_i32, [_vp, _vp, _i32, _vp, _i64, ctypes.c_float, _vp, _sz, _pp, _i32, _vp]),
    "fuelq_add_rmsnorm_q8k_parts": (_i32, [_vp, _vp, _i32, _vp, _i64, ctypes.c_float, _vp, _sz, _vp]),
    "fuelq_qmatmul_packed_tree": (_i32, [_i32, _i64, _i64, _vp, _vp, _vp, _i32, _vp, _vp]),
    "fuelq_qmatmul_packed_tree_peer": (_i32, [_i32, _i64, _i64, _vp, _vp, _vp, _i64, _pp, _i32, _i32, _vp, _vp]),
    "fuelq_moe_ep_pack": (_i32, [_vp, _i64, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i64, _vp, _vp]),
    "fuelq_moe_ep_local_ids": (_i32, [_vp, _i64, _i64, _i32, _i32, _vp, _vp]),
    "fuelq_moe_ep_unpack": (_i32, [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i64, _vp, _vp]),
    "fuelq_rowpar_reduce": (_i32, [_vp, _i32, _i64, _vp, _pp, _i32, _vp]),
    "fuelq_argmax_last_peer": (_i32, [_vp, _i64, _vp, _pp, _i32, _vp, _vp]),
    "fuelq_swiglu": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "fuelq_argmax_last": (_i32, [_vp, _i64, _vp, _vp]),
    # include/fuelq_host.h
    "fuelq_last_error": (ctypes.c_char_p, []),
    "fuelq_qtensor_load": (_i32, [_i32, _vp, _i32, _i64, _i64, _vp, _sz, ctypes.POINTER(_vp)]),
    "fuelq_qtensor_quantize": (_i32, [_i32, _vp, _i32, _i64, _i64, _vp, _i32, ctypes.POINTER(_vp)]),
    "fuelq_qtensor_free": (_i32, [_vp]),
    "fuelq_qtensor_info": (_i32, [_vp, ctypes.POINTER(_i32), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                  ctypes.POINTER(_sz), ctypes.POINTER(_vp)]),
    "fuelq_qtensor_data": (_i32, [_vp, _vp, _sz]),
    "fuelq_qtensor_dequantize": (_i32, [_vp, _vp, _i32]),
    "fuelq_qmatmul_forward": (_i32, [_vp, _vp, _i64, _vp]),
    "fuelq_qmatmul_forward_host": (_i32, [_vp, _vp, _i64, _vp]),
    # include/fuelq_seam.h
    "fuelq_seam_hello": (ctypes.c_int, [_vp]),
    # include/fuelq_gguf.h
    "fuelq_gguf_open": (_i32, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "fuelq_gguf_open_memory": (_i32, [_vp, _sz, ctypes.POINTER(_vp)]),
    "fuelq_gguf_close": (_i32, [_vp]),
    "fuelq_gguf_version": (_i32, [_vp]),
    "fuelq_gguf_alignment": (_u64, [_vp]),
    "fuelq_gguf_tensor_data_offset": (_u64, [_vp]),
    "fuelq_gguf_tensor_count": (_i64, [_vp]),
    "fuelq_gguf_find_tensor": (_i64, [_vp, ctypes.c_char_p]),
    "fuelq_gguf_tensor_at": (_i32, [_vp, _i64, ctypes.POINTER(GgufTensor)]),
    "fuelq_gguf_meta_count": (_i64, [_vp]),
    "fuelq_gguf_find_meta": (_i64, [_vp, ctypes.c_char_p]),
    "fuelq_gguf_meta_at": (_i32, [_vp, _i64, ctypes.POINTER(GgufValue)]),
    "fuelq_gguf_meta_array_string": (_i32, [_vp, _i64, _u64, ctypes.POINTER(_vp), ctypes.POINTER(_u64)]),
    "fuelq_gguf_load_tensor": (_i32, [_vp, _i64, _u64, _u64, _vp, _vp]),
}


class FuelqError(RuntimeError):
    def __init__(self, op: str, status: int, reason: str):
        super().__init__(f"{op}: status {status} ({reason})")
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this library.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the build is stale
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.fuelq_status_string(status).decode()


def check(status: int, op: str) -> None:
    if status != OK:
        raise FuelqError(op, status, status_string(status))
