"""CPU-side checks of the C ABI: the library loads, exports every symbol the header
declares, and rejects bad arguments with the reference's status codes before any
device work (fuel-cuda-backend/src/baracuda/status.rs:5-12). No compute is launched."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(fuelq_\w+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def L():
    from fuel_b200 import _lib
    return _lib


def test_library_exports_every_declared_symbol(L):
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(L.lib, name), f"libfuelq.so lacks {name}"
    assert set(declared) == set(L.PROTOTYPES), set(declared) ^ set(L.PROTOTYPES)


def test_status_strings_and_block_tables(L):
    assert L.status_string(0) == "success"
    for code in range(1, 6):
        assert L.status_string(code) and "unknown" not in L.status_string(code)
    assert "unknown" in L.status_string(99)
    # fuel-ir/src/quantized.rs:77-103
    from fuel_b200 import GgmlDType as T
    for t in (T.Q4_0, T.Q4_1, T.Q5_0, T.Q5_1, T.Q8_0, T.Q8_1, T.Q2K, T.Q3K, T.Q4K, T.Q5K, T.Q6K, T.Q8K):
        assert L.lib.fuelq_block_elems(int(t)) == t.block_size()
        assert L.lib.fuelq_block_bytes(int(t)) == t.type_size()
    assert L.lib.fuelq_block_elems(5) == 0 and L.lib.fuelq_block_bytes(16) == 0  # ids GGUF does not assign to these formats
    assert T.from_u32(12) is T.Q4K and T.Q6K.to_u32() == 14
    with pytest.raises(ValueError):
        T.from_u32(99)


def test_argument_validation_needs_no_device(L):
    f = L.lib
    Q4K, Q8_0 = 12, 8
    # k not a multiple of the block size: every reference entry rejects it (byte_kernels.rs:4768-4773)
    assert f.fuelq_qmatmul(Q4K, 1, 8, 255, 16, 16, 16, 16, 1 << 20, None) == L.INVALID_PROBLEM
    assert f.fuelq_qmatmul(Q8_0, 1, 8, 33, 16, 16, 16, 16, 1 << 20, None) == L.INVALID_PROBLEM
    assert f.fuelq_qmatmul(Q4K, -1, 8, 256, 16, 16, 16, 16, 1 << 20, None) == L.INVALID_PROBLEM
    assert f.fuelq_qmatmul(9, 1, 8, 256, 16, 16, 16, 16, 1 << 20, None) == L.NOT_SUPPORTED   # Q8_1: activation blocks only
    # empty problems succeed without touching anything (byte_kernels.rs:4805-4807)
    assert f.fuelq_qmatmul(Q4K, 0, 8, 256, None, None, None, None, 0, None) == L.OK
    assert f.fuelq_qmatmul(Q4K, 1, 0, 256, None, None, None, None, 0, None) == L.OK
    # null / misaligned operands, missing workspace
    assert f.fuelq_qmatmul(Q4K, 1, 8, 256, None, 16, 16, 16, 1 << 20, None) == L.INVALID_PROBLEM
    assert f.fuelq_qmatmul(Q4K, 1, 8, 256, 8, 16, 16, 16, 1 << 20, None) == L.MISALIGNED
    assert f.fuelq_qmatmul(Q4K, 1, 8, 256, 16, 16, 16, None, 0, None) == L.WORKSPACE
    assert f.fuelq_qmatmul(Q4K, 1, 8, 256, 16, 16, 16, 16, 8, None) == L.WORKSPACE
    assert f.fuelq_quantize_act(Q4K, 1, 100, 16, 16, None) == L.INVALID_PROBLEM
    assert f.fuelq_quantize_act(Q4K, 1, 256, 4, 16, None) == L.MISALIGNED
    assert f.fuelq_dequantize(Q4K, 100, 16, 16, 0, None) == L.INVALID_PROBLEM
    assert f.fuelq_dequantize(Q4K, 256, 16, 16, 12, None) == L.NOT_SUPPORTED
    assert f.fuelq_dequantize(Q4K, 256, 8, 16, 0, None) == L.MISALIGNED
    assert f.fuelq_dequantize(Q4K, 0, None, None, 0, None) == L.OK
    # workspace sizing is pure arithmetic
    assert f.fuelq_qmatmul_workspace_bytes(Q4K, 1, 4096, 4096) == f.fuelq_act_packed_bytes(Q4K, 1, 4096) >= 4096 + 64 + 512
    assert f.fuelq_qmatmul_workspace_bytes(Q4K, 1, 4096, 100) == 0
    # which arithmetic a problem gets: the reference's integer path up to the crossover, tensor cores above
    assert f.fuelq_qmatmul_numerics(Q4K, 1, 4096, 4096) == L.NUMERICS_INTEGER
    assert f.fuelq_qmatmul_numerics(Q8_0, 16, 4096, 4096) == L.NUMERICS_INTEGER
    assert f.fuelq_qmatmul_numerics(Q8_0, 64, 4096, 4096) == L.NUMERICS_INTEGER     # the library's choice: up to 64 rows
    assert f.fuelq_qmatmul_numerics(Q8_0, 65, 4096, 4096) == L.NUMERICS_F16       # tensor cores, f16 operands by default
    assert f.fuelq_qmatmul_numerics(Q8_0, 2048, 4096, 4096) == L.NUMERICS_F16
    try:
        assert f.fuelq_set_option(L.OPT_PREFILL_BF16, 1) == L.OK
        assert f.fuelq_qmatmul_numerics(Q8_0, 2048, 4096, 4096) == L.NUMERICS_BF16
        assert f.fuelq_set_option(L.OPT_PREFILL_TF32, 1) == L.OK
        assert f.fuelq_qmatmul_numerics(Q8_0, 2048, 4096, 4096) == L.NUMERICS_TF32
    finally:
        f.fuelq_set_option(L.OPT_PREFILL_BF16, 0)
        f.fuelq_set_option(L.OPT_PREFILL_TF32, 0)
    # the tensor-core path's workspace: activations in the operand type, one factor per row, and a slab of dequantized rows
    assert f.fuelq_qmatmul_workspace_bytes(Q4K, 2048, 4096, 4096) == 2048 * 4096 * 2 + 2048 * 4 + 4096 * 4096 * 2
    try:   # ... unless Q4_K / Q6_K / Q8_0 are asked to dequantize inside the GEMM kernel
        assert f.fuelq_set_option(L.OPT_PREFILL_ONE_KERNEL, 1) == L.OK and f.fuelq_get_option(L.OPT_PREFILL_ONE_KERNEL) == 1
        assert f.fuelq_qmatmul_workspace_bytes(Q4K, 2048, 4096, 4096) == 2048 * 4096 * 2 + 2048 * 4
        assert f.fuelq_qmatmul_workspace_bytes(13, 2048, 4096, 4096) == 2048 * 4096 * 2 + 2048 * 4 + 4096 * 4096 * 2
    finally:
        f.fuelq_set_option(L.OPT_PREFILL_ONE_KERNEL, 0)
    # Q4_0 and the other formats without in-kernel stages: tensor cores above 16 rows; the workspace then also holds one slab
    assert f.fuelq_qmatmul_numerics(2, 16, 4096, 4096) == L.NUMERICS_INTEGER
    assert f.fuelq_qmatmul_numerics(2, 17, 4096, 4096) == L.NUMERICS_F16
    assert f.fuelq_qmatmul_numerics(13, 2048, 4096, 4096) == L.NUMERICS_F16
    assert f.fuelq_qmatmul_workspace_bytes(13, 2048, 4096, 4096) == 2048 * 4096 * 2 + 2048 * 4 + 4096 * 4096 * 2
    assert f.fuelq_qmatmul_workspace_bytes(2, 32, 1 << 20, 4096) == 32 * 4096 * 2 + 256 + (128 << 20)   # slab capped at 128 MiB
    assert f.fuelq_qmatmul_numerics(13, 64, 4096, 4096) == L.NUMERICS_INTEGER    # Q5_K: the integer tensor-core kernel up to 64 rows
    assert f.fuelq_qmatmul_numerics(13, 65, 4096, 4096) == L.NUMERICS_F16
    assert f.fuelq_qmatmul_numerics(2, 2048, 4096, 4096 + 32) == L.NUMERICS_INTEGER   # k not a multiple of 64: integer path
    assert f.fuelq_qmatmul_numerics(Q4K, 1, 4096, 100) == -L.INVALID_PROBLEM


def test_options_round_trip(L):
    f = L.lib
    assert f.fuelq_get_option(L.OPT_PDL) == 0
    assert f.fuelq_set_option(L.OPT_PDL, 1) == L.OK and f.fuelq_get_option(L.OPT_PDL) == 1
    assert f.fuelq_set_option(L.OPT_PDL, 0) == L.OK
    assert f.fuelq_set_option(L.OPT_DECODE_MAX_M, -1) == L.INVALID_PROBLEM
    assert f.fuelq_set_option(77, 1) == L.INVALID_PROBLEM


def test_argument_validation_of_moe_and_peer_entries_needs_no_gpu():
    """Bad arguments are refused with a status code before anything is launched (status 2 invalid problem, 3 not
    supported, 4 workspace), so these calls are safe on a machine without a GPU."""
    import ctypes

    from fuel_b200 import _lib
    L = _lib.lib
    INV, NOSUP = _lib.INVALID_PROBLEM, _lib.NOT_SUPPORTED
    assert L.fuelq_moe_route(None, 4, 8, 2, None, None, None) == INV            # null pointers
    assert L.fuelq_moe_route(None, 0, 8, 2, None, None, None) == 0              # no tokens: nothing to do
    assert L.fuelq_moe_route(None, 4, 2000, 2, None, None, None) == INV         # more experts than the router handles
    assert L.fuelq_moe_route(None, 4, 8, 9, None, None, None) == INV            # top_k > n_experts
    assert L.fuelq_moe_bucket(None, 16, 0, None, None, None) == INV
    assert L.fuelq_moe_quantize_rows(None, 100, None, 1, 4, None, 0, None) == INV   # k not a multiple of 256
    assert L.fuelq_moe_quantize_rows(None, 256, None, 0, 4, None, 0, None) == INV   # divisor
    assert L.fuelq_moe_swiglu_quantize(None, 300, 4, None, 0, None) == INV
    assert L.fuelq_moe_qmatmul(8, 4, 64, 256, None, None, 4, None, None, None, None) == NOSUP   # Q8_0 experts
    assert L.fuelq_moe_qmatmul(12, 4, 64, 256, None, None, 0, None, None, None, None) == 0      # no rows
    assert L.fuelq_moe_qmatmul(12, 4, 64, 256, None, None, 4, None, None, None, None) == INV
    assert L.fuelq_moe_combine(None, None, None, 4, 99, 64, None, None) == INV
    peers = _lib.Peers()
    peers.world, peers.rank, peers.epoch = 9, 0, 16
    assert L.fuelq_add_rmsnorm_q8k_peer(16, None, 1, 16, 256, 1e-5, 16, 1 << 20, ctypes.byref(peers), -1, None) == INV  # world > 8
    peers.world, peers.rank = 2, 2
    assert L.fuelq_argmax_last_peer(16, 8, 16, ctypes.byref(peers), 0, 16, None) == INV                              # rank >= world
    assert L.fuelq_peer_vec_bytes(10) == 80
