"""Q2_K and Q3_K (fuel-quantized/src/k_quants.rs:764-1367) through the C ABI: the dequantizer is bit-identical to the
CPU path's, and the mat-vec (the exact-integer decode kernel at every batch size, Q8_K activation blocks) matches the
CPU path's matmul within f32 summation order, on blocks drawn from random bytes with finite f16 fields (every bit pattern of
quants, high bits and scales occurs) and on quantizer output; the device weight quantizers (BlockQ2K / BlockQ3K::from_float,
:836-895, :1135-1216) emit the CPU path's bytes."""
import os
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

NAMES = ("q2k", "q3k")
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kquants_golden.npz")
F16_FIELDS = {"q2k": (80, 82), "q3k": (108,)}


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import _lib, ops as _ops
    # these tests are about the integer kernels (the reference's arithmetic) at every batch size: keep batches above 16 rows
    # off the tensor-core path, which has its own tests
    _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 1 << 20), "set_option")
    yield _ops
    _lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 0)
    assert _ops.device_error() == 0, "a kernel recorded an expired bounded wait"


def _T(name):
    from fuel_b200 import GgmlDType as T
    return {"q2k": T.Q2K, "q3k": T.Q3K}[name]


def _ot(O, name):
    return {"q2k": O.Q2K, "q3k": O.Q3K}[name]


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _blocks(O, name, n, k, seed):
    t = _ot(O, name)
    b = np.random.Generator(np.random.PCG64(seed)).integers(0, 256, (n * k // 256, O.block_bytes(t)), dtype=np.uint8)
    for off in F16_FIELDS[name]:
        b[:, off + 1] &= 0x33          # finite, moderate f16 scales
    return b.reshape(-1)


def _acts(m, k, seed=1):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k), dtype=np.float32)


@pytest.mark.parametrize("name", NAMES)
def test_dequantize_bit_identical(ops, oracle, name):
    n, k = 37, 1024
    wb = _blocks(oracle, name, n, k, 3)
    want = oracle.dequantize(_ot(oracle, name), wb)
    got = ops.dequantize(_T(name), _dev(wb), n * k)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for dt in (torch.float16, torch.bfloat16):
        assert torch.equal(ops.dequantize(_T(name), _dev(wb), n * k, dt).cpu(), torch.from_numpy(want).to(dt))


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 16, 17, 40])
def test_matvec_matches_cpu_path(ops, oracle, name, m):
    from test_gpu_kernels import assert_matmul_close
    for n, k in ((1, 256), (7, 256), (33, 512), (64, 4096), (301, 1024), (5, 11008)):
        wb = _blocks(oracle, name, n, k, n)
        x = _acts(m, k, seed=m)
        y = ops.qmatmul(_T(name), _dev(wb), n, _dev(x)).cpu().numpy()
        assert_matmul_close(y, oracle.matmul(_ot(oracle, name), x, wb, n), f"{name} m={m} n={n} k={k}")


@pytest.mark.parametrize("name", NAMES)
def test_benchmark_shapes(ops, oracle, name):
    from fuel_b200 import _lib
    from test_gpu_kernels import assert_matmul_close
    for n, k in ((4096, 4096), (11008, 4096), (4096, 11008)):
        wb = _blocks(oracle, name, n, k, 5)
        for m in (1, 16):
            x = _acts(m, k, seed=3)
            assert _lib.lib.fuelq_qmatmul_numerics(int(_T(name)), m, n, k) == _lib.NUMERICS_INTEGER
            y = ops.qmatmul(_T(name), _dev(wb), n, _dev(x)).cpu().numpy()
            assert_matmul_close(y, oracle.matmul(_ot(oracle, name), x, wb, n), f"{name} m={m} n={n} k={k}")


@pytest.mark.parametrize("name", NAMES)
def test_activation_blocks_are_q8k(ops, oracle, name):
    x = _acts(4, 1024)
    assert np.array_equal(ops.quantize_act(_T(name), _dev(x)).cpu().numpy(), oracle.quantize_act(oracle.Q4K, x))


@pytest.mark.parametrize("name", NAMES)
def test_weight_quantizer_byte_identical(ops, oracle, name):
    from test_gpu_kernels import _weight_edge_cases
    for k in (256, 1024, 4096):
        w = _weight_edge_cases(k)
        got = ops.quantize_weights(_T(name), _dev(w)).cpu().numpy()
        want = oracle.quantize(_ot(oracle, name), w)
        diff = np.nonzero(got != want)[0]
        assert diff.size == 0, f"{name} k={k}: {diff.size} bytes differ, first at block {diff[0] // _T(name).type_size()}"
    w = np.random.Generator(np.random.PCG64(12)).standard_normal((512, 4096), dtype=np.float32) * np.float32(0.02)
    wb = oracle.quantize(_ot(oracle, name), w)
    assert np.array_equal(ops.quantize_weights(_T(name), _dev(w)).cpu().numpy(), wb)
    g = np.load(GOLDEN)
    assert np.array_equal(ops.quantize_weights(_T(name), _dev(g["w"])).cpu().numpy(), g[f"{name}_blocks"])
    # and the quantizer's own blocks through the mat-vec
    from test_gpu_kernels import assert_matmul_close
    x = _acts(3, 4096, seed=9)
    y = ops.qmatmul(_T(name), _dev(wb), 512, _dev(x)).cpu().numpy()
    assert_matmul_close(y, oracle.matmul(_ot(oracle, name), x, wb, 512), name)
