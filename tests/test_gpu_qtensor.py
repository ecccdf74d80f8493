"""QTensor / QMatMul through the native host layer (include/fuelq_host.h), checked against the
CPU restatement of the reference. Mirrors how the reference's own tests drive the path:
build a weight with from_float, run matmul on a ramp, compare with a direct call
(fuel-dispatch/src/pipelined.rs:9916-10139), plus the storage contract of
fuel-backend-contract/src/quantized.rs:29-103 (data() returns the original bytes, fwd keeps
leading dims, non-contiguous or mis-shaped inputs are errors, never crashes)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def Q():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import quantized
    return quantized


def _T(name):
    from fuel_b200 import GgmlDType as T
    return {"q4k": T.Q4K, "q6k": T.Q6K, "q8_0": T.Q8_0, "q4_0": T.Q4_0, "q4_1": T.Q4_1, "q5_0": T.Q5_0, "q5_1": T.Q5_1, "q2k": T.Q2K,
            "q3k": T.Q3K, "q5k": T.Q5K}[name]


def _ot(O, name):
    return {"q4k": O.Q4K, "q6k": O.Q6K, "q8_0": O.Q8_0, "q4_0": O.Q4_0, "q4_1": O.Q4_1, "q5_0": O.Q5_0, "q5_1": O.Q5_1, "q2k": O.Q2K,
            "q3k": O.Q3K, "q5k": O.Q5K}[name]


def _close(y, r):
    y, r = np.asarray(y, np.float64), np.asarray(r, np.float64)
    assert np.abs(y - r).max() <= 2e-6 * np.abs(r).max()


@pytest.mark.parametrize("name", ["q4k", "q6k", "q8_0", "q4_0", "q4_1", "q5_0", "q5_1", "q2k", "q3k", "q5k"])
def test_quantize_data_dequantize_forward(Q, oracle, name):
    n, k = 96, 1024
    w = np.random.Generator(np.random.PCG64(0)).standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    want_blocks = oracle.quantize(_ot(oracle, name), w)
    for src in (w, torch.from_numpy(w).cuda()):  # quantize_onto (host source) and quantize (device source)
        qt = Q.QTensor.quantize(src, _T(name))
        assert qt.dtype() == _T(name) and qt.shape() == (n, k) and qt.rank() == 2
        assert qt.block_size() == _T(name).block_size()
        assert qt.storage_size_in_bytes() == want_blocks.size
        assert np.array_equal(qt.data(), want_blocks)          # data() gives back the block bytes
        assert qt.device_ptr() % 16 == 0
        deq = qt.dequantize().cpu().numpy().reshape(-1)
        assert np.array_equal(deq.view(np.uint32), oracle.dequantize(_ot(oracle, name), want_blocks).view(np.uint32))
        assert torch.equal(qt.dequantize_f16().cpu().reshape(-1), torch.from_numpy(deq).to(torch.float16))
    mm = Q.QMatMul.from_qtensor(qt)
    for shape in ((1, k), (5, k), (2, 3, k), (16, k)):
        x = np.random.Generator(np.random.PCG64(1)).standard_normal(shape, dtype=np.float32)
        want = oracle.matmul(_ot(oracle, name), x, want_blocks, n)
        y = mm.forward(torch.from_numpy(x).cuda())
        assert tuple(y.shape) == (*shape[:-1], n)
        _close(y.cpu().numpy(), want)
        yh = mm(x)                                              # host in, host out
        assert isinstance(yh, np.ndarray) and yh.shape == want.shape
        _close(yh, want)


def test_from_blocks_and_reference_style_ramp(Q, oracle):
    # all-ones weights quantized by from_float, ramp activations: pipelined.rs:10071-10139
    from fuel_b200 import GgmlDType as T
    n, k = 2, 256
    blocks = oracle.quantize(oracle.Q6K, np.ones((n, k), np.float32))
    qt = Q.QTensor.from_blocks(blocks, T.Q6K, (n, k))
    assert np.array_equal(qt.data(), blocks)
    x = (np.arange(1, k + 1, dtype=np.float32) / np.float32(100.0))[None]
    y = Q.QMatMul.from_qtensor(qt).forward(x)
    _close(y, oracle.matmul(oracle.Q6K, x, blocks, n))


def test_error_behaviour(Q):
    from fuel_b200 import GgmlDType as T, _lib
    with pytest.raises(_lib.FuelqError) as e:
        Q.QTensor.quantize(np.zeros((4, 100), np.float32), T.Q4K)     # k not a multiple of the block
    assert e.value.status == _lib.INVALID_PROBLEM
    with pytest.raises(_lib.FuelqError):
        Q.QTensor.from_blocks(np.zeros(100, np.uint8), T.Q4K, (1, 256))  # byte count does not match
    qt = Q.QTensor.quantize(np.ones((8, 256), np.float32), T.Q4K)
    mm = Q.QMatMul.from_qtensor(qt)
    with pytest.raises(_lib.FuelqError):
        mm.forward(torch.zeros(256, device="cuda"))                   # rank 1
    with pytest.raises(_lib.FuelqError):
        mm.forward(torch.zeros(2, 512, device="cuda"))                # wrong k
    with pytest.raises(_lib.FuelqError):
        mm.forward(torch.zeros(512, 2, device="cuda").t())            # not contiguous
    with pytest.raises(_lib.FuelqError):
        mm.forward(torch.zeros(2, 256, device="cuda", dtype=torch.float16))
    assert mm.forward(torch.zeros(0, 256, device="cuda")).shape == (0, 8)   # empty batch is fine
