"""GPU parity: every kernel is called through the C ABI and compared with the CPU
restatement of the reference (oracle/) on the same seeded inputs.

Bars (the stated parity bar): activation blocks byte-identical; dequantization
bit-identical; mat-vec outputs within max relative error 1e-3 of the reference's CPU
path. The integer dot products are exact on both sides, so the measured error is
f32 summation order only and the tests hold a much tighter line:
  tensor-normalised  max|y - r| / max|r|  <= 2e-6, and
  per element        |y - r| / |r|        <= 1e-3 wherever |r| >= 1e-3 * max|r|.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kquants_golden.npz")
NAMES = ("q4k", "q6k", "q8_0", "q4_0")


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import ops as _ops
    yield _ops
    assert _ops.device_error() == 0, "a kernel recorded an expired bounded wait"


def _T(name):
    from fuel_b200 import GgmlDType as T
    return {"q4k": T.Q4K, "q6k": T.Q6K, "q8_0": T.Q8_0, "q4_0": T.Q4_0}[name]


def _ot(O, name):
    return {"q4k": O.Q4K, "q6k": O.Q6K, "q8_0": O.Q8_0, "q4_0": O.Q4_0}[name]


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _weights(n, k, seed=0):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((n, k), dtype=np.float32) * np.float32(0.02)


def _acts(m, k, seed=1):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k), dtype=np.float32)


def assert_matmul_close(y, r, what=""):
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(r, dtype=np.float64)
    scale = np.abs(r).max()
    if scale == 0:
        assert np.abs(y).max() == 0, what
        return
    assert np.abs(y - r).max() / scale <= 2e-6, (what, np.abs(y - r).max() / scale)
    big = np.abs(r) >= 1e-3 * scale
    assert (np.abs(y - r)[big] / np.abs(r)[big]).max() <= 1e-3, what


# ----------------------------------------------------------------- activation quantization
def _edge_rows(k):
    x = _acts(8, k, seed=5)
    x[1] = 0.0                                   # all-zero blocks
    x[2, :] = np.float32(1e-30)                  # tiny but non-zero
    x[3, 0], x[3, 7] = 2.5, -2.5                 # +v / -v tie: first wins
    x[3, 8:16] = (np.arange(8, dtype=np.float32) + 0.5) * np.float32(2.5 / 128)  # exact .5 products
    x[4] *= np.float32(1e20)
    x[5, 3] = -0.0
    x[6, ::2] = 0.0
    x[7] = np.float32(7.0)                       # every element equal: index 0 wins
    return x


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("k", [256, 1024, 4096, 11008])
def test_quantize_act_bytes_identical(ops, oracle, name, k):
    x = np.concatenate([_acts(5, k), _edge_rows(k)])
    got = ops.quantize_act(_T(name), _dev(x)).cpu().numpy()
    want = oracle.quantize_act(_ot(oracle, name), x)
    assert got.shape == want.shape
    assert np.array_equal(got, want), f"{(got != want).sum()} bytes differ"


def test_quantize_act_q8_0_k_not_multiple_of_256(ops, oracle):
    for k in (32, 96, 160, 2080):
        x = _acts(3, k, seed=k)
        got = ops.quantize_act(_T("q8_0"), _dev(x)).cpu().numpy()
        assert np.array_equal(got, oracle.quantize_act(oracle.Q8_0, x))


def test_quantize_act_golden_fixture(ops):
    g = np.load(GOLDEN)
    for name in NAMES:
        got = ops.quantize_act(_T(name), _dev(g["x"])).cpu().numpy()
        assert np.array_equal(got, g[f"{name}_act"]), name


# ----------------------------------------------------------------- dequantize
@pytest.mark.parametrize("name", NAMES)
def test_dequantize_bit_identical(ops, oracle, name):
    n, k = 37, 1024
    wb = oracle.quantize(_ot(oracle, name), _weights(n, k))
    want = oracle.dequantize(_ot(oracle, name), wb)
    got = ops.dequantize(_T(name), _dev(wb), n * k)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    for dt in (torch.float16, torch.bfloat16):
        got16 = ops.dequantize(_T(name), _dev(wb), n * k, dt)
        assert torch.equal(got16.cpu(), torch.from_numpy(want).to(dt))


def test_dequantize_q8k_blocks(ops, oracle):
    from fuel_b200 import GgmlDType as T
    x = _acts(4, 512)
    blocks = oracle.quantize_act(oracle.Q4K, x)
    got = ops.dequantize(T.Q8K, _dev(blocks), x.size).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.dequantize(oracle.Q8K, blocks).view(np.uint32))


# ----------------------------------------------------------------- decode mat-vec
SMALL_SHAPES = {
    "q4k": [(1, 256), (7, 256), (33, 512), (64, 4096), (300, 1024), (5, 11008)],
    "q6k": [(1, 256), (7, 256), (33, 512), (64, 4096), (301, 1024), (5, 11008)],
    "q8_0": [(1, 32), (7, 96), (33, 512), (64, 4096), (299, 1056), (5, 11008)],
    "q4_0": [(1, 32), (7, 96), (33, 512), (64, 4096), (299, 1056), (5, 11008)],
}


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 13, 16])
def test_decode_matches_reference_small(ops, oracle, name, m):
    for n, k in SMALL_SHAPES[name]:
        wb = oracle.quantize(_ot(oracle, name), _weights(n, k, seed=n))
        x = _acts(m, k, seed=k + m)
        want = oracle.matmul(_ot(oracle, name), x, wb, n)
        got = ops.qmatmul(_T(name), _dev(wb), n, _dev(x)).cpu().numpy()
        assert_matmul_close(got, want, f"{name} n={n} k={k} m={m}")


def test_decode_golden_fixture(ops):
    g = np.load(GOLDEN)
    n = g["w"].shape[0]
    for name in NAMES:
        got = ops.qmatmul(_T(name), _dev(g[f"{name}_blocks"]), n, _dev(g["x"])).cpu().numpy()
        assert_matmul_close(got, g[f"{name}_y_scalar"], name)
        assert_matmul_close(got, g[f"{name}_y_avx2"], name)


def test_decode_reference_known_answers(ops):
    """The reference's own Q4_0 tests through the GPU path
    (fuel-cpu-backend/src/byte_kernels.rs:9713-9750, fuel-cuda-backend/src/quantized.rs:729-802)."""
    from fuel_b200 import GgmlDType as T
    blk = np.frombuffer(np.float16(1.0).tobytes() + bytes([0x99] * 16), dtype=np.uint8)
    w = _dev(np.concatenate([blk, blk]))
    y = ops.qmatmul(T.Q4_0, w, 2, _dev(np.arange(1, 33, dtype=np.float32)[None])).cpu().numpy()
    assert np.all(np.abs(y - 528.0) < 0.5), y
    y = ops.qmatmul(T.Q4_0, w, 2, _dev(np.zeros((1, 32), np.float32))).cpu().numpy()
    assert np.array_equal(y, np.zeros((1, 2), np.float32))


def test_decode_batch_shapes_and_row_independence(ops, oracle):
    """fwd keeps leading dims and replaces the last with n (fuel-cpu-backend/src/quantized.rs:85-142)."""
    from fuel_b200 import GgmlDType as T
    n, k = 48, 512
    wb = _dev(oracle.quantize(oracle.Q4K, _weights(n, k)))
    x = _dev(_acts(6, k)).reshape(2, 3, k)
    y = ops.qmatmul(T.Q4K, wb, n, x)
    assert y.shape == (2, 3, n)
    # a row's result does not depend on the batch around it: identical bits from the same
    # kernel variant, summation-order differences only between variants
    y1 = ops.qmatmul(T.Q4K, wb, n, x[1, 2:3].contiguous())
    assert_matmul_close(y1.cpu().numpy(), y[1, 2:3].cpu().numpy())
    from fuel_b200 import _lib
    try:
        _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_DECODE_KERNEL, 1), "set_option")
        yg = ops.qmatmul(T.Q4K, wb, n, x)
        y1g = ops.qmatmul(T.Q4K, wb, n, x[1, 2:3].contiguous())
    finally:
        _lib.lib.fuelq_set_option(_lib.OPT_DECODE_KERNEL, 0)
    assert_matmul_close(yg.cpu().numpy(), y.cpu().numpy())
    assert torch.equal(y1g, yg[1, 2:3])  # the generic kernel gives a row the same bits in any batch
    assert_matmul_close(y1g.cpu().numpy(), y1.cpu().numpy())


@pytest.mark.parametrize("name,n,k", [("q4k", 4096, 4096), ("q4k", 11008, 4096), ("q4k", 4096, 11008),
                                      ("q6k", 11008, 4096), ("q6k", 4096, 11008),
                                      ("q8_0", 11008, 4096), ("q8_0", 4096, 11008)])
def test_decode_benchmark_shapes(ops, oracle, name, n, k):
    """benchmark configurations 1 and 2 at full size, M in {1, 16}."""
    wb = oracle.quantize(_ot(oracle, name), _weights(n, k))
    wd = _dev(wb)
    for m in (1, 16):
        x = _acts(m, k)
        want = oracle.matmul(_ot(oracle, name), x, wb, n)
        got = ops.qmatmul(_T(name), wd, n, _dev(x)).cpu().numpy()
        assert_matmul_close(got, want, f"{name} n={n} k={k} m={m}")
    # linearity in the weights' rows: a permuted weight matrix permutes the output
    perm = np.random.Generator(np.random.PCG64(9)).permutation(n)
    rb = wb.reshape(n, -1)[perm].reshape(-1)
    x = _dev(_acts(1, k))
    y = ops.qmatmul(_T(name), wd, n, x)
    yp = ops.qmatmul(_T(name), _dev(rb), n, x)
    assert torch.equal(yp, y[:, torch.from_numpy(perm).cuda()])


def test_packed_activations_are_shared(ops, oracle):
    from fuel_b200 import GgmlDType as T
    n, k, m = 96, 1024, 3
    wb = _dev(oracle.quantize(oracle.Q6K, _weights(n, k)))
    x = _dev(_acts(m, k))
    packed = ops.quantize_act_packed(T.Q6K, x)
    y = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ops.qmatmul_packed(T.Q6K, wb, n, k, m, packed, y)
    assert torch.equal(y, ops.qmatmul(T.Q6K, wb, n, x))


def test_pdl_launch_gives_same_bits(ops, oracle):
    from fuel_b200 import GgmlDType as T, _lib
    n, k = 1024, 4096
    wb = _dev(oracle.quantize(oracle.Q4K, _weights(n, k)))
    x = _dev(_acts(2, k))
    y0 = ops.qmatmul(T.Q4K, wb, n, x)
    try:
        _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_PDL, 1), "set_option")
        ys = [ops.qmatmul(T.Q4K, wb, n, x) for _ in range(8)]
        torch.cuda.synchronize()
    finally:
        _lib.lib.fuelq_set_option(_lib.OPT_PDL, 0)
    for y in ys:
        assert torch.equal(y, y0)


@pytest.mark.parametrize("name", ["q4k", "q6k"])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (2, 1000, 11008), (1, 33, 256)])
def test_fused_quantization_gives_same_bits(ops, oracle, name, m, n, k):
    """m <= 2, option on: the mat-vec kernel quantizes the activation rows itself; m = 1: same bits as the two-kernel path."""
    from fuel_b200 import _lib
    wb = _dev(oracle.quantize(_ot(oracle, name), _weights(n, k)))
    x = _dev(_acts(m, k))
    y_two = ops.qmatmul(_T(name), wb, n, x)
    try:
        _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_FUSED_QUANT, 1), "set_option")
        y_fused = ops.qmatmul(_T(name), wb, n, x)
    finally:
        _lib.lib.fuelq_set_option(_lib.OPT_FUSED_QUANT, 0)
    if m == 1:
        assert torch.equal(y_fused, y_two)
    else:   # two rows: the two-kernel path runs on the integer tensor cores, another summation order over the blocks
        assert_matmul_close(y_fused.cpu().numpy(), y_two.cpu().numpy())
    assert_matmul_close(y_fused.cpu().numpy(), oracle.matmul(_ot(oracle, name), x.cpu().numpy(), wb.cpu().numpy(), n))


@pytest.mark.parametrize("name,m,n,k", [("q4k", 1, 11008, 4096), ("q6k", 3, 1000, 1024), ("q8_0", 16, 515, 2048),
                                        ("q4k", 40, 256, 4096)])
def test_host_buffers_pinned_or_pageable_give_the_device_path_bits(ops, oracle, name, m, n, k):
    """fuelq_qmatmul_host: pageable host memory is copied, small pinned (device-mapped) memory is read and written in
    place by the kernels; either way the result has the bits of the device-buffer call. (m = 40 x 4096 x 4 bytes is
    above the in-place limit: pinned, but copied.)"""
    wb = _dev(oracle.quantize(_ot(oracle, name), _weights(n, k)))
    x = torch.from_numpy(_acts(m, k))
    want = ops.qmatmul(_T(name), wb, n, x.cuda()).cpu()
    y_page = ops.qmatmul_host(_T(name), wb, n, x)
    torch.cuda.synchronize()
    assert torch.equal(y_page, want)
    from fuel_b200 import _lib
    xp = x.pin_memory()
    for pdl in (0, 1):      # one row: the write-back is inside the mat-vec kernel in plain launches, a kernel of its own with PDL
        y_pin = torch.full((m, n), float("nan")).pin_memory()
        try:
            _lib.lib.fuelq_set_option(_lib.OPT_PDL, pdl)
            for _ in range(3):   # back to back: a call's early read of x runs beside the previous call's kernels
                ops.qmatmul_host(_T(name), wb, n, xp, out_host=y_pin)
            torch.cuda.synchronize()
        finally:
            _lib.lib.fuelq_set_option(_lib.OPT_PDL, 0)
        assert torch.equal(y_pin, want), pdl
    # an odd (4-byte aligned only) pinned output address takes the scalar write-back
    base = torch.full((m * n + 1,), float("nan")).pin_memory()
    ops.qmatmul_host(_T(name), wb, n, xp, out_host=base[1:].view(m, n))
    torch.cuda.synchronize()
    assert torch.equal(base[1:].view(m, n), want) and torch.isnan(base[0])
    assert ops.device_error() == 0


def test_error_statuses_on_device(ops):
    from fuel_b200 import GgmlDType as T, _lib
    x = torch.zeros(1, 100, device="cuda")
    w = torch.zeros(144, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.FuelqError) as e:
        ops.qmatmul(T.Q4K, w, 1, x)
    assert e.value.status == _lib.INVALID_PROBLEM
    with pytest.raises(ValueError):
        ops.qmatmul(T.Q4K, w, 2, torch.zeros(1, 256, device="cuda"))
    with pytest.raises(ValueError):
        ops.qmatmul(T.Q4K, w, 1, torch.zeros(1, 256))


# ----------------------------------------------------------------- weight quantizers on the device
def _weight_edge_cases(k):
    w = _weights(24, k, seed=3)
    w[1] = 0.0                                    # all-zero blocks
    w[2] = np.float32(0.25)                       # constant: max == min
    w[3, :32] = 0.0                               # one zero sub-block inside a live block
    w[4] = np.abs(w[4])                           # all positive: min clamps to 0
    w[5] = -np.abs(w[5])
    w[6] *= np.float32(1e4)
    w[7] *= np.float32(1e-6)
    w[8, ::2] = w[8, 1::2]                        # repeated values (ties)
    w[9] = np.round(w[9] * 64) / 64               # coarse grid: many exact .5 cases
    w[10, :16] = 0.0                              # zero 16-sub-block (Q6_K scale 0)
    w[11] = np.linspace(-1, 1, k, dtype=np.float32)
    return w


@pytest.mark.parametrize("name", NAMES)
def test_quantize_weights_bytes_identical(ops, oracle, name):
    for k in (256, 1024, 4096):
        w = _weight_edge_cases(k)
        got = ops.quantize_weights(_T(name), _dev(w)).cpu().numpy()
        want = oracle.quantize(_ot(oracle, name), w)
        diff = np.nonzero(got != want)[0]
        assert diff.size == 0, f"{name} k={k}: {diff.size} bytes differ, first at block {diff[0] // _T(name).type_size()}"


@pytest.mark.parametrize("name", NAMES)
def test_quantize_weights_large_random(ops, oracle, name):
    w = _weights(1024, 4096, seed=21)
    got = ops.quantize_weights(_T(name), _dev(w)).cpu().numpy()
    assert np.array_equal(got, oracle.quantize(_ot(oracle, name), w))
    g = np.load(GOLDEN)
    assert np.array_equal(ops.quantize_weights(_T(name), _dev(g["w"])).cpu().numpy(), g[f"{name}_blocks"])
