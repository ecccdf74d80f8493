"""Tensor-core path for the formats without a dequantizing stage of their own in the GEMM kernel (Q4_0, Q4_1, Q5_0,
Q5_1, Q2_K, Q3_K, Q5_K): above 16 activation rows their weights are dequantized, a slab of rows at a time, by the
stand-alone kernels (the reference's to_float arithmetic) into the tensor cores' operand type and multiplied by the
same tcgen05 kernel. Ground truth and bars are those of the other formats on that path: the exactly dequantized weights
times the f32 activations in f64, every output within 1e-3 of the tensor's largest value, relative Frobenius error
within 6e-4 (f16 operands, the default), and agreement with the reference's CPU path (8-bit activation blocks) within
the activation-quantization gap. All calls go through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

NAMES = ["q4_0", "q4_1", "q5_0", "q5_1", "q2k", "q3k", "q5k"]


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import _lib, ops as _ops
    # these tests are about the tensor-core path: put the crossover at 16 rows for every format (the library's own choice
    # keeps Q5_K batches of up to 64 rows on the integer tensor-core kernel)
    _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 16), "set_option")
    yield _ops
    _lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 0)
    assert _ops.device_error() == 0, "a kernel recorded an expired bounded wait"


def _types(oracle, name):
    from fuel_b200 import GgmlDType as T
    return {"q4_0": (T.Q4_0, oracle.Q4_0), "q4_1": (T.Q4_1, oracle.Q4_1), "q5_0": (T.Q5_0, oracle.Q5_0),
            "q5_1": (T.Q5_1, oracle.Q5_1), "q2k": (T.Q2K, oracle.Q2K), "q3k": (T.Q3K, oracle.Q3K),
            "q5k": (T.Q5K, oracle.Q5K)}[name]


def _w(n, k, seed=0):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((n, k), dtype=np.float32) * np.float32(0.02)


def _x(m, k, seed=1):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k), dtype=np.float32)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("m,n,k", [(17, 64, 256), (64, 256, 512), (200, 300, 1024), (257, 129, 768)])
def test_matches_float_oracle_and_cpu_path(ops, oracle, name, m, n, k):
    from fuel_b200 import _lib
    t, ot = _types(oracle, name)
    assert _lib.lib.fuelq_qmatmul_numerics(int(t), m, n, k) == _lib.NUMERICS_F16
    wb = oracle.quantize(ot, _w(n, k, seed=n))
    x = _x(m, k, seed=m)
    want = oracle.matmul_dequant_f64(ot, x, wb, n)
    y = torch.full((m, n), float("nan"), device="cuda")
    got = ops.qmatmul(t, torch.from_numpy(wb).cuda(), n, torch.from_numpy(x).cuda(), out=y).cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-3
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 6e-4
    ref_int = oracle.matmul(ot, x[:4], wb, n)  # the reference's CPU path on the same inputs
    assert np.abs(got[:4] - ref_int).max() / np.abs(ref_int).max() <= 2e-2


@pytest.mark.parametrize("name", ["q5k", "q4_0", "q3k"])
def test_several_slabs_and_a_ragged_last_one(ops, oracle, name):
    """The slab size is lowered so that 1000 rows take four slabs (384 rows each at k = 512, the last one 232 rows with a
    partial tile): every slab's columns land where the one-slab call puts them, bit for bit."""
    from fuel_b200 import _lib
    t, ot = _types(oracle, name)
    m, n, k = 96, 1000, 512
    wb = torch.from_numpy(oracle.quantize(ot, _w(n, k, seed=5))).cuda()
    x = torch.from_numpy(_x(m, k, seed=6)).cuda()
    one = ops.qmatmul(t, wb, n, x)
    try:
        _lib.check(_lib.lib.fuelq_set_option(116, 384), "set_option")  # KiB: 384 rows of 512 f16
        # activations as f16 + one factor per row, then exactly one slab
        assert _lib.lib.fuelq_qmatmul_workspace_bytes(int(t), m, n, k) == m * k * 2 + 512 + 384 * 1024
        many = ops.qmatmul(t, wb, n, x)
    finally:
        _lib.lib.fuelq_set_option(116, 0)
    assert torch.equal(one, many)
    want = oracle.matmul_dequant_f64(ot, x.cpu().numpy(), wb.cpu().numpy(), n)
    assert np.abs(one.cpu().numpy() - want).max() / np.abs(want).max() <= 1e-3


@pytest.mark.parametrize("opt,bar_max,bar_fro", [("tf32", 1e-3, 6e-4), ("bf16", 5e-3, 2.5e-3)])
def test_operand_options(ops, oracle, opt, bar_max, bar_fro):
    from fuel_b200 import _lib
    t, ot = _types(oracle, "q5k")
    m, n, k = 130, 200, 1024
    wb = oracle.quantize(ot, _w(n, k, seed=2))
    x = _x(m, k, seed=3)
    want = oracle.matmul_dequant_f64(ot, x, wb, n)
    key = _lib.OPT_PREFILL_TF32 if opt == "tf32" else _lib.OPT_PREFILL_BF16
    try:
        _lib.check(_lib.lib.fuelq_set_option(key, 1), "set_option")
        got = ops.qmatmul(t, torch.from_numpy(wb).cuda(), n, torch.from_numpy(x).cuda()).cpu().numpy()
    finally:
        _lib.lib.fuelq_set_option(key, 0)
    assert np.abs(got - want).max() / np.abs(want).max() <= bar_max
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= bar_fro


def test_block_scales_beyond_f16_saturate_instead_of_poisoning(ops, oracle):
    """A weight whose dequantized value exceeds f16's range (block scale 65504, 5-bit values) enters the product as
    +-65504, the same rule as the in-kernel stages; every output stays finite."""
    from fuel_b200 import GgmlDType as T
    m, n, k = 32, 128, 256
    wb = oracle.quantize(oracle.Q5_0, _w(n, k, seed=9)).copy().reshape(n, k // 32, 22)
    wb[3, 1, 0:2] = np.frombuffer(np.float16(65504.0).tobytes(), dtype=np.uint8)
    x = _x(m, k, seed=4)
    x[:, 32:64] = 0.0  # zeros against the huge block: an infinite operand would give NaN here
    got = ops.qmatmul(T.Q5_0, torch.from_numpy(wb.reshape(-1)).cuda(), n, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.isfinite(got).all()
    want = oracle.matmul_dequant_f64(oracle.Q5_0, x, wb.reshape(-1), n)
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-3


def test_crossover_option_keeps_the_integer_path(ops, oracle):
    from fuel_b200 import _lib
    t, ot = _types(oracle, "q4_1")
    m, n, k = 40, 96, 512
    wb = oracle.quantize(ot, _w(n, k))
    x = _x(m, k)
    want_int = oracle.matmul(ot, x, wb, n)
    try:
        _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 1 << 20), "set_option")
        assert _lib.lib.fuelq_qmatmul_numerics(int(t), m, n, k) == _lib.NUMERICS_INTEGER
        got = ops.qmatmul(t, torch.from_numpy(wb).cuda(), n, torch.from_numpy(x).cuda()).cpu().numpy()
    finally:
        _lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 16)
    assert np.abs(got - want_int).max() / np.abs(want_int).max() <= 2e-6
