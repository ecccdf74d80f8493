"""Pins the CPU restatement (oracle/) before anything is compared against it.

Three kinds of pin:
  * the reference's own known-answer tests for this path, restated
    (fuel-cpu-backend/src/byte_kernels.rs:9700-9760, fuel-dispatch/src/pipelined.rs:9916-10139,
    fuel-cuda-backend/src/quantized.rs:729-802);
  * gguf-py, an independent implementation of the same GGUF block layouts;
  * the committed fixture tests/golden/kquants_golden.npz.
"""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kquants_golden.npz")
FORMATS = ("q4_0", "q4_1", "q5_0", "q5_1", "q8_0", "q4k", "q5k", "q6k")
# byte offsets of the f16 fields of a block (kept finite when blocks are drawn from random bytes)
# formats whose quantizer is not restated: their blocks are random bytes in every test
NO_QUANTIZER = ("q2k", "q3k")
F16_FIELDS = {"q2k": (80, 82), "q3k": (108,), "q4_0": (0,), "q4_1": (0, 2), "q5_0": (0,), "q5_1": (0, 2), "q8_0": (0,), "q4k": (0, 2), "q5k": (0, 2), "q6k": (208,)}


def _t(O, name):
    return {"q4_0": O.Q4_0, "q4_1": O.Q4_1, "q5_0": O.Q5_0, "q5_1": O.Q5_1, "q8_0": O.Q8_0, "q2k": O.Q2K, "q3k": O.Q3K,
            "q4k": O.Q4K, "q5k": O.Q5K, "q6k": O.Q6K}[name]


def _gt(gguf, name):
    G = gguf.GGMLQuantizationType
    return {"q4_0": G.Q4_0, "q4_1": G.Q4_1, "q5_0": G.Q5_0, "q5_1": G.Q5_1, "q8_0": G.Q8_0, "q2k": G.Q2_K, "q3k": G.Q3_K,
            "q4k": G.Q4_K, "q5k": G.Q5_K, "q6k": G.Q6_K}[name]


def test_block_sizes(oracle):
    # fuel-ir/src/quantized.rs:77-103
    O = oracle
    assert [(O.block_elems(t), O.block_bytes(t)) for t in (O.Q4_0, O.Q8_0, O.Q4K, O.Q6K, O.Q8K)] == [
        (32, 18), (32, 34), (256, 144), (256, 210), (256, 292)]
    assert O.act_type(O.Q4K) == O.Q8K and O.act_type(O.Q6K) == O.Q8K
    assert O.act_type(O.Q8_0) == O.Q8_0 and O.act_type(O.Q4_0) == O.Q8_0


def test_f16_conversion_matches_ieee_rne(oracle):
    # the reference decodes f16 with `half`; fuel-graph/src/registry/qmatmul.rs:363-378 checks all finite patterns
    L = oracle.lib()
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([L.fq_oracle_f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.all(np.isnan(got[np.isnan(want)]))
    rng = np.random.Generator(np.random.PCG64(7))
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32),
        bits.view(np.float16).astype(np.float32)[finite],
        np.array([65504.0, 65519.9, 65520.0, 1e-8, 2.98e-8, 2.9802322e-8, 5.96e-8, 0.0, -0.0, np.inf, -np.inf],
                 dtype=np.float32)])
    with np.errstate(over="ignore"):
        want16 = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([L.fq_oracle_f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got16, want16)


def test_reference_q4_0_unit_weight_sums_activations(oracle):
    O = oracle
    blk = np.frombuffer(np.float16(1.0).tobytes() + bytes([0x99] * 16), dtype=np.uint8)
    w = np.concatenate([blk, blk])
    x = np.arange(1, 33, dtype=np.float32)[None]
    for order in (O.SCALAR, O.AVX2):
        y = O.matmul(O.Q4_0, x, w, 2, order)
        assert np.all(np.abs(y - 528.0) < 0.5), y
    assert np.array_equal(O.matmul(O.Q4_0, np.zeros((1, 32), np.float32), np.zeros(36, np.uint8), 2), np.zeros((1, 2)))


def test_reference_cuda_known_answers_q4_0(oracle):
    """Literal values asserted by the reference's CUDA tests. They were recorded on
    its Q8_1-activation GPU path; the CPU path quantizes activations to Q8_0, so the
    agreement is to a few 1e-4, inside the 1e-3 the first of those tests allows."""
    O = oracle
    v = np.arange(256, dtype=np.float32)
    y = O.matmul(O.Q4_0, v[None], O.quantize(O.Q4_0, v), 1)
    assert abs(float(y[0, 0]) - 5_559_680.0) / 5_559_680.0 <= 1e-3
    X = (np.arange(1024, dtype=np.float32) / 4).reshape(4, 256)
    y = O.matmul(O.Q4_0, X, O.quantize(O.Q4_0, X), 4).reshape(-1)
    qref = {0: 347_604.0, 1: 888_153.06, 4: 869_780.7, 5: 2_483_145.0, 11: 9_407_368.0, 14: 9_470_856.0,
            15: 13_138_824.0}
    for i, r in qref.items():
        assert abs(float(y[i]) - r) / r <= 1e-3, (i, y[i], r)


def test_reference_q6k_all_ones_ramp_orders_agree(oracle):
    # pipelined.rs:10071-10139: all-ones weights through from_float, ramp/100 activations
    O = oracle
    n, k = 2, 256
    wb = O.quantize(O.Q6K, np.ones((n, k), np.float32))
    x = (np.arange(1, k + 1, dtype=np.float32) / np.float32(100.0))[None]
    ys, ya = O.matmul(O.Q6K, x, wb, n, O.SCALAR), O.matmul(O.Q6K, x, wb, n, O.AVX2)
    want = float(x.sum())
    assert np.all(np.abs(ys - want) / want < 2e-2)
    assert np.all(np.abs(ys - ya) <= 1e-5 * np.abs(ys))


@pytest.mark.parametrize("name", FORMATS)
def test_layout_matches_gguf_py(oracle, name):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    O = oracle
    gt = _gt(gguf, name)
    w = np.random.Generator(np.random.PCG64(11)).standard_normal((16, 1024), dtype=np.float32) * np.float32(0.02)
    wb = O.quantize(_t(O, name), w)
    theirs = quants.dequantize(wb.reshape(16, -1), gt).reshape(-1)
    assert np.array_equal(O.dequantize(_t(O, name), wb).view(np.uint32), theirs.view(np.uint32))
    if not name.endswith("k"):  # gguf-py quantizes only the 32-element formats
        assert np.array_equal(quants.quantize(w, gt).reshape(-1), wb)
    # random bytes decode identically too (no reliance on what the quantizer emits)
    rb = np.random.Generator(np.random.PCG64(12)).integers(0, 256, wb.size, dtype=np.uint8)
    bb = O.block_bytes(_t(O, name))
    blocks = rb.reshape(-1, bb).copy()
    # keep the f16 scale fields finite
    for off in F16_FIELDS[name]:
        blocks[:, off + 1] &= 0x3B
    rb = blocks.reshape(-1)
    assert np.array_equal(O.dequantize(_t(O, name), rb).view(np.uint32),
                          quants.dequantize(rb.reshape(16, -1), gt).reshape(-1).view(np.uint32))


@pytest.mark.parametrize("name", FORMATS)
def test_golden_fixture(oracle, name):
    O = oracle
    g = np.load(GOLDEN)
    t = _t(O, name)
    w, x = g["w"], g["x"]
    n = w.shape[0]
    wb = O.quantize(t, w)
    assert np.array_equal(wb, g[f"{name}_blocks"])
    assert np.array_equal(O.dequantize(t, wb).view(np.uint32), g[f"{name}_dequant"].view(np.uint32))
    assert np.array_equal(O.quantize_act(t, x), g[f"{name}_act"])
    assert np.array_equal(O.matmul(t, x, wb, n, O.SCALAR).view(np.uint32), g[f"{name}_y_scalar"].view(np.uint32))
    assert np.array_equal(O.matmul(t, x, wb, n, O.AVX2).view(np.uint32), g[f"{name}_y_avx2"].view(np.uint32))


def test_q8k_conventions(oracle):
    """fuel-quantized/src/k_quants.rs:2230-2267: the largest-magnitude element maps to
    -128, ties keep the first, round is half-away-from-zero, zero blocks are all zero."""
    O = oracle
    x = np.zeros((1, 512), np.float32)
    x[0, 256 + 3] = 2.0
    x[0, 256 + 9] = -2.0          # later tie: ignored, so iscale = -64 and d < 0
    x[0, 256 + 10] = 2.0 * 0.5 / 128  # iscale*x = -0.5 -> rounds away from zero to -1
    x[0, 256 + 11] = -2.0 * 2.5 / 128  # +2.5 -> 3
    blk = O.quantize_act(O.Q4K, x).reshape(2, 292)
    assert not blk[0].any()
    d = blk[1, :4].view(np.float32)[0]
    qs = blk[1, 4:260].view(np.int8)
    bs = blk[1, 260:].view(np.int16)
    assert d == np.float32(1.0) / (np.float32(-128.0) / np.float32(2.0))
    assert qs[3] == -128 and qs[9] == 127 and qs[10] == -1 and qs[11] == 3
    assert np.array_equal(bs, qs.reshape(16, 16).astype(np.int32).sum(1).astype(np.int16))


@pytest.mark.parametrize("name", FORMATS)
def test_matmul_close_to_float_product(oracle, name):
    O = oracle
    t = _t(O, name)
    w = np.random.Generator(np.random.PCG64(0)).standard_normal((64, 1024), dtype=np.float32) * np.float32(0.02)
    x = np.random.Generator(np.random.PCG64(1)).standard_normal((4, 1024), dtype=np.float32)
    wb = O.quantize(t, w)
    y = O.matmul(t, x, wb, 64)
    ya = O.matmul(t, x, wb, 64, O.AVX2)
    yd = O.matmul_dequant_f64(t, x, wb, 64)
    assert np.abs(y - ya).max() <= 1e-5 * np.abs(y).max()
    # activation re-quantization (8 bit) is the only gap to the exact-weights product
    assert np.abs(y - yd).max() <= 2e-2 * np.abs(yd).max()
    # rows are independent of batch position
    assert np.array_equal(O.matmul(t, x[2:3], wb, 64), y[2:3])


def _dequant_act_blocks(O, name, act, m, k):
    """The activation blocks as real numbers, decoded here in numpy (not by the restatement):
    Q8_K = {d: f32, qs: i8[256], bsums: i16[16]} -> d * qs (k_quants.rs:162-169);
    Q8_0 = {d: f16, qs: i8[32]} -> d * qs (k_quants.rs:92-98). Also checks the Q8_K block sums."""
    if name.endswith("k"):
        b = act.reshape(m, k // 256, 292)
        d = b[:, :, :4].copy().view(np.float32).astype(np.float64)
        qs = b[:, :, 4:260].copy().view(np.int8).astype(np.float64)
        bs = b[:, :, 260:].copy().view(np.int16).astype(np.int64)
        assert np.array_equal(bs, qs.reshape(m, k // 256, 16, 16).sum(-1).astype(np.int64))
        return (d * qs).reshape(m, k)
    if name in ("q4_1", "q5_1"):   # Q8_1 = {d: f16, s: f16, qs: i8[32]} (k_quants.rs:100-107); s is checked by the caller
        b = act.reshape(m, k // 32, 36)
        d = b[:, :, :2].copy().view(np.float16).astype(np.float64)
        qs = b[:, :, 4:].copy().view(np.int8).astype(np.float64)
        return (d * qs).reshape(m, k)
    b = act.reshape(m, k // 32, 34)
    d = b[:, :, :2].copy().view(np.float16).astype(np.float64)
    qs = b[:, :, 2:].copy().view(np.int8).astype(np.float64)
    return (d * qs).reshape(m, k)


@pytest.mark.parametrize("source", ("quantizer", "random_bytes"))
@pytest.mark.parametrize("name", FORMATS)
def test_vec_dot_pinned_by_independent_dequantizers(oracle, name, source):
    """Tight pin of the integer dot products (k_quants.rs:1388-1468 Q4_K, 1946-2003 Q6_K, 674-692 Q8_0,
    252-269 Q4_0, 1770-1925 Q5_K and their AVX2 bodies): both operands of a vec_dot are exact integers
    times scales, so the restated matmul must equal, up to f32 summation order, the f64 product of
    gguf-py's dequantized weights with the activation blocks decoded in numpy. A wrong scale index,
    nibble order or block-sum sign shows up at 1e-2 or worse; the bar is 2e-6 of the largest output."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    O = oracle
    t = _t(O, name)
    gt = _gt(gguf, name)
    n, k, m = 48, 2048, 3
    rng = np.random.Generator(np.random.PCG64(21))
    if source == "quantizer":
        wb = O.quantize(t, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    else:
        bb = O.block_bytes(t)
        blocks = rng.integers(0, 256, (n * k // O.block_elems(t), bb), dtype=np.uint8)
        for off in F16_FIELDS[name]:
            blocks[:, off + 1] &= 0x3B  # finite f16 scales
        wb = blocks.reshape(-1)
    x = rng.standard_normal((m, k), dtype=np.float32)
    x[1, 256:512] = 0.0  # an all-zero activation block (d = 0 branch)
    act = O.quantize_act(t, x)
    xa = _dequant_act_blocks(O, name, act, m, k)
    w = quants.dequantize(wb.reshape(n, -1), gt).astype(np.float64).reshape(n, k)
    want = xa @ w.T
    if name in ("q4_1", "q5_1"):
        # Formats with a per-block minimum m: the reference adds m * s per block, s being the activation block's stored
        # f16 field (k_quants.rs:285-313, 501-533), where the product of the dequantized operands has m * (d * sum(q)).
        # s itself is restated here in numpy: f16(sum) * d in half arithmetic (k_quants.rs:728-757).
        ab = act.reshape(m, k // 32, 36)
        dy = ab[:, :, :2].copy().view(np.float16)[..., 0]
        s_stored = ab[:, :, 2:4].copy().view(np.float16)[..., 0]
        sums = ab[:, :, 4:].copy().view(np.int8).astype(np.int32).sum(-1)
        s_np = (sums.astype(np.float32).astype(np.float16).astype(np.float32) * dy.astype(np.float32)).astype(np.float16)
        assert np.array_equal(s_stored.view(np.uint16), s_np.view(np.uint16))
        mw = wb.reshape(n, k // 32, -1)[:, :, 2:4].copy().view(np.float16)[..., 0].astype(np.float64)    # [n, blocks]
        exact_ms = dy.astype(np.float64) * sums                                                              # [m, blocks]
        want = want + (s_stored.astype(np.float64) - exact_ms) @ mw.T
    scale = np.abs(want).max()
    for order in (O.SCALAR, O.AVX2):
        got = O.matmul(t, x, wb, n, order).astype(np.float64)
        assert np.abs(got - want).max() <= 2e-6 * scale, (name, source, order, np.abs(got - want).max() / scale)
    # one vec_dot called directly on the blocks, not through the matmul driver
    ab = act.reshape(m, -1)
    rb = wb.reshape(n, -1)
    for (i, j) in ((0, 0), (2, n - 1)):
        for order in (O.SCALAR, O.AVX2):
            v = O.vec_dot(t, order, k, np.ascontiguousarray(rb[j]), np.ascontiguousarray(ab[i]))
            assert abs(v - want[i, j]) <= 2e-6 * scale


@pytest.mark.parametrize("name", ("q2k", "q3k"))
def test_q2k_q3k_dequantize_like_gguf_py(oracle, name):
    """Q2_K / Q3_K (k_quants.rs:958-994, 1314-1366): to_float bit-identical to gguf-py's on random block bytes, and the
    block sizes of fuel-ir/src/quantized.rs:77-103."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    O = oracle
    t = _t(O, name)
    assert (O.block_elems(t), O.block_bytes(t)) == {"q2k": (256, 84), "q3k": (256, 110)}[name]
    blocks = np.random.Generator(np.random.PCG64(31)).integers(0, 256, (64, O.block_bytes(t)), dtype=np.uint8)
    for off in F16_FIELDS[name]:
        blocks[:, off + 1] &= 0x3B
    ours = O.dequantize(t, blocks.reshape(-1))
    theirs = quants.dequantize(blocks.reshape(4, -1), _gt(gguf, name)).reshape(-1)
    assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))


@pytest.mark.parametrize("name,bound", [("q2k", 0.45), ("q3k", 0.25), ("q4k", 0.12), ("q5k", 0.06), ("q6k", 0.03)])
def test_kquant_quantizers_round_trip(oracle, name, bound):
    """The K-quant weight quantizers have no independent implementation to compare bytes with; what can be checked is
    that to_float(from_float(w)) comes back within the format's resolution (rms error / rms of w, N(0, 0.02) weights),
    that constant and all-zero blocks behave as the reference's fit says (make_qkx1_quants returns (0, 0) when max == min,
    utils.rs:240-243: a constant block decodes to zeros in Q2_K / Q4_K / Q5_K), and that finer formats are more accurate."""
    O = oracle
    t = _t(O, name)
    w = np.random.Generator(np.random.PCG64(5)).standard_normal((64, 1024), dtype=np.float32) * np.float32(0.02)
    back = O.dequantize(t, O.quantize(t, w)).reshape(w.shape)
    rel = float(np.sqrt(((back - w) ** 2).mean()) / w.std())
    assert rel <= bound, rel
    assert rel >= bound / 6          # and it is this format's resolution, not a finer one's
    z = np.zeros((1, 256), np.float32)
    assert not O.dequantize(t, O.quantize(t, z)).any()
    c = np.full((1, 256), 0.25, np.float32)
    cb = O.dequantize(t, O.quantize(t, c))
    if name in ("q2k", "q4k", "q5k"):
        assert not cb.any()
    else:
        assert np.abs(cb - 0.25).max() <= 0.02
