"""Q4_1, Q5_0 and Q5_1 (fuel-quantized/src/k_quants.rs:272-603) through the C ABI: the activation partner of the two
formats with a per-block minimum is Q8_1 (:695-762), whose blocks must be byte-identical to the CPU path's; the
dequantizer is bit-identical; the device weight quantizer is byte-identical; the mat-vec (the exact-integer decode
kernel at every batch size) matches the CPU path's matmul within f32 summation order."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kquants_golden.npz")
NAMES = ("q4_1", "q5_0", "q5_1")


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
    return {"q4_1": T.Q4_1, "q5_0": T.Q5_0, "q5_1": T.Q5_1}[name]


def _ot(O, name):
    return {"q4_1": O.Q4_1, "q5_0": O.Q5_0, "q5_1": O.Q5_1}[name]


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _weights(n, k, seed=0):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((n, k), dtype=np.float32) * np.float32(0.02)


def _acts(m, k, seed=1):
    return np.random.Generator(np.random.PCG64(seed)).standard_normal((m, k), dtype=np.float32)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("k", [32, 96, 1024, 4096, 11008])
def test_activation_blocks_byte_identical(ops, oracle, name, k):
    from test_gpu_kernels import _edge_rows
    x = np.concatenate([_acts(5, k), _edge_rows(max(k, 32))[:, :k]])
    x[6, :32] = 127.0                     # block sum 32 * 127 = 4064, above 2048: f16(sum) is a rounded value
    x[7, :32] = np.arange(32) * 4.0 + 1   # an odd sum above 2048
    got = ops.quantize_act(_T(name), _dev(x)).cpu().numpy()
    want = oracle.quantize_act(_ot(oracle, name), x)
    assert got.shape == want.shape
    assert np.array_equal(got, want), f"{(got != want).sum()} bytes differ"


@pytest.mark.parametrize("name", NAMES)
def test_dequantize_bit_identical(ops, oracle, name):
    n, k = 37, 1024
    O = oracle
    wb = O.quantize(_ot(O, name), _weights(n, k))
    rb = np.random.Generator(np.random.PCG64(9)).integers(0, 256, wb.size, dtype=np.uint8).reshape(-1, O.block_bytes(_ot(O, name)))
    rb[:, 1] &= 0x3B
    if name != "q5_0":
        rb[:, 3] &= 0x3B                  # finite f16 fields
    for blocks in (wb, rb.reshape(-1)):
        want = O.dequantize(_ot(O, name), blocks)
        got = ops.dequantize(_T(name), _dev(blocks), n * k)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
        for dt in (torch.float16, torch.bfloat16):
            assert torch.equal(ops.dequantize(_T(name), _dev(blocks), n * k, dt).cpu(), torch.from_numpy(want).to(dt))


@pytest.mark.parametrize("name", NAMES)
def test_weight_quantizer_byte_identical(ops, oracle, name):
    from test_gpu_kernels import _weight_edge_cases
    for k in (32, 1024, 4096):
        w = _weight_edge_cases(max(k, 256))[:, :k].copy()
        got = ops.quantize_weights(_T(name), _dev(w)).cpu().numpy()
        want = oracle.quantize(_ot(oracle, name), w)
        diff = np.nonzero(got != want)[0]
        assert diff.size == 0, f"{name} k={k}: {diff.size} bytes differ, first at block {diff[0] // _T(name).type_size()}"
    w = _weights(512, 4096, seed=12)
    assert np.array_equal(ops.quantize_weights(_T(name), _dev(w)).cpu().numpy(), oracle.quantize(_ot(oracle, name), w))


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 16, 17, 40])
def test_matvec_matches_cpu_path(ops, oracle, name, m):
    from test_gpu_kernels import assert_matmul_close
    for n, k in ((1, 32), (7, 96), (33, 512), (64, 4096), (299, 1056), (5, 11008)):
        wb = oracle.quantize(_ot(oracle, name), _weights(n, k, seed=n))
        x = _acts(m, k, seed=m)
        y = ops.qmatmul(_T(name), _dev(wb), n, _dev(x)).cpu().numpy()
        assert_matmul_close(y, oracle.matmul(_ot(oracle, name), x, wb, n), f"{name} m={m} n={n} k={k}")


@pytest.mark.parametrize("name", NAMES)
def test_benchmark_shapes_and_random_blocks(ops, oracle, name):
    from fuel_b200 import _lib
    from test_gpu_kernels import assert_matmul_close
    O = oracle
    for n, k in ((4096, 4096), (11008, 4096), (4096, 11008)):
        wb = O.quantize(_ot(O, name), _weights(n, k))
        for m in (1, 16):
            x = _acts(m, k, seed=3)
            assert _lib.lib.fuelq_qmatmul_numerics(int(_T(name)), m, n, k) == _lib.NUMERICS_INTEGER
            y = ops.qmatmul(_T(name), _dev(wb), n, _dev(x)).cpu().numpy()
            assert_matmul_close(y, O.matmul(_ot(O, name), x, wb, n), f"{name} m={m} n={n} k={k}")
    # blocks drawn from random bytes (finite f16 fields): every bit pattern of nibbles and fifth bits
    n, k = 96, 2048
    rb = np.random.Generator(np.random.PCG64(4)).integers(0, 256, (n * k // 32, O.block_bytes(_ot(O, name))), dtype=np.uint8)
    rb[:, 1] &= 0x3B
    if name != "q5_0":
        rb[:, 3] &= 0x3B
    x = _acts(3, k, seed=8)
    y = ops.qmatmul(_T(name), _dev(rb.reshape(-1)), n, _dev(x)).cpu().numpy()
    assert_matmul_close(y, O.matmul(_ot(O, name), x, rb.reshape(-1), n), name)


def test_golden_fixture(ops):
    g = np.load(GOLDEN)
    for name in NAMES:
        assert np.array_equal(ops.quantize_act(_T(name), _dev(g["x"])).cpu().numpy(), g[f"{name}_act"]), name
        assert np.array_equal(ops.quantize_weights(_T(name), _dev(g["w"])).cpu().numpy(), g[f"{name}_blocks"]), name
        n = g["w"].shape[0]
        y = ops.qmatmul(_T(name), _dev(g[f"{name}_blocks"]), n, _dev(g["x"])).cpu().numpy()
        assert np.abs(y - g[f"{name}_y_scalar"]).max() <= 2e-6 * np.abs(g[f"{name}_y_scalar"]).max()
        got = ops.dequantize(_T(name), _dev(g[f"{name}_blocks"]), g["w"].size).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), g[f"{name}_dequant"].view(np.uint32))


def test_model_with_mixed_legacy_linears_from_gguf(tmp_path, oracle):
    """A GGUF file whose linears are Q4_1 / Q5_0 / Q5_1 / Q4_0 / Q8_0 (three activation block formats in one layer: Q8_1, Q8_0
    and, for the Q6_K ffn_down, Q8_K) loads and decodes the CPU path's greedy tokens (the plain step: one quantization per
    activation format per input vector)."""
    from fuel_b200 import gguf as G, ops as _ops
    from fuel_b200.ggml import GgmlDType as T
    from fuel_b200.llama import LlamaConfig, QLlama, rope_tables
    from oracle.llama_oracle import OracleLlama
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    O = oracle
    c = LlamaConfig(dim=256, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=128, ffn_dim=512, vocab=512, max_seq=48)
    rng = np.random.Generator(np.random.PCG64(23))
    shapes = {"attn_q": ("q", c.dim, c.dim, T.Q4_1, O.Q4_1), "attn_k": ("k", c.dim, c.dim, T.Q4_1, O.Q4_1),
              "attn_v": ("v", c.dim, c.dim, T.Q5_0, O.Q5_0), "attn_output": ("o", c.dim, c.dim, T.Q5_1, O.Q5_1),
              "ffn_gate": ("gate", c.ffn_dim, c.dim, T.Q4_0, O.Q4_0), "ffn_up": ("up", c.ffn_dim, c.dim, T.Q4_0, O.Q4_0),
              "ffn_down": ("down", c.dim, c.ffn_dim, T.Q6K, O.Q6K)}

    def qb(ot, n, k):
        return np.asarray(O.quantize(ot, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)), np.uint8).reshape(-1)

    emb = qb(O.Q8_0, c.vocab, c.dim)
    tensors, olayers = [("token_embd.weight", T.Q8_0, (c.vocab, c.dim), emb)], []
    for li in range(c.n_layers):
        ol = {}
        for nm, (short, n, k, t, ot) in shapes.items():
            b = qb(ot, n, k)
            tensors.append((f"blk.{li}.{nm}.weight", t, (n, k), b))
            ol[short] = (ot, b, n, k)
        for nm in ("attn_norm", "ffn_norm"):
            tensors.append((f"blk.{li}.{nm}.weight", T.F32, (c.dim,), np.ones(c.dim, np.float32).view(np.uint8)))
        olayers.append(ol)
    tensors.append(("output_norm.weight", T.F32, (c.dim,), np.ones(c.dim, np.float32).view(np.uint8)))
    head = qb(O.Q5_1, c.vocab, c.dim)
    tensors.append(("output.weight", T.Q5_1, (c.vocab, c.dim), head))
    meta = [("general.architecture", G.STRING, "llama"), ("llama.block_count", G.U32, c.n_layers),
            ("llama.attention.head_count", G.U32, c.n_heads)]
    path = str(tmp_path / "legacy.gguf")
    G.write_gguf(path, meta, tensors)
    model = QLlama.from_gguf(path, torch.device("cuda", 0), max_seq=c.max_seq)
    assert not model.fused and model.head.dtype == T.Q5_1
    cos, sin = rope_tables(model.cfg)
    emb_f32 = O.dequantize(O.Q8_0, emb).reshape(c.vocab, c.dim)
    twin = OracleLlama(model.cfg, emb_f32, olayers, (O.Q5_1, head, c.vocab, c.dim), cos, sin)
    prompt = rng.integers(0, c.vocab, 6).tolist()
    assert model.generate(prompt, 8) == twin.generate(prompt, 8)
    assert _ops.device_error() == 0
