"""Q5_K through the decode path (fuel-quantized/src/k_quants.rs:1626-1925): dequantization bit-identical, mat-vec
within the 1e-3 bar of the CPU restatement for every batch size on the exact-integer kernels (batches above 16 rows are
kept there by FUELQ_OPT_DECODE_MAX_M; the tensor-core form they take by default has its own tests), and a model with
Q5_K linears loaded from a GGUF file."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "kquants_golden.npz")

from test_gpu_kernels import _acts, _dev, _weights, assert_matmul_close, ops  # noqa: E402,F401


def test_dequantize_bit_identical(ops, oracle):
    from fuel_b200 import GgmlDType as T
    n, k = 37, 1024
    wb = oracle.quantize(oracle.Q5K, _weights(n, k))
    want = oracle.dequantize(oracle.Q5K, wb)
    assert np.array_equal(ops.dequantize(T.Q5K, _dev(wb), n * k).cpu().numpy().view(np.uint32), want.view(np.uint32))
    for dt in (torch.float16, torch.bfloat16):
        assert torch.equal(ops.dequantize(T.Q5K, _dev(wb), n * k, dt).cpu(), torch.from_numpy(want).to(dt))
    # any bytes, not just what the quantizer emits (f16 scale fields kept finite)
    rb = np.random.Generator(np.random.PCG64(12)).integers(0, 256, wb.size, dtype=np.uint8).reshape(-1, 176).copy()
    rb[:, 1] &= 0x3B
    rb[:, 3] &= 0x3B
    rb = rb.reshape(-1)
    assert np.array_equal(ops.dequantize(T.Q5K, _dev(rb), n * k).cpu().numpy().view(np.uint32),
                          oracle.dequantize(oracle.Q5K, rb).view(np.uint32))


@pytest.fixture
def integer_path():
    from fuel_b200 import _lib
    _lib.check(_lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 1 << 20), "set_option")
    yield
    _lib.lib.fuelq_set_option(_lib.OPT_DECODE_MAX_M, 0)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 16, 21])
def test_matvec_matches_reference(ops, oracle, integer_path, m):
    from fuel_b200 import GgmlDType as T
    for n, k in [(1, 256), (7, 256), (33, 512), (64, 4096), (300, 1024), (5, 11008)]:
        wb = oracle.quantize(oracle.Q5K, _weights(n, k, seed=n))
        x = _acts(m, k, seed=k + m)
        want = oracle.matmul(oracle.Q5K, x, wb, n)
        got = ops.qmatmul(T.Q5K, _dev(wb), n, _dev(x)).cpu().numpy()
        assert_matmul_close(got, want, f"q5k n={n} k={k} m={m}")
        # activations are the same Q8_K blocks every k-quant takes
        assert np.array_equal(ops.quantize_act(T.Q5K, _dev(x)).cpu().numpy(), oracle.quantize_act(oracle.Q5K, x))


def test_golden_fixture_and_benchmark_shape(ops, oracle):
    from fuel_b200 import GgmlDType as T
    g = np.load(GOLDEN)
    got = ops.qmatmul(T.Q5K, _dev(g["q5k_blocks"]), g["w"].shape[0], _dev(g["x"])).cpu().numpy()
    assert_matmul_close(got, g["q5k_y_scalar"])
    assert_matmul_close(got, g["q5k_y_avx2"])
    n, k = 11008, 4096
    wb = oracle.quantize(oracle.Q5K, _weights(n, k))
    for m in (1, 2):
        x = _acts(m, k)
        assert_matmul_close(ops.qmatmul(T.Q5K, _dev(wb), n, _dev(x)).cpu().numpy(), oracle.matmul(oracle.Q5K, x, wb, n), f"m={m}")


def test_device_weight_quantizer_byte_identical(ops, oracle):
    """BlockQ5K::from_float (k_quants.rs:1732-1887) on the device: the bytes of the CPU path's quantizer, edge cases included."""
    from fuel_b200 import GgmlDType as T, _lib
    from test_gpu_kernels import _weight_edge_cases
    for k in (256, 1024, 4096):
        w = _weight_edge_cases(k)
        got = ops.quantize_weights(T.Q5K, _dev(w)).cpu().numpy()
        want = oracle.quantize(oracle.Q5K, w)
        diff = np.nonzero(got != want)[0]
        assert diff.size == 0, f"k={k}: {diff.size} bytes differ, first at block {diff[0] // 176}"
    w = _weights(512, 4096, seed=12)
    assert np.array_equal(ops.quantize_weights(T.Q5K, _dev(w)).cpu().numpy(), oracle.quantize(oracle.Q5K, w))
    g = np.load(GOLDEN)
    assert np.array_equal(ops.quantize_weights(T.Q5K, _dev(g["w"])).cpu().numpy(), g["q5k_blocks"])
    with pytest.raises(_lib.FuelqError) as e:      # an activation block format is not a weight format: refused
        ops.quantize_weights(T.Q8_1, torch.zeros(4, 256, device="cuda"))
    assert e.value.status == _lib.NOT_SUPPORTED


def test_model_with_q5k_linears_from_gguf(tmp_path, oracle):
    from fuel_b200 import gguf as G, ops as _ops
    from fuel_b200.ggml import GgmlDType as T
    from fuel_b200.llama import LlamaConfig, QLlama, rope_tables
    from oracle.llama_oracle import OracleLlama
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    c = LlamaConfig(dim=256, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=128, ffn_dim=512, vocab=512, max_seq=48)
    rng = np.random.Generator(np.random.PCG64(21))
    shapes = {"attn_q": ("q", c.dim, c.dim), "attn_k": ("k", c.dim, c.dim), "attn_v": ("v", c.dim, c.dim),
              "attn_output": ("o", c.dim, c.dim), "ffn_gate": ("gate", c.ffn_dim, c.dim), "ffn_up": ("up", c.ffn_dim, c.dim),
              "ffn_down": ("down", c.dim, c.ffn_dim)}

    def qb(ot, n, k):
        return np.asarray(oracle.quantize(ot, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)), np.uint8).reshape(-1)

    emb = qb(oracle.Q5K, c.vocab, c.dim)
    tensors, olayers = [("token_embd.weight", T.Q5K, (c.vocab, c.dim), emb)], []
    for li in range(c.n_layers):
        ol = {}
        for nm, (short, n, k) in shapes.items():
            t, ot = (T.Q6K, oracle.Q6K) if nm == "ffn_down" else (T.Q5K, oracle.Q5K)
            b = qb(ot, n, k)
            tensors.append((f"blk.{li}.{nm}.weight", t, (n, k), b))
            ol[short] = (ot, b, n, k)
        for nm in ("attn_norm", "ffn_norm"):
            tensors.append((f"blk.{li}.{nm}.weight", T.F32, (c.dim,), np.ones(c.dim, np.float32).view(np.uint8)))
        olayers.append(ol)
    tensors.append(("output_norm.weight", T.F32, (c.dim,), np.ones(c.dim, np.float32).view(np.uint8)))
    head = qb(oracle.Q5K, c.vocab, c.dim)
    tensors.append(("output.weight", T.Q5K, (c.vocab, c.dim), head))
    meta = [("general.architecture", G.STRING, "llama"), ("llama.block_count", G.U32, c.n_layers),
            ("llama.attention.head_count", G.U32, c.n_heads)]
    path = str(tmp_path / "q5k.gguf")
    G.write_gguf(path, meta, tensors)
    model = QLlama.from_gguf(path, torch.device("cuda", 0), max_seq=c.max_seq)
    assert model.fused and model.head.dtype == T.Q5K
    cos, sin = rope_tables(model.cfg)
    emb_f32 = oracle.dequantize(oracle.Q5K, emb).reshape(c.vocab, c.dim)
    twin = OracleLlama(model.cfg, emb_f32, olayers, (oracle.Q5K, head, c.vocab, c.dim), cos, sin)
    prompt = rng.integers(0, c.vocab, 6).tolist()
    assert model.generate(prompt, 8) == twin.generate(prompt, 8)
    assert _ops.device_error() == 0
