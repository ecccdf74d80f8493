"""GGUF checkpoints into the quantized LLaMA decode: tensors go from the file mapping to the device unchanged,
and a model loaded from a file decodes the same greedy tokens as the CPU restatement of the reference's path
(oracle/llama_oracle.py) built from the same file's bytes."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _cfg():
    from fuel_b200.llama import LlamaConfig
    return LlamaConfig(dim=256, n_layers=2, n_heads=2, n_kv_heads=2, head_dim=128, ffn_dim=512, vocab=512, max_seq=48)


def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def test_exported_model_reloads_to_the_same_tokens(tmp_path):
    """Synthetic model -> GGUF file -> from_gguf: same linears byte for byte; the embedding table arrives as f32
    (as the reference's loader holds it), whose rows equal the on-the-fly Q4_K dequantization, so tokens match."""
    dev = _need_cuda()
    from fuel_b200.llama import QLlama, SyntheticWeights
    from fuel_b200 import ops
    cfg = _cfg()
    path = str(tmp_path / "tiny.gguf")
    SyntheticWeights(cfg, dev).export_gguf(path)
    a = QLlama(cfg, dev)
    b = QLlama.from_gguf(path, dev, max_seq=cfg.max_seq)
    import dataclasses
    # the file stores eps and theta as f32
    assert b.cfg == dataclasses.replace(cfg, norm_eps=float(np.float32(cfg.norm_eps))) and b.fused
    for la, lb in zip(a.layers, b.layers):
        for nm in ("qk", "v", "o", "gu", "down"):
            assert (la[nm] is None) == (lb[nm] is None)
            if la[nm] is not None:
                assert la[nm].dtype == lb[nm].dtype and torch.equal(la[nm].blocks, lb[nm].blocks)
    assert torch.equal(a.head.blocks, b.head.blocks)
    prompt = np.random.Generator(np.random.PCG64(5)).integers(0, cfg.vocab, 9).tolist()
    assert a.generate(prompt, 10) == b.generate(prompt, 10)
    assert ops.device_error() == 0


@pytest.mark.parametrize("version", [2, 3])
def test_checkpoint_with_gains_and_q8_0_against_cpu_path(tmp_path, oracle, version):
    """A file in the spirit of a real one: non-trivial norm gains, an f16 output norm, a Q6_K embedding table,
    Q8_0 and Q4_K and Q6_K linears, no output.weight (tied embeddings... to a Q6_K table). Tokens against the
    CPU path on the file's own bytes."""
    dev = _need_cuda()
    from fuel_b200 import gguf as G, ops
    from fuel_b200.ggml import GgmlDType as T
    from fuel_b200.llama import QLlama, rope_tables
    from oracle.llama_oracle import OracleLlama
    c = _cfg()
    rng = np.random.Generator(np.random.PCG64(11))
    ot = {T.Q4K: oracle.Q4K, T.Q6K: oracle.Q6K, T.Q8_0: oracle.Q8_0}
    shapes = {"attn_q": (c.dim, c.dim), "attn_k": (c.dim, c.dim), "attn_v": (c.dim, c.dim), "attn_output": (c.dim, c.dim),
              "ffn_gate": (c.ffn_dim, c.dim), "ffn_up": (c.ffn_dim, c.dim), "ffn_down": (c.dim, c.ffn_dim)}
    fmt = {"attn_q": T.Q4K, "attn_k": T.Q4K, "attn_v": T.Q8_0, "attn_output": T.Q8_0, "ffn_gate": T.Q6K, "ffn_up": T.Q6K,
           "ffn_down": T.Q4K}

    def qblocks(t, n, k):
        w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
        return np.asarray(oracle.quantize(ot[t], w), dtype=np.uint8).reshape(-1)

    tensors, olayers = [], []
    emb = qblocks(T.Q6K, c.vocab, c.dim)
    tensors.append(("token_embd.weight", T.Q6K, (c.vocab, c.dim), emb))
    for li in range(c.n_layers):
        ol = {}
        for nm, (n, k) in shapes.items():
            b = qblocks(fmt[nm], n, k)
            tensors.append((f"blk.{li}.{nm}.weight", fmt[nm], (n, k), b))
            ol[{"attn_q": "q", "attn_k": "k", "attn_v": "v", "attn_output": "o", "ffn_gate": "gate", "ffn_up": "up",
                "ffn_down": "down"}[nm]] = (ot[fmt[nm]], b, n, k)
        for nm in ("attn_norm", "ffn_norm"):
            gain = (1.0 + 0.1 * rng.standard_normal(c.dim)).astype(np.float32)
            tensors.append((f"blk.{li}.{nm}.weight", T.F32, (c.dim,), gain.view(np.uint8)))
            ol[nm] = gain
        olayers.append(ol)
    out_gain = (1.0 + 0.1 * rng.standard_normal(c.dim)).astype(np.float16)
    tensors.append(("output_norm.weight", T.F16, (c.dim,), out_gain.view(np.uint8)))
    meta = [("general.architecture", G.STRING, "llama"), ("llama.block_count", G.U32, c.n_layers),
            ("llama.attention.head_count", G.U32, c.n_heads), ("llama.attention.head_count_kv", G.U32, c.n_kv_heads),
            ("llama.attention.layer_norm_rms_epsilon", G.F32, 1e-6), ("llama.rope.freq_base", G.F32, 50000.0)]
    path = str(tmp_path / "mixed.gguf")
    G.write_gguf(path, meta, tensors, version=version, alignment=64)

    model = QLlama.from_gguf(path, dev, max_seq=c.max_seq)
    cfg = model.cfg
    assert (cfg.dim, cfg.n_layers, cfg.ffn_dim, cfg.vocab, cfg.head_dim) == (c.dim, c.n_layers, c.ffn_dim, c.vocab, 128)
    assert cfg.norm_eps == float(np.float32(1e-6)) and cfg.rope_theta == 50000.0
    assert not model.fused and model.head.dtype == T.Q6K   # Q8_0 linears: per-consumer quantization; tied head
    assert model.layers[0]["v"] is not None                 # v has another format than q/k: its own mat-vec
    emb_f32 = oracle.dequantize(oracle.Q6K, emb).astype(np.float32).reshape(c.vocab, c.dim)
    assert np.array_equal(model.embed.cpu().numpy(), emb_f32)
    cos, sin = rope_tables(cfg)
    twin = OracleLlama(cfg, emb_f32, olayers, (oracle.Q6K, emb, c.vocab, c.dim), cos, sin, out_norm=out_gain.astype(np.float32))
    prompt = rng.integers(0, c.vocab, 7).tolist()
    want = twin.generate(prompt, 10)
    assert model.generate(prompt, 10) == want
    _, ref_logits = twin.step(want[-1])
    model.run_step()
    torch.cuda.synchronize()
    assert np.abs(model.logits.cpu().numpy() - ref_logits).max() <= 1e-4 * np.abs(ref_logits).max()
    model.capture()                                          # graph replay of the plain step: same tokens
    assert model.generate(prompt, 10) == want
    assert ops.device_error() == 0


def test_loader_refusals(tmp_path):
    dev = _need_cuda()
    from fuel_b200 import gguf as G
    from fuel_b200.ggml import GgmlDType as T
    from fuel_b200.llama import QLlama, SyntheticWeights
    cfg = _cfg()
    path = str(tmp_path / "tiny.gguf")
    SyntheticWeights(cfg, dev).export_gguf(path)
    with G.GgufFile(path) as f:
        rows = f.load("blk.0.ffn_gate.weight", dev, 3, 5)   # a tensor-parallel rank's slice: rows 3, 4
        assert np.array_equal(rows.cpu().numpy(), f.tensor_bytes("blk.0.ffn_gate.weight")[3 * 144: 5 * 144])
        with pytest.raises(ValueError, match="outside tensor"):
            f.load("blk.0.ffn_gate.weight", dev, 0, cfg.ffn_dim + 1)
    import dataclasses
    with pytest.raises(ValueError, match="elements, expected"):   # a config that does not fit the file
        QLlama.from_gguf(path, dev, cfg=dataclasses.replace(cfg, ffn_dim=768))
    # a linear in a format the mat-vec does not take (Q8_K is an activation format)
    bad = str(tmp_path / "bad.gguf")
    with G.GgufFile(path) as f:
        tensors = [(n, i.ggml_dtype, i.shape, f.tensor_bytes(n)) for n, i in f.tensor_infos.items() if n != "blk.1.attn_output.weight"]
        meta = [(k, f.metadata_types[k], v) for k, v in f.metadata.items()]
    tensors.append(("blk.1.attn_output.weight", T.Q8K, (cfg.dim, cfg.dim), np.zeros(cfg.dim * cfg.dim // 256 * 292, np.uint8)))
    G.write_gguf(bad, meta, tensors)
    with pytest.raises(NotImplementedError, match="Q8K"):
        QLlama.from_gguf(bad, dev)
    with pytest.raises(KeyError, match="missing tensor"):
        G.write_gguf(bad, meta, tensors[:-1])
        QLlama.from_gguf(bad, dev)
