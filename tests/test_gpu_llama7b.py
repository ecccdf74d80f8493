"""Benchmark configuration 4 at full size against the CPU path: the 7B-architecture model (32 layers, 4096 /
11008 / 32000, Q4_K_M-style mix, f32 KV cache), the seeded 512-token prompt, then greedy tokens — ids
identical to the CPU restatement of the reference's model glue over its quantized linears
(oracle/llama_oracle.py; activation re-quantization + integer dot products per linear, scalar order).

The host twin takes the very block bytes the device model holds (the device quantizer is byte-identical to
the CPU quantizer: tests/test_gpu_kernels.py::test_quantize_weights_*; a sample of rows is re-checked here),
so the comparison is of the forward pass alone. About a minute of host time: the CPU path streams 4 GB of
blocks per token.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

N_NEW = 8


def test_7b_config_greedy_tokens_match_cpu_reference_path(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fuel_b200 import ops
    from fuel_b200.llama import LlamaConfig, QLlama, SyntheticWeights, init_weight, q4km_mix, rope_tables
    from oracle.llama_oracle import OracleLlama
    O = oracle
    dev = torch.device("cuda", 0)
    cfg = LlamaConfig.llama2_7b()
    prompt = np.random.Generator(np.random.PCG64(3)).integers(0, cfg.vocab, 512).tolist()

    model = QLlama(cfg, dev)
    try:
        got = model.generate(prompt, N_NEW)
        torch.cuda.synchronize()
        gpu_logits = model.logits.cpu().numpy().copy()
        assert ops.device_error() == 0
    finally:
        model.release()
    del model
    torch.cuda.empty_cache()

    src = SyntheticWeights(cfg, dev)
    ot = {12: O.Q4K, 14: O.Q6K}
    shapes = {"attn_q": "q", "attn_k": "k", "attn_v": "v", "attn_output": "o", "ffn_gate": "gate", "ffn_up": "up",
              "ffn_down": "down"}

    def host(name, li):
        n, k = src._shape(name)
        t = int(src.dtype(name, li))
        blocks = src.rows(name, li, 0, n).cpu().numpy()
        return (ot[t], blocks, n, k)

    layers = [{short: host(name, li) for name, short in shapes.items()} for li in range(cfg.n_layers)]
    head = host("output", -1)
    embed = src.embedding()[1].cpu().numpy()
    # the device-quantized bytes are the CPU quantizer's bytes: a few rows of a Q4_K and of a Q6_K tensor
    for name, li, seed_slot in (("ffn_gate", 5, 5), ("ffn_down", 4, 7)):
        n, k = src._shape(name)
        t = int(q4km_mix(name, li))
        rows = init_weight(n, k, 1000 * (li + 1) + seed_slot, dev)[100:116].cpu().numpy()
        rb = k // 256 * O.block_bytes(ot[t])
        assert np.array_equal(O.quantize(ot[t], rows), layers[li][shapes[name]][1][100 * rb:116 * rb]), name

    cos, sin = rope_tables(cfg)
    twin = OracleLlama(cfg, embed, layers, head, cos, sin)
    want = twin.generate(prompt, N_NEW)
    assert got == want, (got, want)
    # the logits that picked the last token agree to f32 summation-order accuracy
    ref_logits = twin.last_logits
    assert np.abs(gpu_logits - ref_logits).max() <= 1e-3 * np.abs(ref_logits).max()
