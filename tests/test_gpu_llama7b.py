"""Benchmark configuration 4 at full size against the CPU path: the 7B-architecture model (32 layers, 4096 /
11008 / 32000, Q4_K_M-style mix, f32 KV cache), the seeded 512-token prompt, then greedy tokens, against the
CPU restatement of the reference's model glue over its quantized linears (oracle/llama_oracle.py; activation
re-quantization + integer dot products per linear).

What "the same forward pass" means at this depth. Two correct implementations sum f32 terms in different orders
(~1e-7 per linear). Every linear re-quantizes its input to 8 bits, so such a difference now and then flips one
activation quant (measured on small models: about one flip per 40 steps at dim 256 x 2 layers), which moves that
layer's outputs by ~1e-3 and, through the flips it causes downstream and through the KV cache, stays in every later
step. A one-layer model shows isolated steps at 1e-2 of the logit range; at 32 layers and 512 cached positions
the logits of two correct paths differ by several percent of their range, and a random-init model's nearly flat
logits (32 000 values) then pick different ids. The reference does this to itself: its scalar and its AVX2
summation orders (k_quants.rs vec_dot vs avx.rs) are two such paths.

So the yardstick is the reference's own spread. Three forward passes are fed the same ids (the prompt, then the
scalar-order CPU path's greedy picks): CPU scalar order (A), CPU AVX2 order (B), GPU (G). At every one of the 519
steps the test takes spread = max|B - A| and delta = max|G - A| over the logits, as fractions of A's range, and asks:
  - median(delta) <= 3 * median(spread) and max(delta) <= 3 * max(spread): the GPU is no further from the
    reference than a small multiple of what the reference's two orders are from each other;
  - G's greedy pick equals A's whenever A's top-2 gap exceeds twice delta (then no f32-accurate path can pick
    otherwise), and G agrees with A on about as many picks as B does.

The host twins take the very block bytes the device model holds (the device quantizer is byte-identical to
the CPU quantizer: tests/test_gpu_kernels.py::test_quantize_weights_*; a sample of rows is re-checked here),
so the comparison is of the forward pass alone. A few minutes of host time: each CPU pass streams 4 GB of blocks per token.
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

    # ---- CPU path: free-running greedy decode, logits of every new token kept
    src = SyntheticWeights(cfg, dev)
    ot = {12: O.Q4K, 14: O.Q6K}
    shapes = {"attn_q": "q", "attn_k": "k", "attn_v": "v", "attn_output": "o", "ffn_gate": "gate", "ffn_up": "up",
              "ffn_down": "down"}

    def host(name, li):
        n, k = src._shape(name)
        t = int(src.dtype(name, li))
        return (ot[t], src.rows(name, li, 0, n).cpu().numpy(), n, k)

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
    torch.cuda.empty_cache()
    cos, sin = rope_tables(cfg)
    n_steps = len(prompt) + N_NEW - 1
    a_twin = OracleLlama(cfg, embed, layers, head, cos, sin, order=O.SCALAR)
    b_twin = OracleLlama(cfg, embed, layers, head, cos, sin, order=O.AVX2)
    ids = list(prompt)
    a_logits, a_pick = [], []
    spread, b_same = np.zeros(n_steps), 0
    for i in range(n_steps):
        pa, la = a_twin.step(ids[i])
        pb, lb = b_twin.step(ids[i])
        a_logits.append(la)
        a_pick.append(pa)
        spread[i] = np.abs(lb - la).max() / np.abs(la).max()
        b_same += pb == pa
        if i + 1 >= len(prompt):
            ids.append(pa)                      # greedy continuation of the scalar-order CPU path
    del b_twin

    # ---- GPU path, fed the same ids
    model = QLlama(cfg, dev)
    try:
        model.reset()
        dev_ids = torch.as_tensor(ids, dtype=torch.int32, device=dev)
        delta, g_same, decided = np.zeros(n_steps), 0, 0
        for i in range(n_steps):
            model.token.copy_(dev_ids[i:i + 1])
            model.run_step()
            lg = model.logits.cpu().numpy()
            pick = int(model.next_token.item())
            r = a_logits[i]
            d = float(np.abs(lg - r).max())
            delta[i] = d / float(np.abs(r).max())
            top2 = np.partition(r, -2)[-2:]
            g_same += pick == a_pick[i]
            if float(top2[1] - top2[0]) > 2 * d:
                decided += 1
                assert pick == a_pick[i], (i, pick, a_pick[i])
        assert ops.device_error() == 0
    finally:
        model.release()
    print(f"7B config, {n_steps} teacher-forced steps: logit difference from the scalar CPU path, as a fraction of range: "
          f"GPU median {np.median(delta):.2e} max {delta.max():.2e}; AVX2-order CPU path median {np.median(spread):.2e} "
          f"max {spread.max():.2e}; identical picks GPU {g_same} / AVX2 {b_same} of {n_steps}; {decided} decided at f32 accuracy; "
          f"step 0: GPU {delta[0]:.2e}, AVX2 {spread[0]:.2e}")
    assert np.median(delta) <= 3 * np.median(spread), (np.median(delta), np.median(spread))
    assert delta.max() <= 3 * spread.max(), (delta.max(), spread.max())
    assert g_same >= b_same - max(8, n_steps // 10), (g_same, b_same)
