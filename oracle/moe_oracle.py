"""TEST INFRASTRUCTURE - CPU restatement of the reference's sparse MoE forward with quantized experts.

Router and layer follow fuel-core/src/lazy_nn/moe.rs:92-127 and :296-348 step by step (K rounds of first-maximum
argmax with the picked logit lowered by 1e30; softmax over the picked logits as byte_kernels.rs:2259-2305 computes it;
experts in ascending id, each over its routed rows in ascending token order; result scaled by the gate weight and
added to the token's accumulator). Expert products use the restated quantized matmul (oracle.matmul: activations
re-quantized to Q8_K, integer dot per block), since that is what a quantized expert's forward runs.
Only tests, the smoke check and the CPU leg of the benchmark may import this module.
"""
import numpy as np

from . import oracle as O

MASK_NEG = np.float32(-1.0e30)


def route(logits: np.ndarray, top_k: int):
    work = logits.astype(np.float32).copy()
    n = work.shape[0]
    ids = np.zeros((n, top_k), np.int32)
    picked = np.zeros((n, top_k), np.float32)
    rows = np.arange(n)
    for r in range(top_k):
        idx = np.argmax(work, axis=1)  # first maximum
        ids[:, r] = idx
        picked[:, r] = work[rows, idx]
        work[rows, idx] = work[rows, idx] + MASK_NEG
    w = np.zeros_like(picked)
    for t in range(n):
        mx = picked[t, 0]
        for v in picked[t, 1:]:
            if v > mx:
                mx = v
        e = np.exp((picked[t] - mx).astype(np.float32)).astype(np.float32)
        s = np.float32(0.0)
        for v in e:
            s = np.float32(s + v)
        w[t] = e * np.float32(np.float32(1.0) / s)
    return ids, w


def forward(x, logits, top_k, gate_up_blocks, down_blocks, n_experts, hidden, ffn, qtype=None):
    """gate_up_blocks[e]: uint8 blocks of [2*ffn, hidden]; down_blocks[e]: blocks of [hidden, ffn]."""
    qtype = O.Q4K if qtype is None else qtype
    ids, w = route(logits, top_k)
    n = x.shape[0]
    dense = np.zeros((n, n_experts), np.float32)
    for t in range(n):
        for s in range(top_k):
            dense[t, ids[t, s]] += w[t, s]
    acc = np.zeros((n, hidden), np.float32)
    for e in range(n_experts):
        sel = np.nonzero(dense[:, e])[0]
        if sel.size == 0:
            continue
        xe = np.ascontiguousarray(x[sel])
        gu = O.matmul(qtype, xe, gate_up_blocks[e], 2 * ffn)
        g, u = gu[:, :ffn], gu[:, ffn:]
        h = ((g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u).astype(np.float32)
        y = O.matmul(qtype, np.ascontiguousarray(h), down_blocks[e], hidden)
        acc[sel] = acc[sel] + (y * dense[sel, e][:, None]).astype(np.float32)
    return acc, ids, w
