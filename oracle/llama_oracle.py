"""TEST INFRASTRUCTURE — CPU forward of the quantized LLaMA-architecture decode step, for token parity.

numpy f32 restatement of the reference's model glue around its quantized linears
(fuel-core/src/lazy.rs:7363-7447): RMSNorm as x * 1/sqrt(mean(x^2)+eps) then gain with a sequential
f32 sum (fuel-cpu-backend/src/byte_kernels.rs:2339-2367), rotate-half RoPE (byte_kernels.rs:1885-1960),
max-subtracted softmax (byte_kernels.rs:2259-2305), SwiGLU, and greedy pick of the last maximal index
(fuel-transformers/src/generation/mod.rs:84-93). Linears go through oracle.matmul (activation
re-quantization + integer dot products, the reference's CPU path).
"""
from __future__ import annotations

import numpy as np

from . import oracle as O


def _rmsnorm(x, gain, eps):
    # sequential f32 accumulation, as the reference loop: ss = 0; for v in x: ss += v * v
    # (np.add.accumulate adds left to right in the array's own type, one rounding per element)
    ss = np.add.accumulate((x * x).astype(np.float32), dtype=np.float32)[-1]
    rinv = np.float32(1.0) / np.sqrt(np.float32(ss * (np.float32(1.0) / np.float32(x.size)) + np.float32(eps)))
    return (x * rinv * gain).astype(np.float32)


def _rope(x, cos, sin):               # x [heads, hd]
    h = x.shape[1] // 2
    lo, hi = x[:, :h], x[:, h:]
    return np.concatenate([lo * cos[:h] - hi * sin[:h], hi * cos[h:] + lo * sin[h:]], axis=1).astype(np.float32)


class OracleLlama:
    """weights: dict name -> (ggml type id, uint8 blocks, n, k). Norm gains are ones unless a layer dict holds
    "attn_norm" / "ffn_norm" f32 vectors and `out_norm` is given. `embed_blocks` is the Q4_K block bytes of the
    embedding table, or an f32 [vocab, dim] array (how the reference holds it after loading a checkpoint).
    `order` picks the scalar or the AVX2 summation order of the reference's dot products; the two give logits that
    differ at the 1e-7 level per linear, and (through the 8-bit re-quantization of every linear's input, which turns
    such a difference into an occasional flipped quant) by far more after many layers: the spread between the two is
    the yardstick for what "the same forward pass" can mean at depth."""

    def __init__(self, cfg, embed_blocks, layers, head, cos, sin, out_norm=None, order=O.SCALAR):
        self.cfg, self.embed, self.layers, self.head, self.cos, self.sin = cfg, embed_blocks, layers, head, cos, sin
        self.out_norm = out_norm
        self.order = order      # which of the reference's two f32 summation orders the linears use (scalar / AVX2)
        c = cfg
        self.kc = np.zeros((c.n_layers, c.n_kv_heads, c.max_seq, c.head_dim), np.float32)
        self.vc = np.zeros_like(self.kc)
        self.pos = 0

    def _lin(self, w, x):
        t, blocks, n, k = w
        return O.matmul(t, x[None, :], blocks, n, self.order)[0]

    def step(self, token: int):
        c = self.cfg
        if self.embed.dtype == np.float32:
            x = self.embed[token].astype(np.float32)
        else:
            rb = c.dim // 256 * 144
            x = O.dequantize(O.Q4K, self.embed[token * rb:(token + 1) * rb]).astype(np.float32)
        ones = np.ones(c.dim, np.float32)
        for li, l in enumerate(self.layers):
            h = _rmsnorm(x, l.get("attn_norm", ones), c.norm_eps)
            q = self._lin(l["q"], h).reshape(c.n_heads, c.head_dim)
            k = self._lin(l["k"], h).reshape(c.n_kv_heads, c.head_dim)
            v = self._lin(l["v"], h).reshape(c.n_kv_heads, c.head_dim)
            q = _rope(q, self.cos[self.pos], self.sin[self.pos])
            k = _rope(k, self.cos[self.pos], self.sin[self.pos])
            self.kc[li, :, self.pos], self.vc[li, :, self.pos] = k, v
            n_ctx, rep = self.pos + 1, c.n_heads // c.n_kv_heads
            out = np.zeros((c.n_heads, c.head_dim), np.float32)
            scale = np.float32(1.0 / np.sqrt(c.head_dim))
            for hd in range(c.n_heads):
                kk, vv = self.kc[li, hd // rep, :n_ctx], self.vc[li, hd // rep, :n_ctx]
                s = (kk @ q[hd]).astype(np.float32) * scale
                e = np.exp(s - s.max()).astype(np.float32)
                out[hd] = (e / e.sum(dtype=np.float32)) @ vv
            x = (x + self._lin(l["o"], out.reshape(-1))).astype(np.float32)
            h = _rmsnorm(x, l.get("ffn_norm", ones), c.norm_eps)
            g, u = self._lin(l["gate"], h), self._lin(l["up"], h)
            s = ((g / (np.float32(1.0) + np.exp(-g))) * u).astype(np.float32)
            x = (x + self._lin(l["down"], s)).astype(np.float32)
        h = _rmsnorm(x, ones if self.out_norm is None else self.out_norm, c.norm_eps)
        logits = self._lin(self.head, h)
        self.pos += 1
        m = logits.max()
        return int(np.nonzero(logits == m)[0][-1]), logits

    def generate(self, prompt, n_new):
        self.pos = 0
        tok = None
        for t in prompt:
            tok, logits = self.step(int(t))
        out, self.logits_trace = [tok], [logits]     # logits_trace[i] are the logits that picked out[i]
        for _ in range(n_new - 1):
            tok, logits = self.step(tok)
            out.append(tok)
            self.logits_trace.append(logits)
        return out
