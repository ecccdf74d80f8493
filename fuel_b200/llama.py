"""Quantized LLaMA-architecture decode on top of the quantized mat-vec path (batch 1).

Model glue in the shape of the reference's (fuel-core/src/lazy.rs:7363-7447: RMSNorm -> q/k/v ->
rotate-half RoPE -> attention over an f32 KV cache -> o -> residual -> RMSNorm -> SwiGLU FFN ->
residual; greedy pick = last maximal index), every op one call into libfuelq.so.

Tensor parallelism, one process per GPU: every linear is split along its OUTPUT rows (whole weight
rows, no block is cut) and the pieces are put back with an all-gather; heads are split the same
way, so attention is local. Nothing is ever summed across ranks, which makes every value — and so
every greedy token — bit-identical for 1, 2, 4 or 8 GPUs by construction. The price is four small
all-gathers per layer instead of the usual two all-reduces.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from .ggml import GgmlDType as T

_L = _lib.lib


@dataclasses.dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    ffn_dim: int = 11008
    vocab: int = 32000
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq: int = 640

    @classmethod
    def llama2_7b(cls, max_seq: int = 640) -> "LlamaConfig":
        return cls(max_seq=max_seq)


def q4km_mix(name: str, layer: int) -> T:
    """Q4_K_M-style mix of BASELINE config 4: Q6_K for the output head and for attn_v / ffn_down in
    every other layer, Q4_K elsewhere (embeddings included)."""
    if name == "output":
        return T.Q6K
    if name in ("attn_v", "ffn_down") and layer % 2 == 0:
        return T.Q6K
    return T.Q4K


def rope_tables(cfg: LlamaConfig):
    """cos/sin [max_seq][head_dim], angles computed in f64; both halves of a row hold the same angles."""
    half = cfg.head_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (np.arange(half, dtype=np.float64) * 2.0 / cfg.head_dim))
    ang = np.arange(cfg.max_seq, dtype=np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1).astype(np.float32)
    sin = np.concatenate([np.sin(ang), np.sin(ang)], axis=1).astype(np.float32)
    return cos, sin


def init_weight(n: int, k: int, seed: int, device) -> torch.Tensor:
    """The same N(0, 0.02) tensor on every rank (seeded device generator), so that a rank's slice does
    not depend on how many ranks there are."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02


def _check(st: int, op: str) -> None:
    if st:
        _lib.check(st, op)


def _quantize(t: T, w: torch.Tensor) -> torch.Tensor:
    from . import ops
    return ops.quantize_weights(t, w.contiguous())


class _Linear:
    """Rows [r0, r1) of a quantized [n, k] weight, kept as GGUF blocks on the device."""

    def __init__(self, dtype: T, blocks: torch.Tensor, n: int, k: int):
        self.dtype, self.blocks, self.n, self.k = dtype, blocks, n, k

    def matvec_packed(self, packed: torch.Tensor, out: torch.Tensor, stream: int) -> None:
        _check(_L.fuelq_qmatmul_packed(int(self.dtype), 1, self.n, self.k, self.blocks.data_ptr(), packed.data_ptr(),
                                       out.data_ptr(), stream), "fuelq_qmatmul_packed")


class QLlama:
    def __init__(self, cfg: LlamaConfig, device: torch.device, rank: int = 0, world: int = 1, seed: int = 0,
                 mix=q4km_mix):
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.ffn_dim % world == 0
        assert cfg.dim % world == 0 and cfg.vocab % world == 0 and cfg.head_dim == 128
        self.cfg, self.device, self.rank, self.world = cfg, device, rank, world
        c, g, r = cfg, world, rank
        self.hl, self.kvl = c.n_heads // g, c.n_kv_heads // g
        qd, kvd = self.hl * c.head_dim, self.kvl * c.head_dim
        f32 = dict(dtype=torch.float32, device=device)

        def rows(w, lo, hi):
            return w[lo:hi]

        self.embed = _quantize(T.Q4K, init_weight(c.vocab, c.dim, seed * 100003 + 1, device))
        self.layers = []
        for li in range(c.n_layers):
            s0 = seed * 100003 + 1000 * (li + 1)
            wq = rows(init_weight(c.dim, c.dim, s0 + 1, device), r * qd, (r + 1) * qd)
            wk = rows(init_weight(c.n_kv_heads * c.head_dim, c.dim, s0 + 2, device), r * kvd, (r + 1) * kvd)
            wv = rows(init_weight(c.n_kv_heads * c.head_dim, c.dim, s0 + 3, device), r * kvd, (r + 1) * kvd)
            wo = rows(init_weight(c.dim, c.dim, s0 + 4, device), r * c.dim // g, (r + 1) * c.dim // g)
            wg = rows(init_weight(c.ffn_dim, c.dim, s0 + 5, device), r * c.ffn_dim // g, (r + 1) * c.ffn_dim // g)
            wu = rows(init_weight(c.ffn_dim, c.dim, s0 + 6, device), r * c.ffn_dim // g, (r + 1) * c.ffn_dim // g)
            wd = rows(init_weight(c.dim, c.ffn_dim, s0 + 7, device), r * c.dim // g, (r + 1) * c.dim // g)
            tq, tv, to, tg, td = (mix("attn_q", li), mix("attn_v", li), mix("attn_output", li), mix("ffn_gate", li),
                                  mix("ffn_down", li))
            self.layers.append(dict(
                qk=_Linear(tq, _quantize(tq, torch.cat([wq, wk])), qd + kvd, c.dim),
                v=_Linear(tv, _quantize(tv, wv), kvd, c.dim),
                o=_Linear(to, _quantize(to, wo), c.dim // g, c.dim),
                gu=_Linear(tg, _quantize(tg, torch.cat([wg, wu])), 2 * c.ffn_dim // g, c.dim),
                down=_Linear(td, _quantize(td, wd), c.dim // g, c.ffn_dim),
                attn_norm=torch.ones(c.dim, **f32), ffn_norm=torch.ones(c.dim, **f32),
                kc=torch.zeros(self.kvl, c.max_seq, c.head_dim, **f32),
                vc=torch.zeros(self.kvl, c.max_seq, c.head_dim, **f32)))
            del wq, wk, wv, wo, wg, wu, wd
        th = mix("output", -1)
        wout = rows(init_weight(c.vocab, c.dim, seed * 100003 + 2, device), r * c.vocab // g, (r + 1) * c.vocab // g)
        self.head = _Linear(th, _quantize(th, wout), c.vocab // g, c.dim)
        del wout
        self.out_norm = torch.ones(c.dim, **f32)
        cos, sin = rope_tables(c)
        self.cos, self.sin = torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)

        # step buffers
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.next_token = torch.zeros(1, dtype=torch.int32, device=device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.x = torch.zeros(c.dim, **f32)
        self.h = torch.zeros(c.dim, **f32)
        self.qk = torch.zeros(qd + kvd, **f32)
        self.v = torch.zeros(kvd, **f32)
        self.attn_l = torch.zeros(qd, **f32)
        self.o_l = torch.zeros(c.dim // g, **f32)
        self.gu = torch.zeros(2 * c.ffn_dim // g, **f32)
        self.s_l = torch.zeros(c.ffn_dim // g, **f32)
        self.d_l = torch.zeros(c.dim // g, **f32)
        self.logits_l = torch.zeros(c.vocab // g, **f32)
        if g > 1:
            self.attn = torch.zeros(c.dim, **f32)
            self.o = torch.zeros(c.dim, **f32)
            self.s = torch.zeros(c.ffn_dim, **f32)
            self.d = torch.zeros(c.dim, **f32)
            self.logits = torch.zeros(c.vocab, **f32)
        else:
            self.attn, self.o, self.s, self.d, self.logits = self.attn_l, self.o_l, self.s_l, self.d_l, self.logits_l
        nb = max(_L.fuelq_act_packed_bytes(int(T.Q4K), 1, c.dim), _L.fuelq_act_packed_bytes(int(T.Q4K), 1, c.ffn_dim))
        self.packed = torch.zeros(nb, dtype=torch.uint8, device=device)
        self.attn_ws = torch.zeros(max(_L.fuelq_attn_decode_workspace_bytes(self.hl), 16), dtype=torch.uint8, device=device)
        self.graph = None
        self.fused = True  # single-GPU step uses the fused producers
        self.weight_bytes = (sum(l[k].blocks.numel() for l in self.layers for k in ("qk", "v", "o", "gu", "down"))
                             + self.head.blocks.numel())

    # ---- one decode step: token, pos -> next_token; pos += 1; token = next_token
    def _gather(self, full: torch.Tensor, local: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_gather_into_tensor(full, local)

    def _quant(self, x: torch.Tensor, k: int, stream: int) -> None:
        _check(_L.fuelq_quantize_act_packed(int(T.Q4K), 1, k, x.data_ptr(), self.packed.data_ptr(), self.packed.numel(),
                                            stream), "fuelq_quantize_act_packed")

    def step(self) -> None:
        if self.world == 1 and self.fused:
            return self._step_fused()
        return self._step_plain()

    def _step_fused(self) -> None:
        """Single-GPU step: norm / attention merge / SwiGLU write the quantized activations directly."""
        c = self.cfg
        st = torch.cuda.current_stream().cuda_stream
        scale = 1.0 / math.sqrt(c.head_dim)
        pk, pkn = self.packed.data_ptr(), self.packed.numel()
        _check(_L.fuelq_embed_rows(int(T.Q4K), self.embed.data_ptr(), c.dim, self.token.data_ptr(), 1, self.x.data_ptr(), st),
               "fuelq_embed_rows")
        delta = None
        qd = self.hl * c.head_dim
        for l in self.layers:
            _check(_L.fuelq_add_rmsnorm_q8k(self.x.data_ptr(), delta, l["attn_norm"].data_ptr(), c.dim, c.norm_eps, pk, pkn, st),
                   "add_rmsnorm_q8k")
            l["qk"].matvec_packed(self.packed, self.qk, st)
            l["v"].matvec_packed(self.packed, self.v, st)
            _check(_L.fuelq_rope_store(self.qk.data_ptr(), self.qk.data_ptr() + 4 * qd, self.v.data_ptr(), l["kc"].data_ptr(),
                                       l["vc"].data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                       self.hl, self.kvl, c.head_dim, c.max_seq, st), "rope_store")
            _check(_L.fuelq_attn_decode_q8k(self.qk.data_ptr(), l["kc"].data_ptr(), l["vc"].data_ptr(), self.pos.data_ptr(),
                                            self.hl, self.kvl, c.head_dim, c.max_seq, scale, self.attn_ws.data_ptr(),
                                            self.attn_ws.numel(), pk, pkn, st), "attn_decode_q8k")
            l["o"].matvec_packed(self.packed, self.o_l, st)
            _check(_L.fuelq_add_rmsnorm_q8k(self.x.data_ptr(), self.o_l.data_ptr(), l["ffn_norm"].data_ptr(), c.dim, c.norm_eps,
                                            pk, pkn, st), "add_rmsnorm_q8k")
            l["gu"].matvec_packed(self.packed, self.gu, st)
            _check(_L.fuelq_swiglu_q8k(self.gu.data_ptr(), self.gu.data_ptr() + 4 * c.ffn_dim, c.ffn_dim, pk, pkn, st), "swiglu_q8k")
            l["down"].matvec_packed(self.packed, self.d_l, st)
            delta = self.d_l.data_ptr()
        _check(_L.fuelq_add_rmsnorm_q8k(self.x.data_ptr(), delta, self.out_norm.data_ptr(), c.dim, c.norm_eps, pk, pkn, st),
               "add_rmsnorm_q8k")
        self.head.matvec_packed(self.packed, self.logits_l, st)
        _check(_L.fuelq_argmax_last(self.logits.data_ptr(), c.vocab, self.next_token.data_ptr(), st), "argmax_last")
        self.pos.add_(1)
        self.token.copy_(self.next_token)

    def _step_plain(self) -> None:
        c = self.cfg
        st = torch.cuda.current_stream().cuda_stream
        scale = 1.0 / math.sqrt(c.head_dim)
        _check(_L.fuelq_embed_rows(int(T.Q4K), self.embed.data_ptr(), c.dim, self.token.data_ptr(), 1, self.x.data_ptr(), st),
               "fuelq_embed_rows")
        delta = None
        for l in self.layers:
            _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                        l["attn_norm"].data_ptr(), self.h.data_ptr(), 1, c.dim, c.norm_eps, st), "add_rmsnorm")
            self._quant(self.h, c.dim, st)
            l["qk"].matvec_packed(self.packed, self.qk, st)
            l["v"].matvec_packed(self.packed, self.v, st)
            qd = self.hl * c.head_dim
            _check(_L.fuelq_rope_store(self.qk.data_ptr(), self.qk.data_ptr() + 4 * qd, self.v.data_ptr(), l["kc"].data_ptr(),
                                       l["vc"].data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                       self.hl, self.kvl, c.head_dim, c.max_seq, st), "rope_store")
            _check(_L.fuelq_attn_decode(self.qk.data_ptr(), l["kc"].data_ptr(), l["vc"].data_ptr(), self.attn_l.data_ptr(),
                                        self.pos.data_ptr(), self.hl, self.kvl, c.head_dim, c.max_seq, scale, self.attn_ws.data_ptr(),
                                        self.attn_ws.numel(), st), "attn_decode")
            self._gather(self.attn, self.attn_l)
            self._quant(self.attn, c.dim, st)
            l["o"].matvec_packed(self.packed, self.o_l, st)
            self._gather(self.o, self.o_l)
            _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), self.o.data_ptr(), l["ffn_norm"].data_ptr(), self.h.data_ptr(), 1,
                                        c.dim, c.norm_eps, st), "add_rmsnorm")
            self._quant(self.h, c.dim, st)
            l["gu"].matvec_packed(self.packed, self.gu, st)
            fl = c.ffn_dim // self.world
            _check(_L.fuelq_swiglu(self.gu.data_ptr(), self.gu.data_ptr() + 4 * fl, self.s_l.data_ptr(), fl, st), "swiglu")
            self._gather(self.s, self.s_l)
            self._quant(self.s, c.ffn_dim, st)
            l["down"].matvec_packed(self.packed, self.d_l, st)
            self._gather(self.d, self.d_l)
            delta = self.d
        _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), delta.data_ptr(), self.out_norm.data_ptr(), self.h.data_ptr(), 1, c.dim,
                                    c.norm_eps, st), "add_rmsnorm")
        self._quant(self.h, c.dim, st)
        self.head.matvec_packed(self.packed, self.logits_l, st)
        self._gather(self.logits, self.logits_l)
        _check(_L.fuelq_argmax_last(self.logits.data_ptr(), c.vocab, self.next_token.data_ptr(), st), "argmax_last")
        self.pos.add_(1)
        self.token.copy_(self.next_token)

    def capture(self) -> None:
        """Capture one step into a CUDA graph (after one eager step so every kernel attribute is set)."""
        saved = (self.token.clone(), self.pos.clone())
        self.step()
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.step()
        torch.cuda.synchronize()
        self.token.copy_(saved[0])
        self.pos.copy_(saved[1])

    def run_step(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()

    def reset(self) -> None:
        self.pos.zero_()
        for l in self.layers:
            l["kc"].zero_()
            l["vc"].zero_()

    def generate(self, prompt_ids, n_new: int):
        """Feed the prompt one token at a time (the same M = 1 path as decoding, so the KV cache and every
        logit are independent of GPU count), then greedy-decode n_new tokens. Returns them as a list."""
        self.reset()
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int32, device=self.device)
        assert len(prompt) + n_new <= self.cfg.max_seq
        for i in range(len(prompt)):
            self.token.copy_(prompt[i:i + 1])
            self.run_step()
        out = [self.next_token.clone()]
        for _ in range(n_new - 1):
            self.run_step()
            out.append(self.next_token.clone())
        return torch.cat(out).cpu().tolist()
