"""Quantized LLaMA-architecture decode on top of the quantized mat-vec path (batch 1).

Model glue in the shape of the reference's (fuel-core/src/lazy.rs:7363-7447: RMSNorm -> q/k/v ->
rotate-half RoPE -> attention over an f32 KV cache -> o -> residual -> RMSNorm -> SwiGLU FFN ->
residual; greedy pick = last maximal index), every op one call into libfuelq.so.

Tensor parallelism, one process per GPU, split as the reference's fuel-parallel does
(fuel-parallel/src/tensor_parallel.rs:283-343): q/k/v, gate/up and the output head are COLUMN-parallel (a rank
holds whole weight rows: its heads, its FFN channels, its slice of the vocabulary), o and down are ROW-parallel
(a rank holds its k columns of every row, the columns its own attention heads / FFN channels feed) and their
partial results are summed across ranks — one exchange per row-parallel layer, two per transformer layer.

That sum follows one fixed tree at every GPU count, so every value — and every greedy token — has the same
bits on 1, 2, 4 or 8 GPUs: the k axis of a row-parallel layer is cut into eight leaves of whole 256-blocks
(leaf_split), a rank owns an aligned group of 8 / world leaves, its mat-vec sums its leaves pairwise
(fuelq_qmatmul_packed_tree), and the consumer adds the ranks' vectors pairwise in rank order
(fuelq_add_rmsnorm_q8k_peer / _parts). One GPU runs the same tree over all eight leaves.

Two ways to move the partial vectors: comm="nccl" all-gathers them with the library between the kernels (the
baseline), comm="peer" has the mat-vec kernel store its vector straight into every GPU's buffer over NVLink
as stamped pairs, and the consuming norm kernel polls its own buffer (include/fuelq.h, fuelq_*_peer).
"""
from __future__ import annotations

import dataclasses
import gc
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
    """Q4_K_M-style mix of the 7B-architecture benchmark workload: Q6_K for the output head and for attn_v / ffn_down in
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


def shard_range(total: int, world: int, rank: int, unit: int = 1):
    """Rows [lo, hi) of `total` owned by `rank`: whole `unit`s, the first total/unit % world ranks get one more."""
    assert total % unit == 0
    blocks = total // unit
    q, rem = divmod(blocks, world)
    lo = rank * q + min(rank, rem)
    return lo * unit, (lo + q + (1 if rank < rem else 0)) * unit


def leaf_split(n_blocks: int) -> list:
    """The eight leaves of a row-parallel layer's k axis, in 256-element blocks: halve, floor on the left,
    three times (43 -> 21 | 22 -> 10, 11 | 11, 11 -> 5,5, 5,6, 5,6, 5,6). Leaves may be empty for a short axis."""
    def rec(n, depth):
        return [n] if depth == 0 else rec(n // 2, depth - 1) + rec(n - n // 2, depth - 1)
    return rec(n_blocks, 3)


def rank_leaves(n_blocks: int, world: int, rank: int):
    """(first block, list of leaf sizes) of the aligned group of 8 / world leaves that `rank` owns."""
    assert world in (1, 2, 4, 8)
    leaves = leaf_split(n_blocks)
    per = 8 // world
    return sum(leaves[:rank * per]), leaves[rank * per:(rank + 1) * per]


class _RawCuda:
    """A device range owned elsewhere, for torch.as_tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerRegion:
    """One zeroed device allocation per rank that the other ranks of the node map: the exchange flags and the
    destination buffers. `base[q]` is rank q's region as addressed from this process."""

    def __init__(self, sizes: dict, device: torch.device, rank: int, world: int):
        import ctypes
        self.rank, self.world = rank, world
        self.off, total = {}, 0
        for name, nbytes in sizes.items():
            self.off[name] = total
            total += _align(nbytes)
        self.nbytes = total
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _check(_L.fuelq_ipc_alloc(total, ctypes.byref(own), handle), "fuelq_ipc_alloc")
        self.own = own.value
        self.base = [None] * world
        self.base[rank] = self.own
        self.opened = []
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw)
            for q in range(world):
                if q == rank:
                    continue
                ptr = ctypes.c_void_p()
                _check(_L.fuelq_ipc_open(handles[q], ctypes.byref(ptr)), "fuelq_ipc_open")
                self.base[q] = ptr.value
                self.opened.append(ptr.value)
            dist.barrier()
        self.bytes_view = torch.as_tensor(_RawCuda(self.own, total), device=device)

    def ptrs(self, name: str, extra: int = 0):
        """ctypes array of `name`'s address on every rank (+ extra bytes)."""
        import ctypes
        arr = (ctypes.c_void_p * _lib.PEER_MAX_WORLD)()
        for q in range(self.world):
            arr[q] = self.base[q] + self.off[name] + extra
        return arr

    def view(self, name: str, nbytes: int, dtype) -> torch.Tensor:
        return self.bytes_view[self.off[name]: self.off[name] + nbytes].view(dtype)

    def close(self) -> None:
        """After every rank has finished its last step (callers synchronize and barrier first)."""
        if self.own is None:
            return
        self.bytes_view = None
        for ptr in self.opened:
            _L.fuelq_ipc_close(ptr)
        self.opened = []
        if self.world > 1:
            dist.barrier()
        _L.fuelq_ipc_free(self.own)
        self.own = None


def _check(st: int, op: str) -> None:
    if st:
        _lib.check(st, op)


def _quantize(t: T, w: torch.Tensor) -> torch.Tensor:
    from . import ops
    return ops.quantize_weights(t, w.contiguous())


_SEED_SLOT = {"attn_q": 1, "attn_k": 2, "attn_v": 3, "attn_output": 4, "ffn_gate": 5, "ffn_up": 6, "ffn_down": 7}
_K_QUANTS = (T.Q2K, T.Q3K, T.Q4K, T.Q5K, T.Q6K)  # their activations are Q8_K blocks


def _act_kind(t: T) -> T:
    """The activation block format a weight format takes (GgmlType::VecDotType in the reference)."""
    return T.Q8K if t in _K_QUANTS else T.Q8_1 if t in (T.Q4_1, T.Q5_1) else T.Q8_0


class SyntheticWeights:
    """Random-init N(0, 0.02) weights quantized on the device in a given format mix; norm gains are ones."""

    def __init__(self, cfg: LlamaConfig, device: torch.device, seed: int = 0, mix=q4km_mix):
        self.cfg, self.device, self.seed, self.mix = cfg, device, seed, mix

    def _shape(self, name: str):
        c = self.cfg
        kv = c.n_kv_heads * c.head_dim
        return {"attn_q": (c.dim, c.dim), "attn_k": (kv, c.dim), "attn_v": (kv, c.dim), "attn_output": (c.dim, c.dim),
                "ffn_gate": (c.ffn_dim, c.dim), "ffn_up": (c.ffn_dim, c.dim), "ffn_down": (c.dim, c.ffn_dim),
                "output": (c.vocab, c.dim), "token_embd": (c.vocab, c.dim)}[name]

    def _seed(self, name: str, layer: int) -> int:
        if name == "token_embd":
            return self.seed * 100003 + 1
        if name == "output":
            return self.seed * 100003 + 2
        return self.seed * 100003 + 1000 * (layer + 1) + _SEED_SLOT[name]

    def dtype(self, name: str, layer: int) -> T:
        return T.Q4K if name == "token_embd" else self.mix(name, layer)

    def rows(self, name: str, layer: int, lo: int, hi: int) -> torch.Tensor:
        """GGUF blocks of rows [lo, hi) of a linear's [n_out, k_in] weight (rows are quantized independently, so a
        slice of the quantized matrix is the quantized slice)."""
        n, k = self._shape(name)
        return _quantize(self.dtype(name, layer), init_weight(n, k, self._seed(name, layer), self.device)[lo:hi])

    def embedding(self):
        return T.Q4K, self.rows("token_embd", -1, 0, self.cfg.vocab)

    def norm(self, name: str, layer: int) -> torch.Tensor:
        return torch.ones(self.cfg.dim, dtype=torch.float32, device=self.device)

    def export_gguf(self, path, version: int = 3) -> None:
        """Write the whole model as a GGUF file with the llama.cpp tensor names the reference's loader reads
        (fuel-core/src/lazy_quantized_llama.rs:224-236)."""
        from . import gguf as G
        c = self.cfg
        meta = [("general.architecture", G.STRING, "llama"), ("llama.block_count", G.U32, c.n_layers),
                ("llama.embedding_length", G.U32, c.dim), ("llama.feed_forward_length", G.U32, c.ffn_dim),
                ("llama.attention.head_count", G.U32, c.n_heads), ("llama.attention.head_count_kv", G.U32, c.n_kv_heads),
                ("llama.attention.layer_norm_rms_epsilon", G.F32, c.norm_eps), ("llama.rope.freq_base", G.F32, c.rope_theta),
                ("llama.rope.dimension_count", G.U32, c.head_dim), ("llama.vocab_size", G.U32, c.vocab)]
        tensors = []

        def lin(fname, name, layer):
            n, k = self._shape(name)
            tensors.append((fname, self.dtype(name, layer), (n, k), self.rows(name, layer, 0, n).cpu().numpy()))

        def vec(fname, name, layer):
            tensors.append((fname, T.F32, (c.dim,), self.norm(name, layer).cpu().numpy().view(np.uint8)))

        lin("token_embd.weight", "token_embd", -1)
        for li in range(c.n_layers):
            for name in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"):
                lin(f"blk.{li}.{name}.weight", name, li)
            vec(f"blk.{li}.attn_norm.weight", "attn_norm", li)
            vec(f"blk.{li}.ffn_norm.weight", "ffn_norm", li)
        vec("output_norm.weight", "output_norm", -1)
        lin("output.weight", "output", -1)
        G.write_gguf(path, meta, tensors, version=version)


class GgufWeights:
    """Weights of a GGUF checkpoint with llama.cpp's LLaMA tensor names, as the reference's loader takes them
    (fuel-core/src/lazy_quantized_llama.rs:224-330): linears stay in the file's block format — each rank copies just
    its rows from the mapping to its GPU —, norm gains and the embedding table become f32; `output.weight` falls
    back to `token_embd.weight` (tied embeddings) when absent."""

    LINEAR_FORMATS = (T.Q4K, T.Q5K, T.Q6K, T.Q8_0, T.Q4_0, T.Q4_1, T.Q5_0, T.Q5_1, T.Q2K, T.Q3K)

    def __init__(self, path, device: torch.device):
        from .gguf import GgufFile
        self.file, self.device = GgufFile(path), device

    def _fname(self, name: str, layer: int) -> str:
        if name in ("token_embd", "output_norm"):
            return f"{name}.weight"
        if name == "output":
            return "output.weight" if "output.weight" in self.file.tensor_infos else "token_embd.weight"
        return f"blk.{layer}.{name}.weight"

    def config(self, max_seq: int = 640) -> LlamaConfig:
        """Architecture from the `llama.*` metadata keys and the tensor shapes."""
        m, ti = self.file.metadata, self.file.tensor_infos
        arch = m.get("general.architecture", "llama")
        if arch != "llama":
            raise ValueError(f"gguf: architecture {arch!r} is not the LLaMA layout")
        vocab, dim = self.file.tensor_info("token_embd.weight").shape
        n_heads = int(m["llama.attention.head_count"])
        layers = int(m["llama.block_count"])
        return LlamaConfig(dim=dim, n_layers=layers, n_heads=n_heads,
                           n_kv_heads=int(m.get("llama.attention.head_count_kv", n_heads)), head_dim=dim // n_heads,
                           ffn_dim=ti["blk.0.ffn_gate.weight"].shape[0], vocab=vocab,
                           norm_eps=float(m.get("llama.attention.layer_norm_rms_epsilon", 1e-5)),
                           rope_theta=float(m.get("llama.rope.freq_base", 10000.0)), max_seq=max_seq)

    def check(self, cfg: LlamaConfig) -> None:
        """Element counts as the reference checks them (lazy_quantized_llama.rs:271-277, 288-293)."""
        kv = cfg.n_kv_heads * cfg.head_dim
        want = {"attn_q": cfg.dim * cfg.dim, "attn_k": kv * cfg.dim, "attn_v": kv * cfg.dim, "attn_output": cfg.dim * cfg.dim,
                "ffn_gate": cfg.ffn_dim * cfg.dim, "ffn_up": cfg.ffn_dim * cfg.dim, "ffn_down": cfg.dim * cfg.ffn_dim}
        for li in range(cfg.n_layers):
            for name, n in want.items():
                info = self.file.tensor_info(self._fname(name, li))
                if info.elem_count() != n:
                    raise ValueError(f"gguf: tensor {self._fname(name, li)!r} has {info.elem_count()} elements, expected {n}")
        if self.file.tensor_info("token_embd.weight").elem_count() != cfg.vocab * cfg.dim:
            raise ValueError("gguf token_embd.weight: wrong element count")

    def dtype(self, name: str, layer: int) -> T:
        t = self.file.tensor_info(self._fname(name, layer)).ggml_dtype
        if t not in self.LINEAR_FORMATS:
            raise NotImplementedError(f"gguf: {self._fname(name, layer)!r} is {t.name}; the quantized mat-vec takes "
                                      + ", ".join(x.name for x in self.LINEAR_FORMATS))
        return t

    def rows(self, name: str, layer: int, lo: int, hi: int) -> torch.Tensor:
        self.dtype(name, layer)
        return self.file.load(self._fname(name, layer), self.device, lo, hi)

    def embedding(self):
        return T.F32, self.file.load_f32("token_embd.weight", self.device).contiguous()

    def norm(self, name: str, layer: int) -> torch.Tensor:
        return self.file.load_f32(self._fname(name, layer), self.device).contiguous()


class _Linear:
    """Rows [r0, r1) of a quantized [n, k] weight, kept as GGUF blocks on the device."""

    def __init__(self, dtype: T, blocks: torch.Tensor, n: int, k: int):
        self.dtype, self.blocks, self.n, self.k = dtype, blocks, n, k

    def matvec_packed(self, packed: torch.Tensor, out: torch.Tensor, stream: int) -> None:
        _check(_L.fuelq_qmatmul_packed(int(self.dtype), 1, self.n, self.k, self.blocks.data_ptr(), packed.data_ptr(),
                                       out.data_ptr(), stream), "fuelq_qmatmul_packed")


class _RowParallel(_Linear):
    """This rank's k columns [first_block * 256, ...) of every row of a quantized [n, k_total] weight, repacked
    contiguous, with the sizes of the leaves it covers (row-parallel layer; summed by the fixed tree)."""

    def __init__(self, dtype: T, full_rows: torch.Tensor, n: int, k_total: int, first_block: int, leaves):
        import ctypes
        bb = dtype.type_size()
        nb = sum(leaves)
        slab = full_rows.view(n, k_total // 256, bb)[:, first_block:first_block + nb].contiguous().view(-1)
        super().__init__(dtype, slab, n, nb * 256)
        self.n_leaves = len(leaves)
        self.leaves = (ctypes.c_int32 * 8)(*leaves)

    def matvec_tree(self, packed: torch.Tensor, out: torch.Tensor, stream: int) -> None:
        _check(_L.fuelq_qmatmul_packed_tree(int(self.dtype), self.n, self.k, self.blocks.data_ptr(), packed.data_ptr(),
                                            out.data_ptr(), self.n_leaves, self.leaves, stream), "fuelq_qmatmul_packed_tree")

    def matvec_tree_peer(self, packed: torch.Tensor, dst, dst_offset: int, peers_ref, push_seq: int, stream: int) -> None:
        _check(_L.fuelq_qmatmul_packed_tree_peer(int(self.dtype), self.n, self.k, self.blocks.data_ptr(), packed.data_ptr(),
                                                 dst, dst_offset, peers_ref, push_seq, self.n_leaves, self.leaves, stream),
               "fuelq_qmatmul_packed_tree_peer")


class QLlama:
    def __init__(self, cfg: LlamaConfig, device: torch.device, rank: int = 0, world: int = 1, seed: int = 0,
                 mix=q4km_mix, comm: str = "nccl", weights=None):
        """`weights`: a weight source (GgufWeights, SyntheticWeights); default: synthetic from `seed` and `mix`."""
        assert comm in ("nccl", "peer")
        assert world in (1, 2, 4, 8)
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0
        assert cfg.dim % 256 == 0 and cfg.ffn_dim % 256 == 0 and cfg.vocab % world == 0 and cfg.head_dim == 128
        self.cfg, self.device, self.rank, self.world, self.comm = cfg, device, rank, world, comm
        c, g, r = cfg, world, rank
        self.hl, self.kvl = c.n_heads // g, c.n_kv_heads // g
        qd, kvd = self.hl * c.head_dim, self.kvl * c.head_dim
        # row-parallel layers: this rank's leaves of the k axis. o's columns are the outputs of this rank's heads,
        # down's are this rank's FFN channels (so gate/up are cut at the same channels)
        o_b0, o_leaves = rank_leaves(c.n_heads * c.head_dim // 256, g, r)
        d_b0, d_leaves = rank_leaves(c.ffn_dim // 256, g, r)
        assert o_b0 * 256 == r * qd and sum(o_leaves) * 256 == qd, "the heads of a rank must cover whole leaves of o's k axis"
        self.f_lo, self.f_hi = d_b0 * 256, (d_b0 + sum(d_leaves)) * 256
        fl = self.f_hi - self.f_lo
        assert g == 1 or (fl > 0 and qd % 256 == 0), "every rank needs FFN channels and whole activation blocks"
        f32 = dict(dtype=torch.float32, device=device)

        src = weights if weights is not None else SyntheticWeights(cfg, device, seed, mix)
        self.embed_dtype, self.embed = src.embedding()
        k_quants_only = True
        tree_ok = True

        def lin(names, li, lo_hi, k):
            """One _Linear over the stacked rows of `names` (all the same format), each cut to its [lo, hi)."""
            t = src.dtype(names[0], li)
            parts = [src.rows(nm, li, lo, hi) for nm, (lo, hi) in zip(names, lo_hi)]
            return _Linear(t, parts[0] if len(parts) == 1 else torch.cat(parts), sum(hi - lo for lo, hi in lo_hi), k)

        def rowpar(name, li, k_total, b0, leaves):
            t = src.dtype(name, li)
            if t not in (T.Q4K, T.Q6K):   # no tree form: the whole matrix, plain mat-vec (one GPU only)
                return lin((name,), li, ((0, c.dim),), k_total)
            return _RowParallel(t, src.rows(name, li, 0, c.dim), c.dim, k_total, b0, leaves)

        q_rng, kv_rng, f_rng = (r * qd, (r + 1) * qd), (r * kvd, (r + 1) * kvd), (self.f_lo, self.f_hi)
        self.layers = []
        for li in range(c.n_layers):
            tq, tk, tv = src.dtype("attn_q", li), src.dtype("attn_k", li), src.dtype("attn_v", li)
            assert tq == tk and src.dtype("ffn_gate", li) == src.dtype("ffn_up", li), "q/k and gate/up are stacked: one format each"
            # q, k (and v, where it has the same format) are one stacked matrix: one launch instead of two or three
            stacked_v = tv == tq
            layer = dict(
                qk=lin(("attn_q", "attn_k", "attn_v") if stacked_v else ("attn_q", "attn_k"), li,
                       (q_rng, kv_rng, kv_rng) if stacked_v else (q_rng, kv_rng), c.dim),
                v=None if stacked_v else lin(("attn_v",), li, (kv_rng,), c.dim),
                o=rowpar("attn_output", li, c.n_heads * c.head_dim, o_b0, o_leaves),
                gu=lin(("ffn_gate", "ffn_up"), li, (f_rng, f_rng), c.dim),
                down=rowpar("ffn_down", li, c.ffn_dim, d_b0, d_leaves),
                attn_norm=src.norm("attn_norm", li), ffn_norm=src.norm("ffn_norm", li),
                kc=torch.zeros(self.kvl, c.max_seq, c.head_dim, **f32),
                vc=torch.zeros(self.kvl, c.max_seq, c.head_dim, **f32))
            k_quants_only &= all(layer[nm] is None or layer[nm].dtype in _K_QUANTS for nm in ("qk", "v", "o", "gu", "down"))
            tree_ok &= isinstance(layer["o"], _RowParallel) and isinstance(layer["down"], _RowParallel)
            self.layers.append(layer)
        self.head = lin(("output",), -1, ((r * c.vocab // g, (r + 1) * c.vocab // g),), c.dim)
        k_quants_only &= self.head.dtype in _K_QUANTS
        self.out_norm = src.norm("output_norm", -1)
        cos, sin = rope_tables(c)
        self.cos, self.sin = torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)

        # step buffers
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.next_token = torch.zeros(1, dtype=torch.int32, device=device)
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.x = torch.zeros(c.dim, **f32)
        self.h = torch.zeros(c.dim, **f32)
        self.qkv = torch.zeros(qd + 2 * kvd, **f32)   # q | k | v of the current token
        self.qk = self.qkv[:qd + kvd]
        self.v = self.qkv[qd + kvd:]
        self.attn_l = torch.zeros(qd, **f32)
        self.gu = torch.zeros(2 * fl, **f32)
        self.s_l = torch.zeros(fl, **f32)
        self.part = torch.zeros(c.dim, **f32)            # this rank's partial result of a row-parallel layer
        self.parts = torch.zeros(g, c.dim, **f32) if g > 1 else self.part.view(1, c.dim)   # every rank's, in rank order
        self.logits_l = torch.zeros(c.vocab // g, **f32)
        self._logits = torch.zeros(c.vocab, **f32) if g > 1 else self.logits_l
        nb = max(_L.fuelq_act_packed_bytes(int(t), 1, k) for t in (T.Q4K, T.Q8_0, T.Q4_1) for k in (c.dim, c.ffn_dim))
        self.packed = torch.zeros(nb, dtype=torch.uint8, device=device)
        self.attn_ws = torch.zeros(max(_L.fuelq_attn_decode_workspace_bytes(self.hl), 16), dtype=torch.uint8, device=device)
        # per layer: what the attention call needs to rotate q/k itself and append k, v to that layer's caches
        import ctypes
        self.ropes = []
        for l in self.layers:
            rp = _lib.Rope()
            rp.k, rp.v = self.qkv.data_ptr() + 4 * qd, self.qkv.data_ptr() + 4 * (qd + kvd)
            rp.cos_table, rp.sin_table = self.cos.data_ptr(), self.sin.data_ptr()
            rp.kcache, rp.vcache = l["kc"].data_ptr(), l["vc"].data_ptr()
            self.ropes.append(rp)
        self.rope_refs = [ctypes.byref(rp) for rp in self.ropes]
        self.peer = None
        self.graph = None
        # The fused producers write Q8_K activation blocks, which is what k-quant weights take; a model with other
        # linears runs the plain step on one GPU. The tree-ordered row-parallel mat-vec exists for Q4_K / Q6_K: a
        # k-quant model whose o / down have another format (Q5_K) runs the fused step on one GPU with plain mat-vecs there.
        self.fused = k_quants_only and (tree_ok or g == 1)
        if g > 1 and not self.fused:
            raise NotImplementedError("tensor parallelism needs k-quant linears with Q4_K / Q6_K o and down projections")
        if comm == "peer" and self.fused and tree_ok:
            self._init_peer()
        self.weight_bytes = (sum(l[k].blocks.numel() for l in self.layers for k in ("qk", "v", "o", "gu", "down") if l[k] is not None)
                             + self.head.blocks.numel())

    @classmethod
    def from_gguf(cls, path, device: torch.device, rank: int = 0, world: int = 1, comm: str = "nccl", max_seq: int = 640,
                  cfg: LlamaConfig | None = None) -> "QLlama":
        """Load a GGUF checkpoint (the reference's `from_gguf`, fuel-core/src/lazy_quantized_llama.rs:241-330). The
        architecture comes from the file's metadata unless `cfg` is given, as the reference's caller gives it."""
        w = GgufWeights(path, device)
        cfg = cfg or w.config(max_seq)
        w.check(cfg)
        model = cls(cfg, device, rank, world, comm=comm, weights=w)
        w.file.close()
        return model

    # ---- one decode step: token, pos -> next_token; pos += 1; token = next_token
    def _quant(self, x: torch.Tensor, k: int, stream: int, dtype: T = T.Q4K) -> None:
        """Activation blocks for a consumer of weight format `dtype` (Q8_K for k-quants, Q8_0 for Q8_0 / Q4_0)."""
        _check(_L.fuelq_quantize_act_packed(int(dtype), 1, k, x.data_ptr(), self.packed.data_ptr(), self.packed.numel(),
                                            stream), "fuelq_quantize_act_packed")

    def _mv(self, lins, outs, x: torch.Tensor, k: int, stream: int) -> None:
        """Plain step: mat-vecs of the same vector x, re-quantizing only when the activation format changes."""
        fmt = None
        for lin, out in zip(lins, outs):
            if lin is None:
                continue
            want = _act_kind(lin.dtype)
            if want != fmt:
                self._quant(x, k, stream, lin.dtype)
                fmt = want
            lin.matvec_packed(self.packed, out, stream)

    def step(self) -> None:
        if self.peer is not None:
            return self._step_tp(True)
        if self.fused:
            return self._step_tp(False)
        return self._step_plain()

    # ---- in-kernel exchange over peer-mapped memory
    def _init_peer(self) -> None:
        import ctypes
        c, g, r = self.cfg, self.world, self.rank
        assert 2 * c.n_layers + 1 <= _lib.PEER_MAX_SEQ
        self.peer = PeerRegion({"o": _L.fuelq_peer_vec_bytes(g * c.dim), "d": _L.fuelq_peer_vec_bytes(g * c.dim),
                                "logits": _L.fuelq_peer_vec_bytes(c.vocab)}, self.device, r, g)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.peers = _lib.Peers()
        self.peers.world, self.peers.rank, self.peers.epoch = g, r, self.epoch.data_ptr()
        self.peers_ref = ctypes.byref(self.peers)
        self.dst_o, self.dst_d, self.dst_logits = self.peer.ptrs("o"), self.peer.ptrs("d"), self.peer.ptrs("logits")
        own = self.peer.own
        self.own_o, self.own_d = own + self.peer.off["o"], own + self.peer.off["d"]
        self.own_logits = own + self.peer.off["logits"]
        self.logits_pairs = self.peer.view("logits", 8 * c.vocab, torch.float32)  # {value, stamp} pairs

    @property
    def logits(self) -> torch.Tensor:
        if self.peer is not None:
            return self.logits_pairs[0::2]
        return self._logits

    @logits.setter
    def logits(self, t: torch.Tensor) -> None:
        self._logits = t

    def _step_tp(self, peer: bool) -> None:
        """The decode step of a k-quant model on any number of GPUs: column-parallel q/k/v, gate/up and head,
        row-parallel o and down summed by the fixed tree. `peer`: the partial vectors and the logits travel as
        stamped stores inside the kernels; otherwise through the library's all-gather (nothing travels on one GPU).
        Norm, attention merge and SwiGLU write the next mat-vec's quantized activations directly."""
        c, r, g = self.cfg, self.rank, self.world
        st = torch.cuda.current_stream().cuda_stream
        scale = 1.0 / math.sqrt(c.head_dim)
        pk, pkn = self.packed.data_ptr(), self.packed.numel()
        fl = self.f_hi - self.f_lo
        vl = c.vocab // g
        pr = self.peers_ref if peer else None

        def norm(delta_own, wait_seq, gain):
            """x += (sum of the ranks' partial vectors); packed = Q8_K(rmsnorm(x) * gain)"""
            if peer:
                _check(_L.fuelq_add_rmsnorm_q8k_peer(self.x.data_ptr(), delta_own, g, gain.data_ptr(), c.dim, c.norm_eps, pk, pkn,
                                                     pr, wait_seq, st), "add_rmsnorm_q8k_peer")
            elif delta_own is None:
                _check(_L.fuelq_add_rmsnorm_q8k(self.x.data_ptr(), None, gain.data_ptr(), c.dim, c.norm_eps, pk, pkn, st),
                       "add_rmsnorm_q8k")
            else:
                if g > 1:
                    dist.all_gather_into_tensor(self.parts.view(-1), self.part)
                _check(_L.fuelq_add_rmsnorm_q8k_parts(self.x.data_ptr(), self.parts.data_ptr(), g, gain.data_ptr(), c.dim,
                                                      c.norm_eps, pk, pkn, st), "add_rmsnorm_q8k_parts")

        def rowpar(lin, dst, seq):
            if peer:
                lin.matvec_tree_peer(self.packed, dst, r * c.dim, pr, seq, st)
            elif isinstance(lin, _RowParallel):
                lin.matvec_tree(self.packed, self.part, st)
            else:                       # one GPU, a format without the tree form
                lin.matvec_packed(self.packed, self.part, st)

        _check(_L.fuelq_embed_rows(int(self.embed_dtype), self.embed.data_ptr(), c.dim, self.token.data_ptr(), 1, self.x.data_ptr(), st),
               "fuelq_embed_rows")
        delta, wait = None, -1
        for li, l in enumerate(self.layers):
            norm(delta, wait, l["attn_norm"])
            l["qk"].matvec_packed(self.packed, self.qkv if l["v"] is None else self.qk, st)
            if l["v"] is not None:
                l["v"].matvec_packed(self.packed, self.v, st)
            _check(_L.fuelq_attn_decode_q8k(self.qk.data_ptr(), l["kc"].data_ptr(), l["vc"].data_ptr(), self.pos.data_ptr(),
                                            self.hl, self.kvl, c.head_dim, c.max_seq, scale, self.attn_ws.data_ptr(),
                                            self.attn_ws.numel(), pk, pkn, self.rope_refs[li], st), "attn_decode_q8k")
            rowpar(l["o"], self.dst_o if peer else None, 2 * li)
            norm(self.own_o if peer else self.part, 2 * li, l["ffn_norm"])
            l["gu"].matvec_packed(self.packed, self.gu, st)
            _check(_L.fuelq_swiglu_q8k(self.gu.data_ptr(), self.gu.data_ptr() + 4 * fl, fl, pk, pkn, st), "swiglu_q8k")
            rowpar(l["down"], self.dst_d if peer else None, 2 * li + 1)
            delta, wait = (self.own_d if peer else self.part), 2 * li + 1
        last = 2 * len(self.layers)
        norm(delta, wait, self.out_norm)
        h = self.head
        if peer:
            _check(_L.fuelq_qmatmul_packed_peer(int(h.dtype), c.dim, vl, h.blocks.data_ptr(), pk, self.dst_logits, r * vl, pr, last,
                                                st), "qmatmul_packed_peer")
            _check(_L.fuelq_argmax_last_peer(self.own_logits, c.vocab, self.next_token.data_ptr(), pr, last, self.epoch.data_ptr(),
                                             st), "argmax_last_peer")
        else:
            h.matvec_packed(self.packed, self.logits_l, st)
            if g > 1:
                dist.all_gather_into_tensor(self._logits, self.logits_l)
            _check(_L.fuelq_argmax_last(self._logits.data_ptr(), c.vocab, self.next_token.data_ptr(), st), "argmax_last")
        self.pos.add_(1)
        self.token.copy_(self.next_token)

    def _step_plain(self) -> None:
        """One GPU, any supported linear formats: every op its own call, activations quantized per consumer."""
        c = self.cfg
        st = torch.cuda.current_stream().cuda_stream
        scale = 1.0 / math.sqrt(c.head_dim)
        fl = c.ffn_dim
        _check(_L.fuelq_embed_rows(int(self.embed_dtype), self.embed.data_ptr(), c.dim, self.token.data_ptr(), 1, self.x.data_ptr(), st),
               "fuelq_embed_rows")
        delta = None
        for li, l in enumerate(self.layers):
            _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                        l["attn_norm"].data_ptr(), self.h.data_ptr(), 1, c.dim, c.norm_eps, st), "add_rmsnorm")
            self._mv((l["qk"], l["v"]), (self.qkv if l["v"] is None else self.qk, self.v), self.h, c.dim, st)
            _check(_L.fuelq_attn_decode(self.qk.data_ptr(), l["kc"].data_ptr(), l["vc"].data_ptr(), self.attn_l.data_ptr(),
                                        self.pos.data_ptr(), self.hl, self.kvl, c.head_dim, c.max_seq, scale, self.attn_ws.data_ptr(),
                                        self.attn_ws.numel(), self.rope_refs[li], st), "attn_decode")
            self._mv((l["o"],), (self.part,), self.attn_l, c.dim, st)
            _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), self.part.data_ptr(), l["ffn_norm"].data_ptr(), self.h.data_ptr(), 1,
                                        c.dim, c.norm_eps, st), "add_rmsnorm")
            self._mv((l["gu"],), (self.gu,), self.h, c.dim, st)
            _check(_L.fuelq_swiglu(self.gu.data_ptr(), self.gu.data_ptr() + 4 * fl, self.s_l.data_ptr(), fl, st), "swiglu")
            self._mv((l["down"],), (self.part,), self.s_l, c.ffn_dim, st)
            delta = self.part
        _check(_L.fuelq_add_rmsnorm(self.x.data_ptr(), delta.data_ptr(), self.out_norm.data_ptr(), self.h.data_ptr(), 1, c.dim,
                                    c.norm_eps, st), "add_rmsnorm")
        self._mv((self.head,), (self.logits_l,), self.h, c.dim, st)
        _check(_L.fuelq_argmax_last(self._logits.data_ptr(), c.vocab, self.next_token.data_ptr(), st), "argmax_last")
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

    def release(self) -> None:
        """Drop the captured graph. Must run before the process group is destroyed: tearing down NCCL while a
        graph that holds its kernels is alive stalls."""
        self.graph = None
        gc.collect()
        torch.cuda.synchronize()
        if self.peer is not None:
            keep = self.logits.clone()
            self.logits_pairs = None
            self.peer.close()
            self.peer = None
            self.logits = keep

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


def _main() -> None:
    """python -m fuel_b200.llama [--comm nccl|peer] [--steps N] [--pdl 0|1]: builds the 7B-architecture model on GPU 0,
    runs N eager decode steps and brackets the last one with cudaProfilerStart/Stop, so that a profiler started with
    --profile-from-start off lists exactly the kernels of one token."""
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--comm", default="nccl", choices=["nccl", "peer"])
    ap.add_argument("--steps", type=int, default=41)
    ap.add_argument("--pdl", type=int, default=0)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    _L.fuelq_set_option(_lib.OPT_PDL, args.pdl)
    model = QLlama(LlamaConfig.llama2_7b(), torch.device("cuda", 0), comm=args.comm)
    try:
        for _ in range(args.steps - 1):
            model.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        model.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print("next token", int(model.next_token.item()), "pos", int(model.pos.item()))
    finally:
        model.release()


if __name__ == "__main__":
    _main()
