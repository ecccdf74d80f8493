"""Mixture-of-experts block with GGUF-quantized experts on the decode path.

Mirrors the reference's sparse MoE forward (fuel-core/src/lazy_nn/moe.rs:92-127 router, :296-348 layer; each expert a
SwiGLU FFN down(silu(gate(x)) * up(x)), :130-215) with the experts' three matrices quantized (gate and up stacked as one
[2f, hidden] matrix per expert) and every expert product run as the grouped quantized mat-vec of libfuelq.so. One call of
forward() enqueues nine kernels on the current stream and never touches the host: routing, bucketing and row counts
stay on the device.
"""
from __future__ import annotations

import torch

from . import _lib
from .ggml import GgmlDType as T

_L = _lib.lib


def _check(st: int, op: str) -> None:
    if st:
        _lib.check(st, op)


class QMoeBlock:
    def __init__(self, n_experts: int, hidden: int, ffn: int, top_k: int, gate_up_blocks: torch.Tensor,
                 down_blocks: torch.Tensor, dtype: T = T.Q4K, max_tokens: int = 256, first_expert: int = 0,
                 n_experts_total: int | None = None):
        """gate_up_blocks: GGUF blocks of [n_experts][2*ffn][hidden] (rows 0..ffn gate, ffn..2*ffn up);
        down_blocks: blocks of [n_experts][hidden][ffn]. With first_expert / n_experts_total the block holds a
        contiguous range of a larger expert set (expert parallelism): routing still runs over all experts and
        pairs routed elsewhere are ignored here."""
        assert hidden % 256 == 0 and ffn % 256 == 0
        self.E, self.H, self.F, self.K, self.dtype = n_experts, hidden, ffn, top_k, dtype
        self.first, self.E_total = first_expert, n_experts_total or n_experts
        self.wgu, self.wd = gate_up_blocks, down_blocks
        dev = gate_up_blocks.device
        self.device, self.max_tokens = dev, max_tokens
        P = max_tokens * top_k
        i32, f32 = dict(dtype=torch.int32, device=dev), dict(dtype=torch.float32, device=dev)
        self.topk_ids = torch.zeros(max_tokens, top_k, **i32)
        self.topk_w = torch.zeros(max_tokens, top_k, **f32)
        self.sorted_ids = torch.zeros(P, **i32)
        self.offsets = torch.zeros(self.E_total + 1, **i32)
        self.packed_x = torch.zeros(_L.fuelq_act_packed_bytes(int(T.Q4K), P, hidden), dtype=torch.uint8, device=dev)
        self.packed_h = torch.zeros(_L.fuelq_act_packed_bytes(int(T.Q4K), P, ffn), dtype=torch.uint8, device=dev)
        self.gu = torch.zeros(P, 2 * ffn, **f32)          # sorted-row order
        self.y_pairs = torch.zeros(P, hidden, **f32)      # pair order

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        n = x.shape[0]
        assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (n, self.H) and n <= self.max_tokens
        assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.shape == (n, self.E_total)
        assert self.first == 0 and self.E == self.E_total, "use the expert-parallel driver for a partial expert set"
        if out is None:
            out = torch.empty(n, self.H, dtype=torch.float32, device=self.device)
        st = torch.cuda.current_stream().cuda_stream
        P = n * self.K
        _check(_L.fuelq_moe_route(logits.data_ptr(), n, self.E_total, self.K, self.topk_ids.data_ptr(),
                                  self.topk_w.data_ptr(), st), "fuelq_moe_route")
        _check(_L.fuelq_moe_bucket(self.topk_ids.data_ptr(), P, self.E_total, self.sorted_ids.data_ptr(),
                                   self.offsets.data_ptr(), st), "fuelq_moe_bucket")
        self.experts(x, P, st)
        _check(_L.fuelq_moe_combine(self.y_pairs.data_ptr(), self.topk_ids.data_ptr(), self.topk_w.data_ptr(), n, self.K,
                                    self.H, out.data_ptr(), st), "fuelq_moe_combine")
        return out

    def experts(self, x: torch.Tensor, n_rows: int, stream: int, divisor: int | None = None) -> None:
        """Sorted rows -> y_pairs: gather + quantize, gate/up, SwiGLU + quantize, down (scattered to pair order)."""
        _check(_L.fuelq_moe_quantize_rows(x.data_ptr(), self.H, self.sorted_ids.data_ptr(), divisor or self.K, n_rows,
                                          self.packed_x.data_ptr(), self.packed_x.numel(), stream), "fuelq_moe_quantize_rows")
        _check(_L.fuelq_moe_qmatmul(int(self.dtype), self.E, 2 * self.F, self.H, self.wgu.data_ptr(), self.packed_x.data_ptr(),
                                    n_rows, self.offsets.data_ptr() + 4 * self.first, None, self.gu.data_ptr(), stream),
               "fuelq_moe_qmatmul")
        _check(_L.fuelq_moe_swiglu_quantize(self.gu.data_ptr(), self.F, n_rows, self.packed_h.data_ptr(),
                                            self.packed_h.numel(), stream), "fuelq_moe_swiglu_quantize")
        _check(_L.fuelq_moe_qmatmul(int(self.dtype), self.E, self.H, self.F, self.wd.data_ptr(), self.packed_h.data_ptr(),
                                    n_rows, self.offsets.data_ptr() + 4 * self.first, self.sorted_ids.data_ptr(),
                                    self.y_pairs.data_ptr(), stream), "fuelq_moe_qmatmul")


class QMoeExpertParallel:
    """Expert parallelism over the ranks of a process group: rank r holds experts [r*E/g, (r+1)*E/g) and a share of the
    tokens. A forward routes the local tokens over ALL experts, sends each (token, slot) row to the rank that owns its
    expert, runs the local experts over what arrived, returns the results and combines on the home rank in ascending
    expert id - the order of the single-GPU block, whose output it reproduces bit for bit (a row's products do not
    depend on which other rows share its expert pass).

    Nothing is read on the host and every size is fixed, so a forward is a fixed sequence of stream-ordered calls that a
    CUDA graph can capture: each exchange is ONE all-to-all with equal splits. A (source, destination) pair of ranks owns
    a chunk of C + 1 rows of `hidden` floats, C = max_local_tokens * top_k being the most rows a rank can send anywhere;
    the rows travel sorted by expert in the chunk's first rows, and its last row carries their expert ids as int32
    (-1 = unused). The receiver buckets all chunk slots by local expert (unused slots drop out there), the grouped
    mat-vecs touch only the rows the bucketing lists, and the results go back in the same slots."""

    def __init__(self, n_experts_total: int, hidden: int, ffn: int, top_k: int, local_gate_up_blocks: torch.Tensor,
                 local_down_blocks: torch.Tensor, rank: int, world: int, group=None, dtype: T = T.Q4K,
                 max_local_tokens: int = 256):
        import torch.distributed as dist
        assert n_experts_total % world == 0
        self.dist, self.group, self.rank, self.world = dist, group, rank, world
        self.E, self.El, self.H, self.F, self.K = n_experts_total, n_experts_total // world, hidden, ffn, top_k
        dev = local_gate_up_blocks.device
        self.device = dev
        self.C = max_local_tokens * top_k
        assert self.C <= hidden, "the chunk's id row holds one int32 per row slot"
        self.Sg = self.C + 1
        S = world * self.Sg
        # routing state of the local tokens (all experts), and the local experts as a block over every chunk slot
        self.home = QMoeBlock(self.El, hidden, ffn, top_k, local_gate_up_blocks, local_down_blocks, dtype, max_local_tokens,
                              first_expert=rank * self.El, n_experts_total=n_experts_total)
        self.local = QMoeBlock(self.El, hidden, ffn, 1, local_gate_up_blocks, local_down_blocks, dtype, S)
        f32 = dict(dtype=torch.float32, device=dev)
        self.send = torch.zeros(S, hidden, **f32)
        self.recv = torch.zeros(S, hidden, **f32)
        self.y_back = torch.zeros(S, hidden, **f32)
        self.local_ids = torch.full((S,), -1, dtype=torch.int32, device=dev)
        self.out = torch.zeros(max_local_tokens, hidden, **f32)

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        dist, h, g, C, Sg, H = self.dist, self.home, self.world, self.C, self.Sg, self.H
        n = x.shape[0]
        P = n * self.K
        assert P <= C
        st = torch.cuda.current_stream().cuda_stream
        _check(_L.fuelq_moe_route(logits.data_ptr(), n, self.E, self.K, h.topk_ids.data_ptr(), h.topk_w.data_ptr(), st),
               "fuelq_moe_route")
        _check(_L.fuelq_moe_bucket(h.topk_ids.data_ptr(), P, self.E, h.sorted_ids.data_ptr(), h.offsets.data_ptr(), st),
               "fuelq_moe_bucket")
        _check(_L.fuelq_moe_ep_pack(x.data_ptr(), H, h.sorted_ids.data_ptr(), h.offsets.data_ptr(), h.topk_ids.data_ptr(), self.K,
                                    P, self.El, g, C, self.send.data_ptr(), st), "fuelq_moe_ep_pack")
        dist.all_to_all_single(self.recv, self.send, group=self.group)
        # local experts over every slot that carries a row (bucketed by local expert; unused slots have id -1)
        loc = self.local
        S = g * Sg
        _check(_L.fuelq_moe_ep_local_ids(self.recv.data_ptr(), H, C, g, self.rank * self.El, self.local_ids.data_ptr(), st),
               "fuelq_moe_ep_local_ids")
        _check(_L.fuelq_moe_bucket(self.local_ids.data_ptr(), S, self.El, loc.sorted_ids.data_ptr(), loc.offsets.data_ptr(), st),
               "fuelq_moe_bucket")
        loc.experts(self.recv, g * C, st, divisor=1)      # rows past the bucketed count repeat old slots: in bounds, unused
        dist.all_to_all_single(self.y_back, loc.y_pairs, group=self.group)
        _check(_L.fuelq_moe_ep_unpack(self.y_back.data_ptr(), H, h.sorted_ids.data_ptr(), h.offsets.data_ptr(), P, self.El, g, C,
                                      h.y_pairs.data_ptr(), st), "fuelq_moe_ep_unpack")
        out = self.out[:n]
        _check(_L.fuelq_moe_combine(h.y_pairs.data_ptr(), h.topk_ids.data_ptr(), h.topk_w.data_ptr(), n, self.K, self.H,
                                    out.data_ptr(), st), "fuelq_moe_combine")
        return out
