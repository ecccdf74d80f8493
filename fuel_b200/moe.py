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
    expert with one all-to-all (rows travel sorted by expert, so they arrive grouped by source rank), runs the local
    experts over what arrived, returns the results with a second all-to-all and combines on the home rank in ascending
    expert id - the order of the single-GPU block, whose output it reproduces bit for bit (every row's products do not
    depend on which other rows share its expert pass). The two exchanges need their split sizes on the host, so this
    path has one device-to-host read of the routing counts per block; everything else is stream-ordered."""

    def __init__(self, n_experts_total: int, hidden: int, ffn: int, top_k: int, local_gate_up_blocks: torch.Tensor,
                 local_down_blocks: torch.Tensor, rank: int, world: int, group=None, dtype: T = T.Q4K,
                 max_local_tokens: int = 256, max_recv_rows: int = 4096):
        import torch.distributed as dist
        assert n_experts_total % world == 0
        self.dist, self.group, self.rank, self.world = dist, group, rank, world
        self.E, self.El, self.H, self.F, self.K = n_experts_total, n_experts_total // world, hidden, ffn, top_k
        dev = local_gate_up_blocks.device
        self.device = dev
        # routing state of the local tokens (all experts), and the local experts as a block of their own
        self.home = QMoeBlock(self.El, hidden, ffn, top_k, local_gate_up_blocks, local_down_blocks, dtype, max_local_tokens,
                              first_expert=rank * self.El, n_experts_total=n_experts_total)
        self.local = QMoeBlock(self.El, hidden, ffn, 1, local_gate_up_blocks, local_down_blocks, dtype, max_recv_rows)
        self.max_recv = max_recv_rows

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        dist, h, g = self.dist, self.home, self.world
        n = x.shape[0]
        P = n * self.K
        st = torch.cuda.current_stream().cuda_stream
        _check(_L.fuelq_moe_route(logits.data_ptr(), n, self.E, self.K, h.topk_ids.data_ptr(), h.topk_w.data_ptr(), st),
               "fuelq_moe_route")
        _check(_L.fuelq_moe_bucket(h.topk_ids.data_ptr(), P, self.E, h.sorted_ids.data_ptr(), h.offsets.data_ptr(), st),
               "fuelq_moe_bucket")
        sorted_ids = h.sorted_ids[:P].long()
        edges = h.offsets[0:self.E + 1:self.El].cpu().tolist()          # the one host read: rows per destination rank
        send_counts = [edges[q + 1] - edges[q] for q in range(g)]
        send_x = x.index_select(0, sorted_ids // self.K)
        send_e = h.topk_ids[:n].reshape(-1).index_select(0, sorted_ids)
        counts_in = torch.tensor(send_counts, dtype=torch.int64, device=self.device)
        counts_out = torch.empty_like(counts_in)
        dist.all_to_all_single(counts_out, counts_in, group=self.group)
        recv_counts = counts_out.cpu().tolist()
        R = sum(recv_counts)
        assert R <= self.max_recv, "more rows routed to this rank than its buffers hold"
        recv_x = torch.empty(R, self.H, dtype=torch.float32, device=self.device)
        recv_e = torch.empty(R, dtype=torch.int32, device=self.device)
        dist.all_to_all_single(recv_x, send_x, recv_counts, send_counts, group=self.group)
        dist.all_to_all_single(recv_e, send_e, recv_counts, send_counts, group=self.group)
        # local experts over the received rows (grouped by source rank; bucketed again by local expert)
        loc = self.local
        y_recv = loc.y_pairs[:R]
        if R:
            local_ids = recv_e - self.rank * self.El
            _check(_L.fuelq_moe_bucket(local_ids.data_ptr(), R, self.El, loc.sorted_ids.data_ptr(), loc.offsets.data_ptr(), st),
                   "fuelq_moe_bucket")
            loc.experts(recv_x, R, st, divisor=1)
        y_back = torch.empty(P, self.H, dtype=torch.float32, device=self.device)
        dist.all_to_all_single(y_back, y_recv.contiguous(), send_counts, recv_counts, group=self.group)
        h.y_pairs[:P].index_copy_(0, sorted_ids, y_back)               # sorted order -> pair order
        out = torch.empty(n, self.H, dtype=torch.float32, device=self.device)
        _check(_L.fuelq_moe_combine(h.y_pairs.data_ptr(), h.topk_ids.data_ptr(), h.topk_w.data_ptr(), n, self.K, self.H,
                                    out.data_ptr(), st), "fuelq_moe_combine")
        return out
