"""Column-sharded quantized matmul for the tensor-core path, one process per GPU.

Each rank holds rows [lo, hi) of the weight matrix (whole rows, so no block is cut) and computes those columns of
Y = X . W^T; the kernel's epilogue stores every output tile into every rank's copy of Y over peer-mapped memory
(`fuelq_qmatmul_sharded`), so the all-gather of the shards happens inside the kernel instead of after it. The
reference has no multi-GPU form of this path (fuel-core/src/quantized/mod.rs:854-868).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .ggml import GgmlDType as T
from .llama import PeerRegion, shard_range

_L = _lib.lib


class ShardedQMatMul:
    def __init__(self, dtype: T, local_blocks: torch.Tensor, n_total: int, k: int, max_m: int, rank: int, world: int):
        """local_blocks: GGUF blocks of this rank's rows shard_range(n_total, world, rank) of the [n_total, k] weight."""
        self.dtype, self.w, self.n_total, self.k, self.max_m = dtype, local_blocks, n_total, k, max_m
        self.rank, self.world = rank, world
        self.lo, self.hi = shard_range(n_total, world, rank)
        self.device = local_blocks.device
        self.region = PeerRegion({"y": 4 * max_m * n_total}, self.device, rank, world)
        self.y_dst = self.region.ptrs("y")
        self.y = self.region.view("y", 4 * max_m * n_total, torch.float32)
        self.ws_bytes = 0
        self.ws = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Enqueues this rank's share; the full Y is valid on every rank once `finish()` has returned on all of them."""
        m = x.shape[0]
        assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (m, self.k) and m <= self.max_m
        need = _L.fuelq_qmatmul_workspace_bytes(int(self.dtype), m, self.hi - self.lo, self.k)
        if self.ws is None or self.ws.numel() < need:
            self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_L.fuelq_qmatmul_sharded(int(self.dtype), m, self.hi - self.lo, self.k, self.w.data_ptr(), x.data_ptr(),
                                            self.y_dst, self.world, self.n_total, self.lo, self.ws.data_ptr(), self.ws.numel(),
                                            st), "fuelq_qmatmul_sharded")
        return self.y[:m * self.n_total].view(m, self.n_total)

    def finish(self) -> None:
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()

    def close(self) -> None:
        torch.cuda.synchronize()
        self.y = None
        self.region.close()
