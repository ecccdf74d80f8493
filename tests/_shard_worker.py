"""Worker for the column-sharded prefill test: one rank per GPU under torch.distributed.run. Every rank quantizes
the same weight, keeps its rows, runs the sharded call; rank 0 compares its full Y with the single-GPU call."""
import faulthandler
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
faulthandler.dump_traceback_later(150, exit=True)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fuel_b200 import GgmlDType as T, ops
    from fuel_b200.llama import shard_range
    from fuel_b200.sharded import ShardedQMatMul
    n, k, m = 1000, 1024, 300
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    w = torch.randn(n, k, generator=g, device=dev) * 0.02
    x = torch.randn(m, k, generator=g, device=dev)
    blocks = ops.quantize_weights(T.Q4K, w)
    per_row = blocks.numel() // n
    lo, hi = shard_range(n, world, rank)
    sh = ShardedQMatMul(T.Q4K, blocks[lo * per_row:hi * per_row].contiguous(), n, k, m, rank, world)
    res = {}
    try:
        y = sh.forward(x)
        sh.finish()
        want = ops.qmatmul(T.Q4K, blocks, n, x)
        torch.cuda.synchronize()
        ok = torch.tensor([1 if torch.equal(y, want) else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        res = {"equal_on_every_rank": int(ok.item()), "err": ops.device_error()}
        dist.barrier()
    finally:
        sh.close()
    if rank == 0:
        print("SHRESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
