"""Worker for the expert-parallel test: one rank per GPU under torch.distributed.run. Every rank builds the full set
of expert weights from the same seed, keeps its own experts and its share of the tokens, runs the expert-parallel
block, and rank 0 compares the gathered result with the single-GPU block over all tokens."""
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
    from fuel_b200.moe import QMoeBlock, QMoeExpertParallel
    E, H, F, K, N = 16, 512, 256, 4, 64
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    bgu = ops.quantize_weights(T.Q4K, torch.randn(E * 2 * F, H, generator=g, device=dev) * 0.02)
    bd = ops.quantize_weights(T.Q4K, torch.randn(E * H, F, generator=g, device=dev) * 0.02)
    x = torch.randn(N, H, generator=g, device=dev)
    logits = torch.randn(N, E, generator=g, device=dev)
    El, nl = E // world, N // world
    pgu, pd = bgu.numel() // E, bd.numel() // E
    ep = QMoeExpertParallel(E, H, F, K, bgu[rank * El * pgu:(rank + 1) * El * pgu].contiguous(),
                            bd[rank * El * pd:(rank + 1) * El * pd].contiguous(), rank, world, max_local_tokens=nl)
    xl, ll = x[rank * nl:(rank + 1) * nl].contiguous(), logits[rank * nl:(rank + 1) * nl].contiguous()
    out_local = ep.forward(xl, ll).clone()
    out_again = ep.forward(xl, ll)            # a second call over the same buffers: stale slots must not matter
    assert torch.equal(out_again, out_local)
    # the block has no host reads and fixed sizes: captured once, replayed as a CUDA graph (collectives included). The
    # graph is destroyed before the process group is touched again: a communicator must outlive the graphs that use it.
    graph_equal = None
    stream = torch.cuda.Stream(dev)
    try:
        with torch.cuda.stream(stream):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                out_g = ep.forward(xl, ll)
            out_g.zero_()
            gr.replay()
            stream.synchronize()
        graph_equal = bool(torch.equal(out_g, out_local))
        del gr
    except Exception as e:
        graph_equal = f"not captured: {type(e).__name__}"
    torch.cuda.synchronize()
    full = torch.empty(N, H, device=dev)
    dist.all_gather_into_tensor(full, out_local)
    torch.cuda.synchronize()
    res = {"err": ops.device_error()}
    if rank == 0:
        want = QMoeBlock(E, H, F, K, bgu, bd, max_tokens=N).forward(x, logits)
        torch.cuda.synchronize()
        res["equal"] = bool(torch.equal(full, want))
        res["graph_equal"] = graph_equal
        res["max_abs_diff"] = float((full - want).abs().max().item())
        print("EPRESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
