"""Worker for the multi-GPU tests: one rank per GPU under torch.distributed.run. Builds the small test model
tensor-parallel over all ranks with the chosen exchange (argv[1]), decodes, and has rank 0 print one JSON line.
With a path as argv[2], rank 0 first writes the model to that GGUF file and every rank loads its rows from it."""
import faulthandler
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
faulthandler.dump_traceback_later(150, exit=True)  # a stuck rank ends itself instead of holding the GPUs

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    comm = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fuel_b200 import _lib, ops
    from fuel_b200.llama import LlamaConfig, QLlama, SyntheticWeights
    cfg = LlamaConfig(vocab=512, dim=1024, n_layers=3, n_heads=8, n_kv_heads=8, ffn_dim=2816, max_seq=96)
    if len(sys.argv) > 2:
        if rank == 0:
            SyntheticWeights(cfg, dev).export_gguf(sys.argv[2])
        dist.barrier()
        model = QLlama.from_gguf(sys.argv[2], dev, rank, world, comm=comm, max_seq=cfg.max_seq)
    else:
        model = QLlama(cfg, dev, rank, world, comm=comm)
    prompt = np.random.Generator(np.random.PCG64(4)).integers(0, 512, 20).tolist()
    out = {}
    try:
        out["eager"] = model.generate(prompt, 12)
        _lib.lib.fuelq_set_option(_lib.OPT_PDL, 1)
        model.capture()
        out["graph_pdl"] = model.generate(prompt, 12)
        out["logits_sum"] = float(model.logits.double().sum().item())
        out["err"] = ops.device_error()
    finally:
        model.release()
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("TPRESULT " + json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
