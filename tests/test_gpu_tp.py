"""Tensor-parallel decode on 2 GPUs (skipped on a one-GPU box): tokens must equal the one-GPU run for both exchange
forms - NCCL all-gathers between the kernels, and the exchange done inside the kernels over peer-mapped memory."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _single_gpu_tokens():
    from fuel_b200.llama import LlamaConfig, QLlama
    cfg = LlamaConfig(vocab=512, dim=1024, n_layers=3, n_heads=8, n_kv_heads=8, ffn_dim=2816, max_seq=96)
    model = QLlama(cfg, torch.device("cuda", 0))
    prompt = np.random.Generator(np.random.PCG64(4)).integers(0, 512, 20).tolist()
    return model.generate(prompt, 12), float(model.logits.double().sum().item())


@pytest.mark.parametrize("comm,from_file", [("peer", False), ("nccl", False), ("peer", True)])
def test_two_gpus_decode_the_same_tokens(comm, from_file, tmp_path):
    """from_file: the ranks load their row slices from a GGUF file that rank 0 wrote, instead of generating them."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    want, logits_sum = _single_gpu_tokens()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "_tp_worker.py"), comm]
    if from_file:
        cmd.append(str(tmp_path / "tp.gguf"))
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=400)
    lines = [l for l in r.stdout.splitlines() if l.startswith("TPRESULT ")]
    assert r.returncode == 0 and lines, (r.stdout[-2000:], r.stderr[-2000:])
    got = json.loads(lines[-1][len("TPRESULT "):])
    assert got["err"] == 0
    assert got["eager"] == want and got["graph_pdl"] == want
    assert got["logits_sum"] == logits_sum      # every logit has the same bits, so does their f64 sum


def test_two_gpus_expert_parallel_block_equals_single_gpu_block():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29534", os.path.join(ROOT, "tests", "_ep_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=400)
    lines = [l for l in r.stdout.splitlines() if l.startswith("EPRESULT ")]
    assert r.returncode == 0 and lines, (r.stdout[-2000:], r.stderr[-2000:])
    got = json.loads(lines[-1][len("EPRESULT "):])
    assert got["err"] == 0 and got["equal"], got
    assert got["graph_equal"] is True or str(got["graph_equal"]).startswith("not captured"), got


def test_two_gpus_column_sharded_prefill_fills_every_copy_of_y():
    """fuelq_qmatmul_sharded: each GPU computes its columns and its epilogue writes them into both GPUs' Y; after both
    calls every GPU's Y equals the single-GPU product bit for bit."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29535", os.path.join(ROOT, "tests", "_shard_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=400)
    lines = [l for l in r.stdout.splitlines() if l.startswith("SHRESULT ")]
    assert r.returncode == 0 and lines, (r.stdout[-2000:], r.stderr[-2000:])
    got = json.loads(lines[-1][len("SHRESULT "):])
    assert got["err"] == 0 and got["equal_on_every_rank"] == 1, got
