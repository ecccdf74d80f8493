"""Benchmark of the quantized mat-vec hot path.

Workload (benchmark configuration 2, the Q4_K decode case): y[1, 11008] = x[1, 4096] . W^T with W a
Q4_K matrix [11008 x 4096] (25 362 432 bytes of blocks). One step = one pass over LAYERS
distinct weight matrices (each with its own activation row), i.e. LAYERS quantized
mat-vec calls; cycling over 32 x 25.4 MB = 811 MB of weights keeps every read in HBM, not L2.
Weights are N(0, 0.02) from a seeded generator, quantized by the library's device quantizer
(byte-identical to the reference's); activations N(0, 1).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Metric: achieved HBM GB/s = algorithmic bytes (W blocks + 4*M*k + 4*M*n per mat-vec) / time.
N > 1 (torchrun): the SAME 32 matrices, each split by output rows over the N GPUs (strong scaling): a rank
streams its rows, its kernel stores its slice of y into every GPU's copy over NVLink, and a consumer kernel on every
GPU waits for the whole vector (takes its argmax) before the next mat-vec — the exchange is inside the kernels, no
library collective. Beside the headline the line carries the 7B-architecture decode (tensor-parallel at N > 1), the
prefill GEMM of configuration 3 (`prefill`; column-sharded `prefill_sharded` at N > 1) and the MoE block of configuration 5
(`moe_block`; expert-parallel `moe_ep` at N > 1).
--impl reference: the reference's CPU path (its arithmetic restated under oracle/, AVX2 order,
all host threads) on the same step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_OUT, K_IN, M_ROWS = 11008, 4096, 1
LAYERS = 32
W_BYTES = N_OUT * (K_IN // 256) * 144
ALGO_BYTES = W_BYTES + 4 * M_ROWS * K_IN + 4 * M_ROWS * N_OUT  # 25 422 848
WORKLOAD = f"q4k_qmatmul_m{M_ROWS}_k{K_IN}_n{N_OUT}_x{LAYERS}_distinct_matrices"


REF_MIN_SECONDS = 5.0


def bench_scaling(world: int) -> str:
    return "strong"   # the same 32 matrices at every GPU count


def bench_config(world: int, pdl: bool) -> dict:
    """The workload description both arms print (the driver compares the two dicts)."""
    return {"workload": WORKLOAD, "m": M_ROWS, "k": K_IN, "n": N_OUT, "format": "Q4_K", "layers": LAYERS,
            "l2": f"inputs larger than L2: {LAYERS * W_BYTES / 1e6:.0f} MB of distinct weights per step", "cuda_graph": True,
            "pdl": pdl, "parallelism": "one GPU" if world == 1 else
            f"each matrix split by output rows over {world} GPUs; every GPU receives the whole y inside the kernels"}


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _tensor_peaks():
    """Measured dense bf16 rates of this pool's GPUs: (burst, sustained under the power cap, which)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained") or j["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def tensor_roofline(tflops: float) -> dict:
    burst, sustained, kind = _tensor_peaks()
    return {"bound": "tensor", "achieved": tflops, "peak": burst, "unit": "TFLOP/s", "frac": tflops / burst,
            "peak_sustained": sustained, "frac_of_sustained": tflops / sustained, "peak_kind": f"of {kind}",
            "flops": "2*M*N*K over the whole step (activation pre-pass, weight dequantization, GEMM)"}


class ClockSampler:
    """Samples SM clock and throttle reasons through nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self, t0: float, t1: float):
        rows = [s for t, s in self.samples if t0 <= t <= t1] or [s for _, s in self.samples[-5:]]
        mhz, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            p = [c.strip() for c in r.split(",")]
            try:
                mhz.append(float(p[0]))
                mx = max(mx, float(p[1]))
            except Exception:
                continue
            for name, val in zip(names, p[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def _dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def make_weights(torch, ops, T, device, lo, hi):
    """Rows [lo, hi) of the LAYERS seeded matrices (the same matrices at every GPU count)."""
    ws = []
    g = torch.Generator(device=device)
    for i in range(LAYERS):
        g.manual_seed(i)
        w = torch.randn(N_OUT, K_IN, generator=g, device=device, dtype=torch.float32) * 0.02
        ws.append(ops.quantize_weights(T.Q4K, w[lo:hi].contiguous()))
        del w
    return ws


def host_threads(O) -> int:
    """Threads for the CPU legs: every core this process may run on. A launcher that exports OMP_NUM_THREADS=1 for
    its workers (torch.distributed.run does) must not turn the CPU baseline into a one-thread run."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(n, O.max_threads())


def cpu_pass(O, w_host, x_host, threads):
    for wb, x in zip(w_host, x_host):
        O.matmul(O.Q4K, x, wb, N_OUT, O.AVX2, threads)


def run_reference(args):
    """The reference's CPU path on the same step (all host threads)."""
    rank, local_rank, world = _dist_env()
    if rank != 0:
        return
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the OpenMP runtime reads it when it is loaded,
    # so put the real core count back before the oracle library comes in
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    except AttributeError:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    import numpy as np
    from oracle import oracle as O
    threads = host_threads(O)
    rng = np.random.Generator(np.random.PCG64(0))
    # one quantized matrix per layer would cost ~1 s of host quantization each; the CPU timing
    # does not depend on the weight values, so LAYERS views of 4 distinct matrices are used,
    # still 4 x 25 MB > any host cache
    base = [O.quantize(O.Q4K, rng.standard_normal((N_OUT, K_IN), dtype=np.float32) * np.float32(0.02))
            for _ in range(4)]
    w_host = [base[i % 4] for i in range(LAYERS)]
    x_host = [rng.standard_normal((M_ROWS, K_IN), dtype=np.float32) for _ in range(LAYERS)]
    # Warm-up until the OpenMP team is hot, then size a step so that the timed region lasts at least REF_MIN_SECONDS:
    # a step is `repeats` passes over the LAYERS matrices (a 0.25 s region under-reports this path by ~1.4x).
    cpu_pass(O, w_host, x_host, threads)
    t0 = time.perf_counter()
    n_warm = 0
    while n_warm < max(args.warmup, 1) or time.perf_counter() - t0 < 1.0:
        cpu_pass(O, w_host, x_host, threads)
        n_warm += 1
    t_pass = (time.perf_counter() - t0) / n_warm
    repeats = max(1, int(np.ceil(REF_MIN_SECONDS / (args.steps * t_pass))))
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(repeats):
            cpu_pass(O, w_host, x_host, threads)
    dt = time.perf_counter() - t0
    passes = args.steps * repeats
    gbs = ALGO_BYTES * LAYERS * passes / dt / 1e9
    line = {
        "impl": "reference", "metric": "q4k_qmatmul_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / passes * 1e3, "higher_is_better": True,
        "scaling": bench_scaling(args.gpus), "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": bench_config(args.gpus, bool(args.pdl)),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{args.steps} steps x {repeats} passes of {LAYERS} mat-vecs in {dt:.1f} s (4 distinct matrices "
                                   f"cycled, AVX2 order, OpenMP); ms_per_step is per pass"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _time_graph(torch, stream, fn, reps):
    """Average microseconds per call of fn(), replayed as a CUDA graph on `stream` (events on that stream)."""
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(3):
            g.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def run_side_workload(args):
    """benchmark configurations 2 (batch sweep), 3 (prefill GEMM) and 5 (MoE block): one JSON line per case. Several GPUs: the
    column-sharded prefill GEMM or the expert-parallel MoE block."""
    rank, local_rank, world = _dist_env()
    if world > 1:
        assert args.workload in ("moe", "prefill"), "multi-GPU forms: the MoE block (expert-parallel), the prefill GEMM (column-sharded)"
        if args.workload == "prefill":
            return run_prefill_sharded(args, rank, local_rank, world)
        return run_moe_expert_parallel(args, rank, local_rank, world)
    for line in side_lines(args, args.workload):
        print(json.dumps(line), flush=True)


def side_lines(args, workload):
    """The cases of one side workload on one GPU, as a generator of result dicts: seeded synthetic tensors of the stated
    shapes, distinct weight copies cycling through more than L2, CUDA-graph replay."""
    import torch

    from fuel_b200 import GgmlDType as T, _lib, ops
    from fuel_b200.moe import QMoeBlock
    L = _lib.lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    L.fuelq_set_option(_lib.OPT_PDL, 1 if args.pdl else 0)
    L.fuelq_set_option(_lib.OPT_PREFILL_TF32, 1 if args.tf32 else 0)
    L.fuelq_set_option(_lib.OPT_PREFILL_BF16, 1 if args.bf16 else 0)
    st = torch.cuda.Stream(dev)
    peak, peak_kind = _peaks()
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)

    def matmul_case(t, name, n, k, m, copies, reps, parity_rows=0):
        ws = [ops.quantize_weights(t, torch.randn(n, k, generator=gen, device=dev) * 0.02) for _ in range(copies)]
        x = torch.randn(m, k, generator=gen, device=dev)
        y = torch.empty(m, n, device=dev)
        wsb = L.fuelq_qmatmul_workspace_bytes(int(t), m, n, k)
        scratch = torch.empty(max(wsb, 16), dtype=torch.uint8, device=dev)

        def p():
            for w in ws:
                _lib.check(L.fuelq_qmatmul(int(t), m, n, k, w.data_ptr(), x.data_ptr(), y.data_ptr(), scratch.data_ptr(), wsb,
                                           st.cuda_stream), "fuelq_qmatmul")
        us = _time_graph(torch, st, p, reps) / copies
        algo = ws[0].numel() + 4 * m * k + 4 * m * n
        line = {"workload": f"{name}_k{k}_n{n}_m{m}", "us": us, "GB/s": algo / us / 1e3, "TFLOP/s": 2 * m * n * k / us / 1e6,
                "hbm_frac": algo / us / 1e3 / peak, "peak_kind": f"of {peak_kind}", "weight_copies": copies}
        if parity_rows:
            # observed error of the last copy's product on a sample of activation rows: against the exact dequantized
            # product (f64) and against the reference's CPU path (8-bit activation blocks, integer dot products)
            import numpy as np
            from oracle import oracle as O
            ot = {T.Q4K: O.Q4K, T.Q6K: O.Q6K, T.Q8_0: O.Q8_0, T.Q5K: O.Q5K, T.Q4_0: O.Q4_0, T.Q4_1: O.Q4_1, T.Q5_0: O.Q5_0,
                  T.Q5_1: O.Q5_1, T.Q2K: O.Q2K, T.Q3K: O.Q3K}[t]
            rows = np.unique(np.linspace(0, m - 1, parity_rows).astype(np.int64))
            wb = ws[-1].cpu().numpy()
            xs_ = x[torch.from_numpy(rows).to(dev)].cpu().numpy()
            got = y[torch.from_numpy(rows).to(dev)].cpu().numpy().astype(np.float64)
            exact = O.matmul_dequant_f64(ot, xs_, wb, n)
            ref = O.matmul(ot, xs_, wb, n, O.AVX2).astype(np.float64)
            line["parity"] = {"rows_sampled": int(rows.size), "numerics": int(L.fuelq_qmatmul_numerics(int(t), m, n, k)),
                              "max_err_vs_exact_dequant_over_max": float(np.abs(got - exact).max() / np.abs(exact).max()),
                              "frobenius_vs_exact_dequant": float(np.linalg.norm(got - exact) / np.linalg.norm(exact)),
                              "max_err_vs_cpu_path_over_max": float(np.abs(got - ref).max() / np.abs(ref).max()),
                              "frobenius_vs_cpu_path": float(np.linalg.norm(got - ref) / np.linalg.norm(ref))}
        return line

    if workload == "sweep":
        for t, name in ((T.Q4K, "Q4_K"), (T.Q6K, "Q6_K"), (T.Q8_0, "Q8_0")):
            for n, k in ((11008, 4096), (4096, 11008)):
                for m in (1, 2, 4, 8, 16, 32, 64, 128):
                    if args.only and args.only not in f"{name}_k{k}_n{n}_m{m}":
                        continue
                    yield matmul_case(t, name, n, k, m, 12, 20)
    elif workload == "q5k":
        for n, k in ((11008, 4096), (4096, 11008)):
            for m in (1, 2, 4, 8, 16):
                yield matmul_case(T.Q5K, "Q5_K", n, k, m, 12, 20)
    elif workload == "formats":
        # the formats served by the generic exact-integer decode kernel up to 16 rows, and above that by the tensor-core
        # kernel on slabs of rows dequantized into its operand type (512 rows here, with the observed error)
        for t, name in ((T.Q4_0, "Q4_0"), (T.Q4_1, "Q4_1"), (T.Q5_0, "Q5_0"), (T.Q5_1, "Q5_1"), (T.Q2K, "Q2_K"), (T.Q3K, "Q3_K"),
                        (T.Q5K, "Q5_K")):
            for m in (1, 4, 16, 512):
                if args.only and args.only not in f"{name}_k4096_n11008_m{m}":
                    continue
                parity = 8 if m == 512 and not args.no_cpu_baseline else 0
                yield matmul_case(t, name, 11008, 4096, m, 12 if m < 512 else 4, 20, parity_rows=parity)
    elif workload == "prefill":
        line = matmul_case(T.Q4K, "Q4_K", 14336, 4096, 2048, 6, 10, parity_rows=0 if args.no_cpu_baseline else 32)
        line["operands"] = "tf32" if args.tf32 else "bf16" if args.bf16 else "f16"
        line["roofline"] = tensor_roofline(line["TFLOP/s"])
        yield line
    else:
        E, H, F, K, N, copies = 128, 2048, 768, 8, 256, 4
        blocks = []
        for _ in range(copies):
            bgu = ops.quantize_weights(T.Q4K, torch.randn(E * 2 * F, H, generator=gen, device=dev) * 0.02)
            bd = ops.quantize_weights(T.Q4K, torch.randn(E * H, F, generator=gen, device=dev) * 0.02)
            blocks.append(QMoeBlock(E, H, F, K, bgu, bd, max_tokens=N))
        x = torch.randn(N, H, generator=gen, device=dev)
        logits = torch.randn(N, E, generator=gen, device=dev)
        outs = [torch.empty(N, H, device=dev) for _ in range(copies)]

        def p():
            for b, o in zip(blocks, outs):
                b.forward(x, logits, o)
        us = _time_graph(torch, st, p, 20) / copies
        wbytes = E * 3 * F * H // 256 * 144
        yield {"workload": f"moe_block_e{E}_h{H}_f{F}_top{K}_tokens{N}_q4k", "us": us, "GB/s": wbytes / us / 1e3,
               "tokens_per_s": N / us * 1e6, "hbm_frac": wbytes / us / 1e3 / peak, "peak_kind": f"of {peak_kind}",
               "weight_bytes": wbytes, "weight_copies": copies, "launches_per_block": 9}
    assert ops.device_error() == 0, "a kernel recorded an expired bounded wait"


def run_prefill_sharded(args, rank, local_rank, world, own_group=True):
    """benchmark configuration 3 across GPUs: W [14336 x 4096] Q4_K split by rows (columns of Y) over the ranks, X [2048 x 4096]
    on every rank; each rank's kernel writes its columns into every rank's Y (the all-gather is the kernel's epilogue).
    CUDA events around the call on each rank, max over ranks."""
    import torch
    import torch.distributed as dist

    from fuel_b200 import GgmlDType as T, _lib, ops
    from fuel_b200.llama import shard_range
    from fuel_b200.sharded import ShardedQMatMul
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if own_group:
        dist.init_process_group("nccl", device_id=dev)
    result = None
    _lib.lib.fuelq_set_option(_lib.OPT_PREFILL_TF32, 1 if args.tf32 else 0)
    _lib.lib.fuelq_set_option(_lib.OPT_PREFILL_BF16, 1 if args.bf16 else 0)
    n, k, m, copies = 14336, 4096, 2048, 4
    lo, hi = shard_range(n, world, rank)
    gen = torch.Generator(device=dev)
    shards = []
    for c in range(copies):
        gen.manual_seed(100 * c + rank)
        wb = ops.quantize_weights(T.Q4K, torch.randn(hi - lo, k, generator=gen, device=dev) * 0.02)
        shards.append(ShardedQMatMul(T.Q4K, wb, n, k, m, rank, world))
    gen.manual_seed(7)
    x = torch.randn(m, k, generator=gen, device=dev)
    try:
        for sh in shards:
            sh.forward(x)
        shards[0].finish()
        reps = 10
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            for sh in shards:
                sh.forward(x)
        e1.record()
        shards[0].finish()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3 / (reps * copies)
        assert ops.device_error() == 0
        if rank == 0:
            peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
            result = {"workload": f"Q4_K_k{k}_n{n}_m{m}_column_sharded", "n_gpus": world, "us": us,
                      "TFLOP/s": 2 * m * n * k / us / 1e6, "operands": "tf32" if args.tf32 else "bf16" if args.bf16 else "f16",
                      "all_gather": "inside the kernel epilogue (stores into every GPU's Y over NVLink)",
                      "y_bytes_stored_per_gpu": 4 * m * (hi - lo) * world,
                      "bf16_tflops_measured_per_gpu": peak.get("bf16_tflops")}
            if own_group:
                print(json.dumps(result), flush=True)
    finally:
        for sh in shards:
            sh.close()
    dist.barrier()
    if own_group:
        dist.destroy_process_group()
    return result


def run_moe_expert_parallel(args, rank, local_rank, world, own_group=True):
    """benchmark configuration 5 expert-parallel: 128 experts split over the ranks, 256 tokens split over the ranks, one NCCL
    all-to-all with equal splits each way per block, nothing read on the host; replayed from a CUDA graph when the capture
    succeeds on every rank, else eager. CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist

    from fuel_b200 import GgmlDType as T, _lib, ops
    from fuel_b200.moe import QMoeExpertParallel
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if own_group:
        dist.init_process_group("nccl", device_id=dev)
    result = None
    _lib.lib.fuelq_set_option(_lib.OPT_PDL, 1 if args.pdl else 0)
    E, H, F, K, N, copies = 128, 2048, 768, 8, 256, 4
    El, nl = E // world, N // world
    gen = torch.Generator(device=dev)
    blocks = []
    for c in range(copies):
        gen.manual_seed(1000 * c + rank)
        bgu = ops.quantize_weights(T.Q4K, torch.randn(El * 2 * F, H, generator=gen, device=dev) * 0.02)
        bd = ops.quantize_weights(T.Q4K, torch.randn(El * H, F, generator=gen, device=dev) * 0.02)
        blocks.append(QMoeExpertParallel(E, H, F, K, bgu, bd, rank, world, max_local_tokens=nl))
    gen.manual_seed(77 + rank)
    x = torch.randn(nl, H, generator=gen, device=dev)
    logits = torch.randn(nl, E, generator=gen, device=dev)
    for b in blocks:
        b.forward(x, logits)
    torch.cuda.synchronize()
    dist.barrier()
    # The block is a fixed sequence of stream-ordered calls, so it replays from a CUDA graph (collectives included).
    # The graph is destroyed before anything else touches the process group: a communicator must outlive the
    # graphs that captured its collectives.
    graph = None
    stream = torch.cuda.Stream(dev)
    if not os.environ.get("FUELQ_BENCH_EP_EAGER"):
        try:
            with torch.cuda.stream(stream):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for b in blocks:
                        b.forward(x, logits)
                graph.replay()
                stream.synchronize()
        except Exception:
            graph = None
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    torch.cuda.synchronize()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)     # every rank replays, or none does
    if int(ok.item()) == 0:
        graph = None
    captured = graph is not None
    reps = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(reps):
            if captured:
                graph.replay()
            else:
                for b in blocks:
                    b.forward(x, logits)
        e1.record(stream)
        stream.synchronize()
    torch.cuda.synchronize()
    del graph
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.item()) * 1e3 / (reps * copies)
    assert ops.device_error() == 0
    if rank == 0:
        wbytes = E * 3 * F * H // 256 * 144
        result = {"workload": f"moe_block_e{E}_h{H}_f{F}_top{K}_tokens{N}_q4k_expert_parallel", "n_gpus": world, "us": us,
                  "tokens_per_s": N / us * 1e6, "GB/s": wbytes / us / 1e3, "weight_bytes_per_gpu": wbytes // world,
                  "exchange": "one NCCL all-to-all with equal splits each way per block (fixed-capacity chunks, expert ids in the chunk's "
                              "last row); no host reads",
                  "cuda_graph": captured}
        if own_group:
            print(json.dumps(result), flush=True)
    dist.barrier()
    if own_group:
        dist.destroy_process_group()
    return result


def run_config0(torch, device, pdl):
    """Benchmark configuration 0, the CPU-runnable case: Q4_K weight [4096 x 4096] from N(0, 0.02) seed 0, activation
    [1, 4096] from N(0, 1) seed 1, checked against the CPU path; then timed as 64 distinct matrices of that shape
    (604 MB of blocks, larger than L2; matrix 0 is the seeded one) replayed from a CUDA graph."""
    import numpy as np

    from fuel_b200 import GgmlDType as T, _lib, ops
    from oracle import oracle as O
    L = _lib.lib
    n = k = 4096
    copies = 64
    g = torch.Generator(device=device)
    ws = []
    for i in range(copies):
        g.manual_seed(0 if i == 0 else 100 + i)
        ws.append(ops.quantize_weights(T.Q4K, torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * 0.02))
    g.manual_seed(1)
    x = torch.randn(1, k, generator=g, device=device)
    ys = torch.empty(copies, n, device=device)
    wsb = L.fuelq_qmatmul_workspace_bytes(int(T.Q4K), 1, n, k)
    scratch = torch.empty(copies, wsb, dtype=torch.uint8, device=device)
    stream = torch.cuda.Stream(device)
    sp = stream.cuda_stream

    def one_pass():
        for i in range(copies):
            _lib.check(L.fuelq_qmatmul(int(T.Q4K), 1, n, k, ws[i].data_ptr(), x.data_ptr(), ys[i].data_ptr(), scratch[i].data_ptr(),
                                       wsb, sp), "fuelq_qmatmul")

    with torch.cuda.stream(stream):
        one_pass()
        stream.synchronize()
        us = _time_graph(torch, stream, one_pass, 50) / copies
    ref = O.matmul(O.Q4K, x.cpu().numpy(), ws[0].cpu().numpy(), n, O.SCALAR)
    err = float(np.abs(ys[0].cpu().numpy() - ref[0]).max() / np.abs(ref).max())
    assert err <= 2e-6, f"configuration 0: GPU result off the CPU path by {err}"
    algo = n * (k // 256) * 144 + 4 * k + 4 * n
    peak, peak_kind = _peaks()
    return {"workload": "q4k_qmatmul_m1_k4096_n4096 (seed 0 weights, seed 1 activation), timed over 64 distinct matrices",
            "avg_launch_us": us, "algorithmic_bytes_per_launch": algo, "gbs": algo / (us * 1e-6) / 1e9,
            "hbm_frac": algo / (us * 1e-6) / 1e9 / peak, "peak_kind": f"of {peak_kind}", "pdl": bool(pdl),
            "max_rel_err_vs_cpu_path": err}


def run_decode_7b(torch, dist, device, rank, world):
    """LLaMA-2-7B-architecture greedy decode, batch 1 (Q4_K_M-style mix, random-init weights, f32 KV cache):
    a 512-token seeded prompt fed one token at a time, then 128 new tokens timed with CUDA events on a replayed
    CUDA graph. With more than one GPU the model is tensor-parallel over all of them (column-parallel q/k/v, gate/up
    and head; row-parallel o and down, their partial vectors exchanged inside the kernels and summed by one fixed
    tree); the token hash must not depend on the GPU count."""
    import hashlib

    import numpy as np

    from fuel_b200 import ops
    from fuel_b200.llama import LlamaConfig, QLlama

    model = QLlama(LlamaConfig.llama2_7b(), device, rank, world, comm="peer" if world > 1 else "nccl")
    try:
        model.capture()
        prompt = np.random.Generator(np.random.PCG64(3)).integers(0, 32000, 512).tolist()
        model.reset()
        ids = torch.as_tensor(prompt, dtype=torch.int32, device=device)
        for i in range(len(prompt)):
            model.token.copy_(ids[i:i + 1])
            model.run_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        toks = [model.next_token.clone()]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(127):
            model.run_step()
            toks.append(model.next_token.clone())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out = torch.cat(toks).cpu().tolist()
        assert ops.device_error() == 0, "a kernel recorded an expired bounded wait"
        peak, peak_kind = _peaks()
        ms_tok = ms / 127
        # per token every rank streams its weight shard once and its share of the f32 KV cache (ctx ~ 576)
        kv_bytes = 2 * 32 * 576 * 4096 * 4 // world
        return {"tok_s": 1e3 / ms_tok, "ms_per_token": ms_tok, "n_gpus": world, "prompt_tokens": 512, "new_tokens": 128,
                "timed_tokens": 127, "tokens_sha256": hashlib.sha256(str(out).encode()).hexdigest()[:16],
                "exchange": "none (one GPU)" if world == 1 else
                            "column-parallel q/k/v, gate/up, head; row-parallel o, down summed by a fixed tree; two exchanges per layer, "
                            "as stamped stores inside the kernels over peer-mapped memory",
                "weight_bytes_per_gpu": model.weight_bytes, "kv_bytes_per_gpu_per_token": kv_bytes,
                "hbm_frac_per_gpu": (model.weight_bytes + kv_bytes) / (ms_tok * 1e-3) / 1e9 / peak,
                "peak_kind": f"of {peak_kind}", "cuda_graph": True, "launches_per_token": sum(9 if l["v"] is None else 10 for l in model.layers) + 6}
    finally:
        model.release()


def main():
    global LAYERS, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fuelq", choices=["fuelq", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--layers", type=int, default=LAYERS, help="distinct weight matrices per step (profiling runs use fewer)")
    ap.add_argument("--tf32", action="store_true", help="--workload prefill: tensor-core path in tf32 instead of f16")
    ap.add_argument("--only", default="", help="--workload sweep: run only the cases whose name contains this text, e.g. Q4_K_k4096_n11008_m8")
    ap.add_argument("--bf16", action="store_true", help="--workload prefill: 16-bit operands as bf16 instead of f16")
    ap.add_argument("--decode-grid", type=int, default=0, help="thread blocks of the decode mat-vec (0: the library's choice, two per SM)")
    ap.add_argument("--no-model", action="store_true", help="skip the 7B-architecture decode that is reported beside the metric")
    ap.add_argument("--workload", default="decode", choices=["decode", "sweep", "prefill", "moe", "q5k", "formats"],
                    help="decode: the headline line (default). sweep / prefill / moe: benchmark configurations 2 / 3 / 5 on one GPU, "
                         "one JSON line per case")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    LAYERS = args.layers
    WORKLOAD = f"q4k_qmatmul_m{M_ROWS}_k{K_IN}_n{N_OUT}_x{LAYERS}_distinct_matrices"
    if args.impl == "reference":
        return run_reference(args)
    if args.workload != "decode":
        return run_side_workload(args)

    import ctypes

    import numpy as np
    import torch
    import torch.distributed as dist

    from fuel_b200 import GgmlDType as T, _lib, ops

    rank, local_rank, world = _dist_env()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    L = _lib.lib
    _lib.check(L.fuelq_set_option(_lib.OPT_PDL, 1 if args.pdl else 0), "set_option")
    _lib.check(L.fuelq_set_option(_lib.OPT_DECODE_GRID, args.decode_grid), "set_option")

    from fuel_b200.llama import PeerRegion, shard_range
    lo, hi = shard_range(N_OUT, world, rank)
    n_loc = hi - lo
    ws = make_weights(torch, ops, T, device, lo, hi)
    g = torch.Generator(device=device)
    g.manual_seed(7)
    xs = [torch.randn(M_ROWS, K_IN, generator=g, device=device) for _ in range(LAYERS)]
    ys = [torch.empty(M_ROWS, n_loc, device=device) for _ in range(LAYERS)]
    ws_bytes = L.fuelq_qmatmul_workspace_bytes(int(T.Q4K), M_ROWS, n_loc, K_IN)
    scratch = [torch.empty(ws_bytes, dtype=torch.uint8, device=device) for _ in range(LAYERS)]

    stream = torch.cuda.Stream(device)
    sptr = stream.cuda_stream

    region = None
    if world > 1:
        # one destination vector per matrix on every GPU ({value, stamp} pairs), mapped into every rank
        region = PeerRegion({f"y{i}": L.fuelq_peer_vec_bytes(N_OUT) for i in range(LAYERS)}, device, rank, world)
        epoch = torch.zeros(1, dtype=torch.int32, device=device)
        picks = torch.zeros(LAYERS, dtype=torch.int32, device=device)
        peers = _lib.Peers()
        peers.world, peers.rank, peers.epoch = world, rank, epoch.data_ptr()
        peers_ref = ctypes.byref(peers)
        dsts = [region.ptrs(f"y{i}") for i in range(LAYERS)]
        owns = [region.own + region.off[f"y{i}"] for i in range(LAYERS)]

    def one_pass():
        if world > 1:
            for i, (w, x, s) in enumerate(zip(ws, xs, scratch)):
                _lib.check(L.fuelq_quantize_act_packed(int(T.Q4K), M_ROWS, K_IN, x.data_ptr(), s.data_ptr(), ws_bytes, sptr), "quantize")
                _lib.check(L.fuelq_qmatmul_packed_peer(int(T.Q4K), K_IN, n_loc, w.data_ptr(), s.data_ptr(), dsts[i], lo, peers_ref, 0,
                                                       sptr), "fuelq_qmatmul_packed_peer")
                # the consumer: waits until every rank's slice of y has arrived here, takes the arg-max, ends the exchange step
                _lib.check(L.fuelq_argmax_last_peer(owns[i], N_OUT, picks.data_ptr() + 4 * i, peers_ref, 0, epoch.data_ptr(), sptr),
                           "fuelq_argmax_last_peer")
            return
        for w, x, y, s in zip(ws, xs, ys, scratch):
            st = L.fuelq_qmatmul(int(T.Q4K), M_ROWS, n_loc, K_IN, w.data_ptr(), x.data_ptr(), y.data_ptr(),
                                 s.data_ptr(), ws_bytes, sptr)
            if st:
                _lib.check(st, "fuelq_qmatmul")

    ys_mv = [torch.empty(M_ROWS, n_loc, device=device) for _ in range(LAYERS)]

    def matvec_only_pass():  # activations quantized beforehand into `scratch`: the mat-vec arithmetic alone
        for w, y, s in zip(ws, ys_mv, scratch):
            st = L.fuelq_qmatmul_packed(int(T.Q4K), M_ROWS, n_loc, K_IN, w.data_ptr(), s.data_ptr(), y.data_ptr(), sptr)
            if st:
                _lib.check(st, "fuelq_qmatmul_packed")

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.cuda.stream(stream):
        one_pass()  # eager once: sets kernel attributes outside capture
        for x, sc in zip(xs, scratch):
            _lib.check(L.fuelq_quantize_act_packed(int(T.Q4K), M_ROWS, K_IN, x.data_ptr(), sc.data_ptr(), ws_bytes, sptr),
                       "fuelq_quantize_act_packed")
        matvec_only_pass()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        graph_mv = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph_mv, stream=stream):
            matvec_only_pass()

        sampler = ClockSampler(local_rank)
        sampler.start()
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.time()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        barrier()
        t_wall1 = time.time()
        ms_total = max_over_ranks(e0.elapsed_time(e1))
        if t_wall1 - t_wall0 < 0.4:  # region shorter than the sampler period: hold the same load a little longer
            t_end = time.time() + 0.6
            while time.time() < t_end:
                for _ in range(50):
                    graph.replay()
                stream.synchronize()
            t_wall1 = time.time()
        clocks = sampler.summary(t_wall0, t_wall1)

        # dominant kernel alone (activations already quantized): average launch duration
        for _ in range(3):
            graph_mv.replay()
        stream.synchronize()
        reps = max(args.steps, 50)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(reps):
            graph_mv.replay()
        k1.record(stream)
        stream.synchronize()
        mv_only_us = k0.elapsed_time(k1) * 1e3 / (reps * LAYERS)
        fused = L.fuelq_get_option(_lib.OPT_FUSED_QUANT) == 1

        # end to end through the host-buffer entry point: pinned x in, y out, every mat-vec
        # (with several GPUs every rank does this for its rows; the host ends up with its slice of each y)
        hws_bytes = L.fuelq_qmatmul_host_workspace_bytes(int(T.Q4K), M_ROWS, n_loc, K_IN)
        hws = [torch.empty(hws_bytes, dtype=torch.uint8, device=device) for _ in range(LAYERS)]
        xh = [x.cpu().pin_memory() for x in xs]
        yh = [torch.empty(M_ROWS, n_loc).pin_memory() for _ in range(LAYERS)]

        def host_pass():
            for w, x, y, s in zip(ws, xh, yh, hws):
                st = L.fuelq_qmatmul_host(int(T.Q4K), M_ROWS, n_loc, K_IN, w.data_ptr(), x.data_ptr(), y.data_ptr(),
                                          s.data_ptr(), hws_bytes, sptr)
                if st:
                    _lib.check(st, "fuelq_qmatmul_host")
            stream.synchronize()  # the step's results are read on the host

        for _ in range(args.warmup):
            host_pass()
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record(stream)
        e2e_steps = args.steps
        for _ in range(e2e_steps):
            host_pass()
        h1.record(stream)
        stream.synchronize()
        e2e_ms = max_over_ranks(h0.elapsed_time(h1))
        sampler.stop()

    torch.cuda.synchronize()
    assert ops.device_error() == 0, "a kernel recorded an expired bounded wait"
    # the graph path and the host path must agree bit for bit on the last layer
    assert torch.equal(ys_mv[-1].cpu(), yh[-1]), "graph and host-buffer results differ"
    if world == 1:
        assert torch.equal(ys[-1], ys_mv[-1]), "one-kernel and two-kernel results differ"
    else:
        # the gathered vector of the last matrix: this rank's rows are its own product, and every rank holds the same vector
        y_all = region.view(f"y{LAYERS - 1}", 8 * N_OUT, torch.float32)[0::2].clone()
        assert torch.equal(y_all[lo:hi], ys_mv[-1][0]), "the gathered y does not hold this rank's rows"
        chk = torch.stack([y_all.double().sum(), picks[-1].double()])
        every = [torch.empty_like(chk) for _ in range(world)]
        dist.all_gather(every, chk)
        assert all(torch.equal(e, every[0]) for e in every), "ranks disagree on the gathered y"

    decode_7b, prefill_sharded, moe_ep, config0 = None, None, None, None
    del hws, scratch
    if region is not None:
        torch.cuda.synchronize()
        dist.barrier()
        region.close()
    torch.cuda.empty_cache()
    if world == 1 and not args.no_cpu_baseline:
        config0 = run_config0(torch, device, args.pdl)
        torch.cuda.empty_cache()
    prefill, moe_block = None, None
    if not args.no_model:
        decode_7b = run_decode_7b(torch, dist, device, rank, world)
        if world == 1:  # configurations 3 (prefill GEMM) and 5 (MoE block) on this GPU
            torch.cuda.empty_cache()
            prefill = list(side_lines(args, "prefill"))[0]
            torch.cuda.empty_cache()
            moe_block = list(side_lines(args, "moe"))[0]
        if world > 1:  # the other two multi-GPU forms at the same GPU count
            torch.cuda.empty_cache()
            prefill_sharded = run_prefill_sharded(args, rank, local_rank, world, own_group=False)
            torch.cuda.empty_cache()
            moe_ep = run_moe_expert_parallel(args, rank, local_rank, world, own_group=False)

    ms_per_step = ms_total / args.steps
    value = LAYERS * ALGO_BYTES / (ms_per_step * 1e-3) / 1e9      # the whole job: the same 32 matrices at every GPU count
    e2e_value = LAYERS * ALGO_BYTES / (e2e_ms / e2e_steps * 1e-3) / 1e9
    peak, peak_kind = _peaks()
    # the dominant kernel: with in-kernel activation quantization the step IS one kernel per matrix, timed above
    kern_us = ms_per_step * 1e3 / LAYERS if (fused and world == 1) else mv_only_us
    algo_launch = W_BYTES // N_OUT * n_loc + 4 * M_ROWS * K_IN + 4 * M_ROWS * n_loc   # this GPU's rows of one matrix
    achieved = algo_launch / (kern_us * 1e-6) / 1e9

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle as O
        threads = host_threads(O)
        w_host = [ws[i].cpu().numpy() for i in range(4)]
        x_host = [xs[i].cpu().numpy() for i in range(4)]
        # parity spot check beside the timing: GPU output vs the CPU path on layer 0
        r = O.matmul(O.Q4K, x_host[0], w_host[0], N_OUT, O.SCALAR, threads)
        err = float(np.abs(ys[0].cpu().numpy() - r).max() / np.abs(r).max())
        assert err <= 2e-6, f"GPU result off the CPU path by {err}"
        cpu_pass(O, w_host, x_host, threads)
        n_mv, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 10.0:
            cpu_pass(O, w_host, x_host, threads)
            n_mv += 4
        dt = time.perf_counter() - t0
        cpu_baseline = {"value": ALGO_BYTES * n_mv / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                        "sample": f"{n_mv} mat-vecs over 4 of the {LAYERS} matrices in {dt:.1f} s (AVX2 order, OpenMP)",
                        "parity_max_rel_err_vs_gpu": err}

    traffic = None
    try:  # per-launch DRAM bytes from the committed ncu summary, if present
        with open(os.path.join(ROOT, "profiles", "decode_q4k_m1_traffic.json")) as f:
            traffic = json.load(f).get("dram_bytes_per_launch")
    except Exception:
        pass

    line = {
        "metric": "q4k_qmatmul_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": bench_scaling(world),
        "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": bench_config(world, bool(args.pdl)),
        "pct_of_8tbs": value / world / 8000.0 * 100.0,   # per GPU
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "decode_regs_kernel<Q4KRegs,1,1>",
                     "avg_launch_us": kern_us, "algorithmic_bytes_per_launch": algo_launch,
                     "activation_quantization": "inside the kernel" if fused else "separate kernel, not in this figure",
                     "prequantized_activations_avg_launch_us": mv_only_us},
        "cpu_baseline": cpu_baseline,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": world * LAYERS * M_ROWS * K_IN * 4,
                "d2h_bytes_per_step": LAYERS * M_ROWS * N_OUT * 4, "ms_per_step": e2e_ms / e2e_steps,
                "api": "fuelq_qmatmul_host (pinned host x in, host y out, per mat-vec" +
                       ("" if world == 1 else "; every rank its rows of each matrix, no exchange") + ")"},
        "gpu_launches": args.steps * LAYERS * (3 if world > 1 else 1 if fused else 2) * world,
        "clocks": clocks,
        "decode_7b": decode_7b,
    }
    if config0 is not None:
        line["config0"] = config0
    if prefill is not None:
        line["prefill"] = prefill
        line["moe_block"] = moe_block
    if world > 1:
        line["exchange"] = ("per mat-vec: each rank's kernel stores its rows of y as stamped 8-byte pairs into every GPU's copy over "
                            "NVLink; a consumer kernel on every GPU polls its copy until complete (no collective, no multicast)")
        line["prefill_sharded"] = prefill_sharded
        line["moe_ep"] = moe_ep
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
