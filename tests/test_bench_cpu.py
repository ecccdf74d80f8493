"""Host logic of bench.py that needs no GPU: the workload description both arms print, the roofline helpers, and the
reference arm itself (the CPU restatement of the reference's path on a short step), including what its ranks do under a
multi-process launch."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_both_arms_describe_the_same_workload():
    b = _bench()
    one, eight = b.bench_config(1, True), b.bench_config(8, True)
    assert one["workload"] == eight["workload"] and "model" not in one
    assert one["m"] == 1 and one["k"] == 4096 and one["n"] == 11008 and one["layers"] == 32
    assert "larger than L2" in one["l2"]
    assert b.bench_scaling(1) == b.bench_scaling(8) == "strong"
    # algorithmic bytes of one mat-vec: blocks + activations + result
    assert b.W_BYTES == 11008 * 16 * 144 and b.ALGO_BYTES == b.W_BYTES + 4 * 4096 + 4 * 11008


def test_roofline_helpers():
    b = _bench()
    peak, kind = b._peaks()
    assert peak > 1000 and kind in ("measured", "fallback")
    r = b.tensor_roofline(800.0)
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and r["achieved"] == 800.0
    assert abs(r["frac"] - 800.0 / r["peak"]) < 1e-12 and abs(r["frac_of_sustained"] - 800.0 / r["peak_sustained"]) < 1e-12
    assert r["peak_sustained"] <= r["peak"]


def test_reference_arm_prints_the_contract_line_and_only_rank_zero_works():
    env = dict(os.environ)
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3"]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600, check=True).stdout
    line = json.loads(out.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "q4k_qmatmul_hbm_gbs" and line["unit"] == "GB/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["config"] == _bench().bench_config(1, True)
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # a non-zero rank of a multi-process launch exits 0 without output
    env2 = dict(env, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    res = subprocess.run(cmd + ["--gpus", "2"], cwd=ROOT, env=env2, capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.strip() == ""
