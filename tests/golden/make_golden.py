"""Regenerates tests/golden/kquants_golden.npz.

The reference (Rust) cannot be built where this repository is developed, so the
fixture is produced by the CPU restatement under oracle/, after that restatement
has been checked against the reference's own known-answer tests and against
gguf-py's independent implementation of the same byte layouts (tests/test_oracle.py).
It freezes those results so any later drift in the restatement or in the CUDA
kernels shows up as a byte or bit difference.

Inputs: numpy Generator(PCG64(seed)); weights standard_normal*0.02 (seed 0),
activations standard_normal (seed 1) — the distributions of the benchmark configs
at a size small enough to commit.

Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

N, K, M = 6, 512, 3


def inputs():
    w = np.random.Generator(np.random.PCG64(0)).standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    x = np.random.Generator(np.random.PCG64(1)).standard_normal((M, K), dtype=np.float32)
    # edge rows: an all-zero super-block, a +v/-v tie (first wins), exact .5 rounding cases
    x[1, :256] = 0.0
    x[2, 0] = 3.0
    x[2, 5] = -3.0
    x[2, 6:10] = [0.01171875, 0.03515625, -0.01171875, 1.5]
    return w, x


def main():
    w, x = inputs()
    out = {"w": w, "x": x}
    for name, t in (("q4_0", O.Q4_0), ("q4_1", O.Q4_1), ("q5_0", O.Q5_0), ("q5_1", O.Q5_1), ("q8_0", O.Q8_0), ("q2k", O.Q2K), ("q3k", O.Q3K), ("q4k", O.Q4K),
                    ("q5k", O.Q5K), ("q6k", O.Q6K)):
        wb = O.quantize(t, w, nthreads=1)
        out[f"{name}_blocks"] = wb
        out[f"{name}_dequant"] = O.dequantize(t, wb)
        out[f"{name}_act"] = O.quantize_act(t, x)
        out[f"{name}_y_scalar"] = O.matmul(t, x, wb, N, O.SCALAR)
        out[f"{name}_y_avx2"] = O.matmul(t, x, wb, N, O.AVX2)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kquants_golden.npz")
    np.savez_compressed(path, **out)
    h = hashlib.sha256(open(path, "rb").read()).hexdigest()
    print(path, os.path.getsize(path), "bytes sha256", h)


if __name__ == "__main__":
    main()
