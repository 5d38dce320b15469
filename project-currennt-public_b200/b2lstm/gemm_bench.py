"""Micro-benchmark of b2_matrix_multiply (the helpers::Matrix GEMM wrapper): tensor-core 3xTF32
kernel against the FFMA kernel on one shape, with the error of both against float64.

    python -m b2lstm.gemm_bench --m 2048 --n 38240 --k 512 --ta 1 --tb 0 [--iters 10] [--ffma 0|1]

--ta/--tb are the transpose flags of the reference's Matrix::assignProduct (column-major operands):
  ta=1 tb=0  K-major x K-major   (input projection:  W^T X)
  ta=0 tb=0  MN-major x K-major  (error back-projection: W delta)
  ta=0 tb=1  MN-major x MN-major (weight gradient: X delta^T)
The timed region contains the operand split kernels and the GEMM; TFLOP/s counts 2*m*n*k.
"""
import argparse
import json

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=38240)
    ap.add_argument("--k", type=int, default=512)
    ap.add_argument("--ta", type=int, default=1)
    ap.add_argument("--tb", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ffma", type=int, default=0)
    ap.add_argument("--check", type=int, default=1)
    a = ap.parse_args()
    import torch
    import b2lstm
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(1)
    m, n, k = a.m, a.n, a.k
    A = torch.randn((k, m) if not a.ta else (m, k), device=dev, generator=g)
    B = torch.randn((n, k) if not a.tb else (k, n), device=dev, generator=g)
    C = torch.zeros((n, m), device=dev)
    lda = m if not a.ta else k
    ldb = k if not a.tb else n

    def run():
        b2lstm.matrix_multiply(C, m, A, lda, a.ta, B, ldb, a.tb, m, n, k, accumulate=False, force_ffma=bool(a.ffma))

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    out = {"m": m, "n": n, "k": k, "ta": a.ta, "tb": a.tb, "kernel": "ffma" if a.ffma else "tcgen05_3xtf32",
           "ms": ms, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12}
    if a.check:
        rows = min(m, 64)
        opA = (A.T if not a.ta else A)[:rows].double()
        opB = (B.T if not a.tb else B).double()
        want = (opA @ opB).cpu().numpy()
        got = C.T[:rows].double().cpu().numpy()
        out["rel_l2_err_vs_f64"] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
