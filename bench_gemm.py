#!/usr/bin/env python
"""Dense-layer GEMM benchmark: the hand-written tcgen05/TMEM TF32 kernel (``ops.dense.gemm_tn``) against
cuBLAS through ``torch.matmul`` with TF32 enabled, on fully-connected-layer shapes.

  python bench_gemm.py                       # default shapes
  python bench_gemm.py --shapes 4096x4096x4096 --iters 20

Prints one JSON line per shape: TFLOP/s of both, their ratio and the maximum deviation from an fp64
product.  Inputs are larger than L2 for the big shapes; a 256 MiB buffer is rewritten between timed
calls for the small ones (L2 flush).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main() -> None:
    import torch

    from parameter_server_b200.ops import dense

    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="1024x1024x1024,4096x4096x4096,8192x1024x4096,16384x256x1024")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--act", default="IDENTITY")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.backends.cuda.matmul.allow_tf32 = True
    for shape in args.shapes.split(","):
        M, N, K = (int(x) for x in shape.split("x"))
        a = torch.randn(M, K, device=dev)
        b = torch.randn(N, K, device=dev) / K ** 0.5
        out = torch.empty(M, N, device=dev)

        def timed(fn):
            for _ in range(args.warmup):
                fn()
            ms = []
            for _ in range(args.iters):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1))
            return sorted(ms)[len(ms) // 2]

        ms_ours = timed(lambda: dense.gemm_tn(a, b, args.act, out=out))
        dense.check_status(dev)
        ms_blas = timed(lambda: torch.matmul(a, b.T, out=out))
        ref = (a[:256].double() @ b.double().T).float()
        got = dense.gemm_tn(a, b, "IDENTITY")[:256]
        flops = 2.0 * M * N * K
        print(json.dumps({"shape": [M, N, K], "tcgen05_ms": ms_ours, "tcgen05_tflops": flops / ms_ours / 1e9,
                          "cublas_tf32_ms": ms_blas, "cublas_tf32_tflops": flops / ms_blas / 1e9,
                          "ratio_vs_cublas": ms_blas / ms_ours, "max_abs_err_vs_fp64": (got - ref).abs().max().item()}), flush=True)


if __name__ == "__main__":
    main()
