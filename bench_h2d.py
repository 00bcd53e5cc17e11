#!/usr/bin/env python
"""Host-to-device copy throughput from pinned memory for different copy sizes (one stream, nothing else running).

  python bench_h2d.py [--total-mb 400]

The streaming paths (online minibatches, out-of-core column blocks) issue one cudaMemcpyAsync per minibatch
or block; this shows what the host link of the box gives at those sizes.  Prints one line per size.
"""
from __future__ import annotations

import argparse


def main() -> None:
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--total-mb", type=int, default=400)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    total = args.total_mb << 20
    host = torch.empty(total, dtype=torch.uint8).pin_memory()
    dst = torch.empty(total, dtype=torch.uint8, device=dev)
    for size in (1 << 20, 1350000, 4 << 20, 21 << 20, 77 << 20, total):
        n = max(total // size, 1)
        for _ in range(2):                      # the second round is the measurement
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n):
                dst[i * size:(i + 1) * size].copy_(host[i * size:(i + 1) * size], non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        print(f"copy size {size / 1e6:8.2f} MB x {n:4d}: {ms:7.2f} ms  {n * size / ms / 1e6:6.1f} GB/s", flush=True)


if __name__ == "__main__":
    main()
