#!/usr/bin/env python
"""Key-set / sparse-matrix preprocessing kernels: stable uint64 radix sort with payload, unique with counts,
dictionary remap and CSR→CSC transposition, timed on one GPU against the torch (CUB) equivalents.

  python bench_sparse.py --n 50000000 [--bits 30]

Prints one JSON line per operation: milliseconds, keys/s, and the time of the library counterpart.
Inputs are larger than L2 (n uint64 keys = 8n bytes).
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

    from parameter_server_b200.data.synthetic import mix64, zipf_ranks
    from parameter_server_b200.ops import sparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=50_000_000)
    ap.add_argument("--bits", type=int, default=64, help="significant key bits (fewer bits = fewer radix passes)")
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    keys = mix64(zipf_ranks(args.n, 1.1, 1 << 30, gen, dev))
    if args.bits < 64:
        keys = keys & ((1 << args.bits) - 1)
    vals = torch.arange(args.n, dtype=torch.int32, device=dev)

    def timed(fn):
        fn()
        ms = []
        for _ in range(args.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        return sorted(ms)[len(ms) // 2], out

    ms, (sk, sv) = timed(lambda: sparse.sort_pairs(keys, vals))
    ms_t, _ = timed(lambda: torch.sort(keys ^ (-(1 << 63)), stable=True))
    print(json.dumps({"op": "radix_sort_u64_pairs", "n": args.n, "bits": args.bits, "ms": ms, "mkeys_per_s": args.n / ms / 1e3,
                      "torch_sort_ms": ms_t}), flush=True)
    ms, (uk, cnt) = timed(lambda: sparse.unique_sorted(sk))
    ms_t, _ = timed(lambda: torch.unique_consecutive(sk, return_counts=True))
    print(json.dumps({"op": "unique_with_counts", "n": args.n, "unique": int(uk.numel()), "ms": ms, "torch_ms": ms_t}), flush=True)
    ms, idx = timed(lambda: sparse.remap(keys, uk))
    ms_t, _ = timed(lambda: torch.searchsorted(uk ^ (-(1 << 63)), keys ^ (-(1 << 63))))
    print(json.dumps({"op": "remap", "n": args.n, "ms": ms, "torch_searchsorted_ms": ms_t}), flush=True)
    rows = args.n // 100
    off = torch.arange(0, rows * 100 + 1, 100, dtype=torch.int64, device=dev)
    col = idx[: rows * 100].contiguous()
    ms, _ = timed(lambda: sparse.csr_to_csc(off, col, None, int(uk.numel())))
    print(json.dumps({"op": "csr_to_csc", "nnz": rows * 100, "cols": int(uk.numel()), "ms": ms}), flush=True)


if __name__ == "__main__":
    main()
