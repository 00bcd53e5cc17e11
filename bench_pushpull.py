#!/usr/bin/env python
"""Push / pull microbenchmark on key-range sharded peer memory, against the NCCL all-to-all baseline.

Key sets of n uint64 keys (Zipf(1.1) over a 2^32 key space, de-duplicated) with value lengths
1 / 8 / 64 fp32, sharded by key range over the GPUs.  For each (n, k) it times
  * pull  — one kernel gathering rows from the owners over NVLink (``DeviceKVVector.pull``)
  * push  — one kernel reducing rows into the owners with ``red.add`` (``DeviceKVVector.push``)
  * the same two operations with ``all_to_all_single`` + local gather / scatter-add kernels
and the two fused FTRL kernels (pull+SpMV, push+update) through their in-kernel phase marks.
It reports GB/s of value payload per GPU and the fraction of the NVLink roofline
(bytes that must cross NVLink / 770 GB/s measured peer-copy bandwidth per direction per GPU).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
      --master-port 29533 bench_pushpull.py --sizes 1000,100000,10000000 --klens 1,8,64
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NVLINK_GBS = 770.0


def main() -> None:
    import torch

    from parameter_server_b200.data.synthetic import mix64, zipf_ranks
    from parameter_server_b200.ops import sparse
    from parameter_server_b200.parallel.kv_vector import DeviceKVVector
    from parameter_server_b200.parallel.peer import PeerGroup

    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1000,100000,10000000")
    ap.add_argument("--klens", default="1,8,64")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    group = PeerGroup.from_env()
    dev, rank, W = group.device, group.rank, group.world
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    results = []

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        group.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return group.all_reduce_max(e0.elapsed_time(e1)) / args.iters

    for n in [int(x) for x in args.sizes.split(",")]:
        ranks = zipf_ranks(int(n * 1.3) + 16, 1.1, 1 << 32, gen, dev)
        keys, _ = sparse.count_unique(mix64(ranks))          # hashed, de-duplicated, unsigned order
        keys = keys[torch.randperm(keys.numel(), generator=gen, device=dev)[:n]].contiguous()
        for k in [int(x) for x in args.klens.split(",")]:
            if keys.numel() * k * 4 > (8 << 30):
                continue
            row = {"n_keys": int(keys.numel()), "value_len": k, "n_gpus": W}
            for impl in ("fused", "nccl"):
                kv = DeviceKVVector(group, k=k, impl=impl)
                kv.set_keys(kv.merge_keys(keys))
                owner, slot = kv.resolve(keys)
                vals = torch.randn(keys.numel(), k, device=dev)
                out = torch.empty_like(vals)
                ms_pull = timeit(lambda: kv.pull(owner, slot, out))
                ms_push = timeit(lambda: kv.push(owner, slot, vals))
                payload = keys.numel() * k * 4
                remote = payload * (W - 1) / max(W, 1)
                for name, ms in (("pull", ms_pull), ("push", ms_push)):
                    row[f"{impl}_{name}_ms"] = ms
                    row[f"{impl}_{name}_gbs"] = payload / ms / 1e6
                    row[f"{impl}_{name}_roofline_frac"] = (remote / (NVLINK_GBS * 1e6)) / ms if W > 1 else None
                del kv
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0:
        print(json.dumps({"summary": "push/pull microbenchmark", "rows": len(results), "nvlink_gbs_used": NVLINK_GBS}))
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
