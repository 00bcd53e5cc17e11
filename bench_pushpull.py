#!/usr/bin/env python
"""Push / pull microbenchmark on key-range sharded peer memory, against the NCCL all-to-all baseline.

Key sets of n uint64 keys (Zipf(1.1) over a 2^32 key space, de-duplicated) with value lengths
1 / 8 / 64 fp32, sharded by key range over the GPUs.  For each (n, k) it times
  * pull  — one kernel gathering rows from the owners over NVLink (``DeviceKVVector.pull``)
  * push  — one kernel reducing rows into the owners with ``red.add`` (``DeviceKVVector.push``)
  * the same two operations with ``all_to_all_single`` + local gather / scatter-add kernels
and, with ``--fused``, the two fused FTRL kernels on a minibatch whose n non-zeros are n distinct keys
(32 per row, value length 1): pull + SpMV (``psb_ftrl_pull_spmv``) and push + FTRL update
(``psb_ftrl_push_update``), each timed alone with CUDA events, against the NCCL-only engine's pull and
push of the same minibatch.  It reports GB/s of payload per GPU and the fraction of the NVLink roofline
(bytes that must cross NVLink / 770 GB/s measured peer-copy bandwidth per direction per GPU); for the
fused kernels the payload is 12 bytes per key for the pull (key out, weight back) and 4 bytes for the
push (gradient), and small key sets are reported as latency.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
      --master-port 29533 bench_pushpull.py --sizes 1000,100000,10000000 --klens 1,8,64 --fused
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
    import ctypes as C

    import torch

    from parameter_server_b200.data.synthetic import mix64, zipf_ranks
    from parameter_server_b200.ops import _native as N
    from parameter_server_b200.ops import sparse
    from parameter_server_b200.parallel.kv_vector import DeviceKVVector
    from parameter_server_b200.parallel.peer import PeerGroup

    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1000,100000,10000000")
    ap.add_argument("--klens", default="1,8,64")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--fused", action="store_true", help="also time the fused FTRL pull+SpMV / push+update kernels")
    ap.add_argument("--no-kv", action="store_true", help="skip the plain key-value push / pull kernels")
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

    def fused_row(keys):
        """Pull+SpMV and push+update of a minibatch with one non-zero per key, fused kernels against the NCCL engine."""
        from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper, _pow2_at_least

        n = keys.numel()
        per_row = 32
        rows = (n + per_row - 1) // per_row
        off = torch.clamp(torch.arange(rows + 1, device=dev, dtype=torch.int64) * per_row, max=n)
        y = torch.where(torch.rand(rows, generator=gen, device=dev) < 0.5, 1.0, -1.0).to(torch.float32)
        mb = DeviceMinibatch(off, keys, y)
        iters = args.iters if n <= 20_000_000 else max(args.iters // 4, 3)
        row = {"kind": "fused_ftrl", "n_keys": int(n), "value_len": 1, "n_gpus": W}
        for impl in ("fused", "nccl"):
            eng = FTRLEngine(group, FTRLHyper(alpha=0.1, beta=1.0, lambda1=1.0, lambda2=0.1, rule="sumsq"),
                             table_capacity=_pow2_at_least(3 * n), max_rows=rows, max_nnz=n,
                             local_capacity=_pow2_at_least(int(1.7 * n) + 4096 * W), timeout_s=10.0, impl=impl)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            t_pull = t_push = 0.0
            for it in range(args.warmup + iters):
                if impl == "fused":
                    M = eng._mb(mb)
                    eng._L.parity = (eng.push_seq + 1) & 1
                    ev[0].record()
                    eng._launch_pull(M, insert=True)
                    ev[1].record()
                    eng.push_seq += 1
                    N.check(eng._lib.psb_ftrl_push_update(C.byref(eng._P), C.byref(M), C.byref(eng._L), C.byref(eng._H),
                                                          C.c_uint32(eng.push_seq), N.stream_ptr()), "ftrl_push_update")
                    ev[2].record()
                else:
                    M = eng._mb(mb)
                    ev[0].record()
                    ctx = eng._pull_nccl(M)
                    ev[1].record()
                    eng._push_nccl(M, *ctx)
                    ev[2].record()
                torch.cuda.synchronize(dev)
                if it >= args.warmup:
                    t_pull += ev[0].elapsed_time(ev[1])
                    t_push += ev[1].elapsed_time(ev[2])
            eng.check_status()
            ms_pull = group.all_reduce_max(t_pull / iters)
            ms_push = group.all_reduce_max(t_push / iters)
            remote = (W - 1) / max(W, 1)
            for name, ms, bytes_per_key in (("pull", ms_pull, 12), ("push", ms_push, 4)):
                row[f"{impl}_{name}_us"] = ms * 1e3
                row[f"{impl}_{name}_gbs"] = n * bytes_per_key / ms / 1e6
                row[f"{impl}_{name}_roofline_frac"] = (n * bytes_per_key * remote / (NVLINK_GBS * 1e6)) / ms if W > 1 else None
            del eng
            torch.cuda.empty_cache()
        return row

    for n in [int(x) for x in args.sizes.split(",")]:
        ranks = zipf_ranks(int(n * 1.3) + 16, 1.1, 1 << 32, gen, dev)
        keys, _ = sparse.count_unique(mix64(ranks))          # hashed, de-duplicated, unsigned order
        keys = keys[torch.randperm(keys.numel(), generator=gen, device=dev)[:n]].contiguous()
        if args.fused:
            row = fused_row(keys)
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        for k in [] if args.no_kv else [int(x) for x in args.klens.split(",")]:
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
