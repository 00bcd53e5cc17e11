#!/usr/bin/env python
"""Headline benchmark: examples/sec of CTR-scale online FTRL-proximal (L1-LR) on N B200s.

Config (the CTR-scale FTRL configuration of the baseline): hashed uint64 keys over a 2^30-key
space drawn Zipf(1.1), 12 feature groups x ~8 binary features (~96-100 nnz/row), minibatches of
100,000 rows per GPU (weak scaling: every GPU streams its own minibatches), labels
Bernoulli(sigmoid(X.w* - 3.2)), per-key fp32 state, alpha=0.1 beta=1 lambda1=1 lambda2=0.1.
A step = one minibatch per GPU through the pull-fused SpMV and the push-fused FTRL update.

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

``value`` is device-timed (CUDA events, max over ranks) on minibatches resident on the device
(a ring of distinct minibatches larger than L2); ``e2e`` times the public streaming API
(`FTRLTrainer.train`) including the pinned host->device copy of every minibatch and the
device->host read of every step's loss.  ``--impl nccl`` runs the unfused NCCL baseline of the
same algorithm; ``--impl reference`` reports why the CPU/ZeroMQ reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REFERENCE_UNAVAILABLE = ("reference is a CPU-only C++/ZeroMQ program with a make build and no Python package: "
                         "pip install of the reference tree fails (no setup.py/pyproject.toml) and its build needs "
                         "zeromq, gflags, glog, protobuf+protoc, snappy, eigen3, tcmalloc, none present offline")

CLOCK_QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
               "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples this rank's GPU clocks with nvidia-smi while the timed region runs."""

    def __init__(self, device):
        import torch

        self.proc, self.path = None, f"/tmp/psb_clocks_{os.getpid()}.csv"
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.cmd = ["nvidia-smi", "-i", uuid, f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                        "-lms", "100"]
        except Exception:
            self.cmd = None

    def start(self):
        if self.cmd:
            try:
                self.proc = subprocess.Popen(self.cmd, stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            except Exception:
                self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0])); mx.append(float(f[1]))
                except ValueError:
                    continue
                for n, v in zip(names, f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def run_ftrl(args) -> dict:
    import torch

    from parameter_server_b200.data.synthetic import ctr_minibatch
    from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper
    from parameter_server_b200.models.ftrl_trainer import FTRLTrainer, HostMinibatch
    from parameter_server_b200.parallel.peer import PeerGroup

    group = PeerGroup.from_env()
    dev, rank, world = group.device, group.rank, group.world
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    rows, ring = args.rows, args.ring
    batches = []
    for i in range(ring):
        off, keys, y = ctr_minibatch(rows, seed=1000 * rank + i + 1, device=dev)
        batches.append(DeviceMinibatch(off, keys, y))
    max_nnz = max(b.nnz for b in batches)
    eng = FTRLEngine(group, FTRLHyper(alpha=0.1, beta=1.0, lambda1=1.0, lambda2=0.1, rule=args.rule),
                     table_capacity=1 << args.table_log2, max_rows=rows, max_nnz=max_nnz,
                     local_capacity=1 << args.local_log2, timeout_s=args.timeout_s,
                     impl="nccl" if args.impl == "nccl" else "fused",
                     track_counts=True if args.track_counts else None)
    # ---------------------------------------------------------------- device-resident timing
    for i in range(args.warmup):
        eng.step(batches[i % ring])
    eng.read_stats()
    eng.check_status()
    group.barrier()
    sampler = ClockSampler(dev)
    sampler.start()
    launches0 = eng.kernel_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        eng.step(batches[(args.warmup + i) % ring])
    e1.record()
    torch.cuda.synchronize(dev)
    ms = group.all_reduce_max(e0.elapsed_time(e1))
    group.barrier()
    launches = eng.kernel_launches - launches0
    phases = eng.phase_times_us() if args.impl != "nccl" else None
    st = eng.read_stats()
    eng.check_status()
    # ---------------------------------------------------------------- end to end (public API)
    ex_per_step = rows * world
    e2e = None
    if not args.no_e2e:
        host = [HostMinibatch(b.offsets.cpu(), b.keys.cpu(), b.y.cpu()).pin() for b in batches]
        trainer = FTRLTrainer(eng)
        trainer.train(host[i % ring] for i in range(max(3, args.warmup)))
        group.barrier()
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        losses = trainer.train(host[i % ring] for i in range(args.steps))
        t1.record()
        torch.cuda.synchronize(dev)
        e2e_ms = group.all_reduce_max(t0.elapsed_time(t1))
        e2e = {"value": ex_per_step * args.steps / (e2e_ms / 1e3), "unit": "examples/s",
               "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": trainer.h2d_bytes // args.steps,
               "d2h_bytes_per_step": trainer.d2h_bytes // args.steps,
               "mean_logloss_last": losses[-1] if losses else None,
               "h2d_gbs_per_gpu": trainer.h2d_bytes / args.steps / (e2e_ms / args.steps) / 1e6,
               "numa": getattr(group, "numa", None)}
    clocks = sampler.stop()
    group.barrier()
    return {
        "metric": "examples/sec (online FTRL-proximal L1-LR, CTR-scale stream)",
        "value": ex_per_step * args.steps / (ms / 1e3),
        "unit": "examples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic",
        "impl": "nccl-baseline" if args.impl == "nccl" else "fused",
        "config": {"model": "FTRL-proximal logistic regression, 2^30 hashed uint64 keys Zipf(1.1), ~96 nnz/row, "
                            "alpha=0.1 beta=1 lambda1=1 lambda2=0.1, per-key fp32 state, rule=" + args.rule,
                   "global_batch": ex_per_step, "seq_len": None, "nnz_per_row": max_nnz / rows,
                   "parallelism": f"dp{world} x key-range shards {world} (worker+server per GPU)",
                   "l2_policy": f"inputs larger than L2: ring of {ring} distinct minibatches "
                                f"({batches[0].nbytes() >> 20} MiB each) plus {max_nnz * 4 >> 20} MiB slot map per step",
                   "mean_logloss_last": st["loss_sum"] / max(st["rows"], 1), "nnz_w": st["nnz_w"],
                   "unique_keys_per_step": st["unique_keys"] / max(args.steps, 1),
                   "phase_us_last_step_rank0": phases},
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clocks,
    }, rank


def run_darlin(args):
    """Batch L1-LR by DARLIN block coordinate descent on the medium sparse configuration: 677,399 rows x
    47,236 features, ~74 nnz/row, Zipf(1.0) column ids, lognormal values with unit-norm rows, labels from
    a planted 2 % w*, lambda1 = 1.  A step is one pass over all feature blocks; the rows are split over
    the GPUs (strong scaling).  `value` times K passes from the initial state with the data resident on
    the GPUs; `e2e` times the out-of-core mode of the public solver: every pass streams all column blocks
    from pinned host memory and reads the objective back to the host."""
    import numpy as np
    import torch

    from parameter_server_b200.data.synthetic import zipf_sparse_matrix
    from parameter_server_b200.models.darlin import DarlinConfig, DarlinSolver, block_order
    from parameter_server_b200.parallel.peer import PeerGroup

    group = PeerGroup.from_env()
    dev, rank, world = group.device, group.rank, group.world
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    ooc_shape = args.config == "ooc"
    if ooc_shape:
        # the out-of-core configuration, scaled to --ooc-rows rows per GPU (weak scaling): ~120 binary features per
        # row, hashed uint64 keys over a 2^32 key space drawn Zipf(1.05), labels Bernoulli(sigmoid(X.w*)) from a
        # planted 0.5 % w*, lambda1 = 4, 64 feature blocks, KKT filter ratio 10
        from parameter_server_b200.data.synthetic import ctr_minibatch

        rows_total, cols = args.ooc_rows * world, 1 << 32
        off, idx, y = ctr_minibatch(args.ooc_rows, seed=31 + rank, device=dev, key_space_log2=32, zipf_s=1.05, groups=12,
                                    feats_lo=8, feats_hi=12, bias=0.0, wstar_frac=0.005, wstar_std=1.0)
        vals = None
        per_row = idx.numel() / max(args.ooc_rows, 1)
        cfg = DarlinConfig(lambda1=4.0, eta=1.0, delta_init=1.0, delta_max=5.0, kkt_ratio=10.0, max_pass=args.steps,
                           epsilon=0.0, feature_block_ratio=63.5 / per_row, random_block_order=True, seed=0,
                           max_block_delay=args.block_delay)
    else:
        rows_total, cols = args.darlin_rows, 47236
        r0, r1 = rows_total * rank // world, rows_total * (rank + 1) // world
        # every rank generates the same matrix chunk-wise and keeps its rows (no file system, no network)
        off, idx, vals, y, _ = zipf_sparse_matrix(r1 - r0, cols, 90, seed=17 + rank, device=dev, zipf_s=1.0, wstar_frac=0.02,
                                                 noise=0.3, wstar_seed=4242)
        cfg = DarlinConfig(lambda1=1.0, eta=1.0, delta_init=5.0, delta_max=10.0, kkt_ratio=100.0, max_pass=args.steps,
                           epsilon=0.0, feature_block_ratio=4.0, random_block_order=True, seed=0,
                           max_block_delay=args.block_delay)
    impl = "nccl" if args.impl == "nccl" else "fused"

    def timed(sol, with_eval):
        orders = block_order(sol.nblk, args.warmup + args.steps, True, 0)
        for i in range(args.warmup):
            sol.launch_pass(orders[i])
        torch.cuda.synchronize(dev)
        sol.check_status()
        sol.reset_state()
        l0, h0 = sol.kernel_launches, sol.h2d_bytes
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        objs = []
        e0.record()
        for i in range(args.steps):
            if with_eval:
                objs.append(sol.run_pass(orders[i]).objv)     # includes the device->host read of the objective
            else:
                sol.launch_pass(orders[i])
        e1.record()
        torch.cuda.synchronize(dev)
        ms = group.all_reduce_max(e0.elapsed_time(e1))
        sol.check_status()
        return ms, sol.kernel_launches - l0, sol.h2d_bytes - h0, objs

    sol = DarlinSolver(group, cfg, timeout_s=args.timeout_s, impl=impl)
    sol.preprocess(off, idx, vals, y)
    nnz_total = int(group.all_reduce_sum([idx.numel()])[0])
    nblk = sol.nblk
    sampler = ClockSampler(dev)
    sampler.start()
    ms, launches, _, _ = timed(sol, False)
    objv, nnz_w, nnz_as, _ = sol.evaluate()
    e2e = None
    if not args.no_e2e and impl == "fused":
        del sol
        torch.cuda.empty_cache()
        ooc = DarlinSolver(group, cfg, timeout_s=args.timeout_s, impl="fused", out_of_core=True,
                           prefetch_depth=args.prefetch_depth)
        ooc.preprocess(off, idx, vals, y)
        ms2, _, h2d, objs = timed(ooc, True)
        e2e = {"value": rows_total * args.steps / (ms2 / 1e3), "unit": "examples/s", "ms_per_step": ms2 / args.steps,
               "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": 40, "objective_last": objs[-1] if objs else None,
               # time to objective: objective after every pass; pass i completes at (i+1) * ms_per_step
               "objective_trace": [round(o, 2) for o in objs]}
    clocks = sampler.stop()
    group.barrier()
    return {
        "metric": "examples/sec (L1-LR, DARLIN block coordinate descent, one pass = one step)",
        "value": rows_total * args.steps / (ms / 1e3), "unit": "examples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak" if ooc_shape else "strong", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic",
        "impl": "nccl-baseline" if impl == "nccl" else "fused",
        "config": {"model": ("out-of-core L1 logistic regression, DARLIN over 64 feature blocks, lambda1=4, KKT ratio 10, binary "
                             "features, uint64 keys over 2^32 Zipf(1.05); e2e streams every block from pinned host memory")
                            if ooc_shape else
                            "L1 logistic regression, DARLIN, lambda1=1, feature_block_ratio=4, delta 5/10, KKT ratio 100",
                   "global_batch": rows_total, "seq_len": None, "rows": rows_total, "features": cols,
                   "max_block_delay": args.block_delay,
                   "nnz_per_row": nnz_total / rows_total, "feature_blocks": nblk,
                   "parallelism": f"dp{world} rows x key-range shards {world} (worker+server per GPU)",
                   "l2_policy": f"inputs larger than L2: {nnz_total * (4 if vals is None else 8) >> 20} MiB of CSC row ids"
                                f"{'' if vals is None else ' and values'} read per pass",
                   "objective_after_timed_passes": objv, "nnz_w": nnz_w, "active_keys": nnz_as},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
    }, rank


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="ftrl", choices=["ftrl", "darlin", "ooc"],
                    help="ftrl: CTR-scale online FTRL (headline); darlin: batch L1-LR by block coordinate descent; "
                         "ooc: the out-of-core batch configuration (64 blocks, binary hashed features), scaled by --ooc-rows")
    ap.add_argument("--darlin-rows", type=int, default=677399)
    ap.add_argument("--ooc-rows", type=int, default=1000000, help="rows per GPU of the out-of-core configuration")
    ap.add_argument("--block-delay", type=int, default=0,
                    help="DARLIN bounded delay tau (max_block_delay): tau+1 blocks share their synchronisation points")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "fused", "nccl", "reference"])
    ap.add_argument("--rows", type=int, default=100000, help="minibatch rows per GPU")
    ap.add_argument("--ring", type=int, default=4, help="distinct minibatches per GPU")
    ap.add_argument("--table-log2", type=int, default=26, help="log2 slots of each GPU's shard table")
    ap.add_argument("--local-log2", type=int, default=22, help="log2 slots of the per-minibatch dedup table")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host-streaming) measurement")
    ap.add_argument("--rule", default="sumsq", choices=["count", "sumsq"],
                    help="per-key learning-rate statistic: reference count-based estimate or sum of g^2")
    ap.add_argument("--prefetch-depth", type=int, default=4,
                    help="DARLIN end-to-end run: column blocks in flight between pinned host memory and the GPU")
    ap.add_argument("--track-counts", action="store_true",
                    help="keep per-key pos/neg row counts although the sum-of-squares rule does not need them")
    ap.add_argument("--timeout-s", type=float, default=5.0, help="limit of in-kernel cross-GPU waits")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:       # one line per job, also under torch.distributed.run
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return
    if args.warmup < 3:
        args.warmup = 3
    result, rank = run_darlin(args) if args.config in ("darlin", "ooc") else run_ftrl(args)
    if rank == 0:
        print(json.dumps(result))
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
