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
                        "-lms", "50"]
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


def _cpu_ftrl_arm(rows: int, steps: int) -> dict:
    """The host runtime's own online step (what a CPU worker + CPU server do per minibatch: radix localizer,
    model lookup, threaded margins / loss / gradient, per-key FTRL update; csrc/host) on a sub-sample of the
    same stream, all cores of this machine, no network in between."""
    import numpy as np

    from parameter_server_b200.data.synthetic import ctr_minibatch
    from parameter_server_b200.runtime import host

    H = host()
    threads = os.cpu_count() or 1
    model = H.FTRLModel(0.1, 1.0, 1.0, 0.1)
    data = []
    for i in range(steps + 1):
        off, keys, y = ctr_minibatch(rows, seed=900001 + i, device="cpu")
        data.append((off.numpy(), keys.numpy().view(np.uint64), y.numpy().astype(np.float64)))
    t0 = None
    for i, (off, keys, y) in enumerate(data):
        if i == 1:
            t0 = time.perf_counter()        # the first minibatch warms the code up
        ukeys, _, loc = H.localize(keys)
        w = model.get(ukeys)
        _, g, pos, neg = H.ftrl_minibatch(off, loc, None, y, w, threads)
        model.update(ukeys, g, pos, neg)
    dt = time.perf_counter() - t0
    return {"value": rows * steps / dt, "unit": "examples/s", "rows_per_minibatch": rows, "minibatches": steps,
            "threads": threads, "what": "native host runtime step (localize, lookup, minibatch gradient, FTRL update), "
                                        "count rule, in-process, declared sub-sample of the same stream"}


def run_ftrl(args) -> dict:
    import torch

    from parameter_server_b200.data.synthetic import ctr_minibatch
    from parameter_server_b200.models.ftrl import KEY_U32_HASHED, DeviceMinibatch, FTRLEngine, FTRLHyper
    from parameter_server_b200.models.ftrl_trainer import FTRLTrainer, HostMinibatch
    from parameter_server_b200.parallel.peer import PeerGroup

    group = PeerGroup.from_env()
    dev, rank, world = group.device, group.rank, group.world
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    rows = args.rows
    # every step of warm-up and of the timed region gets a minibatch of its own, so that the timed steps
    # meet keys that the model has not seen (entries are created inside the timed region)
    # (at most 48 per GPU: beyond that the stream wraps around and `new_keys_per_step` says so)
    ring = min(max(args.ring, args.warmup + args.steps), max(args.ring, 48))
    if args.ring < 0:
        ring = -args.ring        # replay exactly this many minibatches (after warm-up no step creates a key)
    batches, ids = [], []
    for i in range(ring):
        off, keys, y, fid = ctr_minibatch(rows, seed=1000 * rank + i + 1, device=dev, return_ids=True)
        batches.append(DeviceMinibatch(off, keys, y))
        ids.append(fid)
    max_nnz = max(b.nnz for b in batches)
    hyper = FTRLHyper(alpha=0.1, beta=1.0, lambda1=1.0, lambda2=0.1, rule=args.rule)

    def engine(impl):
        return FTRLEngine(group, hyper, table_capacity=1 << args.table_log2, max_rows=rows, max_nnz=max_nnz,
                          local_capacity=1 << args.local_log2, timeout_s=args.timeout_s, impl=impl,
                          track_counts=True if args.track_counts else None)

    def device_arm(impl, sampler=None):
        """W warm-up steps, then K timed steps on minibatches resident on the device; CUDA events, max over ranks."""
        eng = engine(impl)
        for i in range(args.warmup):
            eng.step(batches[i % ring])
        st0 = eng.read_stats()
        eng.check_status()
        group.barrier()
        if sampler:
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
        out = {"ms": ms, "launches": eng.kernel_launches - launches0,
               "phases": eng.phase_times_us() if impl == "fused" else None}
        st = eng.read_stats()
        eng.check_status()
        out["stats"], out["entries_before"] = st, st0["table_entries"]
        del eng
        torch.cuda.empty_cache()
        return out

    def e2e_arm(impl, host, what):
        """The public streaming API on a fresh model: every step copies its minibatch from pinned host memory and
        reads its loss back; W warm-up steps, K timed steps."""
        eng = engine(impl)
        trainer = FTRLTrainer(eng)
        warm = trainer.train(host[i % ring] for i in range(args.warmup))
        group.barrier()
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        losses = trainer.train(host[(args.warmup + i) % ring] for i in range(args.steps))
        t1.record()
        torch.cuda.synchronize(dev)
        ms = group.all_reduce_max(t0.elapsed_time(t1))
        group.barrier()
        out = {"value": rows * world * args.steps / (ms / 1e3), "unit": "examples/s", "ms_per_step": ms / args.steps,
               "h2d_bytes_per_step": trainer.h2d_bytes // args.steps, "d2h_bytes_per_step": trainer.d2h_bytes // args.steps,
               "h2d_gbs_per_gpu": trainer.h2d_bytes / args.steps / (ms / args.steps) / 1e6, "input_encoding": what,
               # progressive validation: every minibatch is scored with the model from before it was trained on
               "logloss_per_step_rank0": [round(x, 4) for x in warm + losses], "table_grown": eng.grown}
        del trainer, eng
        torch.cuda.empty_cache()
        return out

    ex_per_step = rows * world
    main_impl = "nccl" if args.impl == "nccl" else "fused"
    sampler = ClockSampler(dev)      # samples from the first timed region to the last one
    fused = device_arm(main_impl, sampler)
    nccl = None if (args.no_baseline or main_impl == "nccl") else device_arm("nccl")
    value = ex_per_step * args.steps / (fused["ms"] / 1e3)
    vs = None
    if nccl is not None:
        nccl_value = ex_per_step * args.steps / (nccl["ms"] / 1e3)
        vs = {"baseline": "NCCL-only path of the same algorithm (stand-alone kernels, all_to_all_single), same process "
                          "group, same minibatches, same warm-up and steps",
              "nccl_ms_per_step": nccl["ms"] / args.steps, "nccl_value": nccl_value, "ratio": value / nccl_value,
              "nccl_gpu_launches": nccl["launches"]}
    # ---------------------------------------------------------------- end to end (public API)
    e2e = None
    if not args.no_e2e:
        # The stream in its compact form — 32-bit feature ids (hashed to the same uint64 keys on the device) and 32-bit
        # row offsets, half the bytes per example — is what a job with a 2^30 feature space feeds; the uint64 form of
        # the same stream is measured beside it.
        compact = [HostMinibatch(b.offsets.to(torch.int32).cpu(), f.cpu(), b.y.cpu(), None, KEY_U32_HASHED).pin()
                   for b, f in zip(batches, ids)]
        enc = "uint32 feature ids hashed on the device, int32 row offsets"
        e2e = e2e_arm(main_impl, compact, enc)
        if nccl is not None:
            base = e2e_arm("nccl", compact, enc)
            vs["nccl_e2e_value"], vs["e2e_ratio"] = base["value"], e2e["value"] / base["value"]
            # time to a stated progressive logloss: both arms run the same arithmetic, so the step count is the same
            target = args.logloss_target
            trace = e2e["logloss_per_step_rank0"]
            hit = next((i + 1 for i, x in enumerate(trace) if i > 0 and x <= target), None)
            vs["time_to_logloss"] = {"target": target, "steps": hit,
                                     "fused_ms": None if hit is None else hit * e2e["ms_per_step"],
                                     "nccl_ms": None if hit is None else hit * base["ms_per_step"]}
        # what the host link gives when every rank only copies (no kernel running): the roofline of the end-to-end arms
        stage = [torch.empty_like(t, device=dev) for t in (compact[0].offsets, compact[0].keys, compact[0].y)]
        group.barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        nbytes = 0
        for i in range(args.steps):
            hb = compact[(args.warmup + i) % ring]
            for dst, src in zip(stage, (hb.offsets, hb.keys, hb.y)):
                n = min(src.numel(), dst.numel())
                dst[:n].copy_(src[:n], non_blocking=True)
                nbytes += n * src.element_size()
        c1.record()
        torch.cuda.synchronize(dev)
        copy_ms = group.all_reduce_max(c0.elapsed_time(c1))
        e2e["h2d_roofline_gbs_per_gpu"] = nbytes / copy_ms / 1e6
        e2e["fraction_of_h2d_roofline"] = e2e["h2d_gbs_per_gpu"] / e2e["h2d_roofline_gbs_per_gpu"]
        del stage, compact
        host = [HostMinibatch(b.offsets.cpu(), b.keys.cpu(), b.y.cpu()).pin() for b in batches]
        e2e["uint64_inputs"] = e2e_arm(main_impl, host, "uint64 keys, int64 row offsets")
        e2e["uint64_inputs"]["fraction_of_h2d_roofline"] = e2e["uint64_inputs"]["h2d_gbs_per_gpu"] / e2e["h2d_roofline_gbs_per_gpu"]
        del host
    clocks = sampler.stop()
    cpu = None
    if rank == 0 and not args.no_cpu:
        try:
            cpu = _cpu_ftrl_arm(20000, 3)
        except Exception as e:      # the CPU arm never fails the GPU benchmark
            cpu = {"unavailable": repr(e)}
    group.barrier()
    st = fused["stats"]
    return {
        "metric": "examples/sec (online FTRL-proximal L1-LR, CTR-scale stream)",
        "value": value,
        "unit": "examples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": fused["ms"] / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": vs,
        "dtype": "fp32", "data": "synthetic",
        "impl": "nccl-baseline" if main_impl == "nccl" else "fused",
        "config": {"model": "FTRL-proximal logistic regression, 2^30 hashed uint64 keys Zipf(1.1), ~96 nnz/row, "
                            "alpha=0.1 beta=1 lambda1=1 lambda2=0.1, per-key fp32 state, rule=" + args.rule,
                   "global_batch": ex_per_step, "seq_len": None, "nnz_per_row": max_nnz / rows,
                   "parallelism": f"dp{world} x key-range shards {world} (worker+server per GPU)",
                   "l2_policy": f"inputs larger than L2: every step reads a minibatch of its own "
                                f"({batches[0].nbytes() >> 20} MiB, {ring} distinct ones per GPU) and writes a "
                                f"{max_nnz * 4 >> 20} MiB slot map",
                   "mean_logloss_last": st["loss_sum"] / max(st["rows"], 1), "nnz_w": st["nnz_w"],
                   "unique_keys_per_step": st["unique_keys"] / max(args.steps, 1),
                   "new_keys_per_step": (st["table_entries"] - fused["entries_before"]) / max(args.steps, 1),
                   "table_entries": st["table_entries"],
                   "phase_us_last_step_rank0": fused["phases"]},
        "e2e": e2e,
        "cpu": cpu,
        "gpu_launches": fused["launches"],
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
    import dataclasses

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

    def arm(which, tau, ooc=False):
        """Device-timed bare passes, then the same passes again through run_pass (KKT filter threshold updated and
        objective read back after every pass): ms per pass and the objective after every pass."""
        sol = DarlinSolver(group, dataclasses.replace(cfg, max_block_delay=tau), timeout_s=args.timeout_s, impl=which,
                           out_of_core=ooc, prefetch_depth=args.prefetch_depth, ctas_per_sm=args.darlin_ctas)
        sol.preprocess(off, idx, vals, y)
        out = {"nblk": sol.nblk}
        if not ooc:
            sol.phase_times_ms()
            out["ms"], out["launches"], _, _ = timed(sol, False)
            if which == "fused":     # in-kernel timers of thread block 0 over warm-up + timed passes, scaled to one pass
                out["phases"] = {k: round(v / (args.warmup + args.steps), 4) for k, v in sol.phase_times_ms().items()}
            out["final"] = sol.evaluate()
        out["ms_eval"], l2, out["h2d"], out["objs"] = timed(sol, True)
        out.setdefault("launches", l2)
        del sol
        torch.cuda.empty_cache()
        return out

    def first_reaching(objs, target):
        return next((i + 1 for i, o in enumerate(objs) if o <= target), None)

    nnz_total = int(group.all_reduce_sum([idx.numel()])[0])
    sampler = ClockSampler(dev)
    sampler.start()
    main = arm(impl, args.block_delay)
    nblk, ms, launches = main["nblk"], main["ms"], main["launches"]
    objv, nnz_w, nnz_as, _ = main["final"]
    value = rows_total * args.steps / (ms / 1e3)
    vs, variants = None, {}
    if impl == "fused" and not args.no_baseline:
        base = arm("nccl", args.block_delay)
        # time to objective: passes (and device time of that many bare passes) until the objective is within 1 % of
        # the best value this arm reaches during the timed passes
        target = 1.01 * min(main["objs"])
        pf, pn = first_reaching(main["objs"], target), first_reaching(base["objs"], target)
        vs = {"baseline": "NCCL-only path of the same algorithm (stand-alone kernels per block, all_reduce of the block's "
                          "(G,U) and weights), same process group, same data, same block orders",
              "nccl_ms_per_step": base["ms"] / args.steps, "nccl_value": rows_total * args.steps / (base["ms"] / 1e3),
              "ratio": base["ms"] / ms, "nccl_gpu_launches": base["launches"],
              "nccl_objective_trace": [round(o, 2) for o in base["objs"]],
              "time_to_objective": {"target": target, "fused_passes": pf, "nccl_passes": pn,
                                    "fused_ms": None if pf is None else pf * ms / args.steps,
                                    "nccl_ms": None if pn is None else pn * base["ms"] / args.steps}}
        if args.also_delay is not None and args.also_delay != args.block_delay:
            v = arm("fused", args.also_delay)
            pv = first_reaching(v["objs"], target)
            variants[f"tau{args.also_delay}"] = {
                "ms_per_step": v["ms"] / args.steps, "value": rows_total * args.steps / (v["ms"] / 1e3),
                "objective_trace": [round(o, 2) for o in v["objs"]], "passes_to_target": pv,
                "ms_to_target": None if pv is None else pv * v["ms"] / args.steps}
    e2e = None
    if not args.no_e2e and impl == "fused":
        ooc = arm("fused", args.block_delay, ooc=True)
        ms2 = ooc["ms_eval"]
        e2e = {"value": rows_total * args.steps / (ms2 / 1e3), "unit": "examples/s", "ms_per_step": ms2 / args.steps,
               "h2d_bytes_per_step": ooc["h2d"] // args.steps, "d2h_bytes_per_step": 40,
               "objective_last": ooc["objs"][-1] if ooc["objs"] else None,
               # time to objective: objective after every pass; pass i completes at (i+1) * ms_per_step
               "objective_trace": [round(o, 2) for o in ooc["objs"]]}
        if vs is not None:
            vs["nccl_e2e_value"] = rows_total * args.steps / (base["ms_eval"] / 1e3)     # resident data, objective read back
            vs["e2e_ratio"] = e2e["value"] / vs["nccl_e2e_value"]
    clocks = sampler.stop()
    group.barrier()
    return {
        "metric": "examples/sec (L1-LR, DARLIN block coordinate descent, one pass = one step)",
        "value": value, "unit": "examples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak" if ooc_shape else "strong", "vs_baseline": vs, "dtype": "fp32",
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
                   "objective_after_timed_passes": objv, "nnz_w": nnz_w, "active_keys": nnz_as,
                   "objective_trace": [round(o, 2) for o in main["objs"]],
                   "phase_ms_per_pass_rank0_block0": main.get("phases")},
        "variants": variants or None,
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
    ap.add_argument("--also-delay", type=int, default=None,
                    help="DARLIN: also run the fused arm with this bounded delay and report it under `variants`")
    ap.add_argument("--darlin-ctas", type=int, default=None, help="DARLIN: thread blocks of the pass kernel per SM (1 or 2)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "fused", "nccl", "reference"])
    ap.add_argument("--rows", type=int, default=100000, help="minibatch rows per GPU")
    ap.add_argument("--ring", type=int, default=0, help="distinct minibatches per GPU (at least warm-up + steps; negative: replay exactly that many)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL-only arm (vs_baseline stays null)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU arm")
    ap.add_argument("--logloss-target", type=float, default=0.2,
                    help="progressive mean logloss whose first crossing is reported as time to objective")
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
