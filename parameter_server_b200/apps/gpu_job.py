"""Run a ``.conf`` job on the GPU engines: one rank per B200 (worker + server), launched by
``torch.distributed.run`` or as a single process.

Solver selection follows LinearMethod::create (src/linear_method/linear_method.cc:20-39): no
``solver`` but ``validation_data`` + ``model_input`` → model evaluation; ``solver.minibatch_size <= 0``
→ batch solver (DARLIN when ``darling{}`` is present, otherwise block proximal gradient);
otherwise ``ftrl{}`` → online FTRL.  Files are assigned round-robin to the ranks
(src/data/common.cc:148-166), text is parsed by the native slot/stream readers, and every rank writes
its shard of the model as ``<model_output.file>_S<rank>``.
"""
from __future__ import annotations

import sys
import time
from typing import List, Optional

import numpy as np
import torch

from .. import config as cfg
from ..parallel.peer import PeerGroup
from ..runtime import host


def _my_files(data_conf, group: PeerGroup, load_limit: int) -> List[str]:
    H = host()
    patterns = cfg.data_files(data_conf, H)
    files = H.search_files(patterns)
    if patterns and not files:
        raise FileNotFoundError(f"no file matches {list(patterns)}")
    return H.divide_files(files, group.world, load_limit)[group.rank]


def load_csr(data_conf, files: List[str], flags: cfg.Flags, cache_dir: str, device):
    """(offsets int64, keys int64 bit patterns, vals float32|None, y float32) of this rank's files (all slots merged)."""
    H = host()
    fmt = getattr(H.TextFormat, data_conf.text if data_conf.has("text") else "LIBSVM")
    r = H.SlotReader()
    r.init(files, fmt, cache_dir, True, bool(flags.shuffle_fea_id), bool(flags.add_beta_feature), int(flags.line_limit),
           int(flags.load_data_max_mb_per_thread))
    info, _ = r.read(max(int(flags.num_threads), 1))
    y = torch.from_numpy(r.value(0).astype(np.float32))
    y = torch.where(y > 0, 1.0, -1.0)
    off = torch.from_numpy(r.offset(1).astype(np.int64))
    keys = torch.from_numpy(r.index(1).view(np.int64))
    v = r.value(1)
    vals = None if len(v) == 0 else torch.from_numpy(v)
    to = lambda t: None if t is None else t.to(device)
    return to(off), to(keys), to(vals), to(y), info


def _gather_model(group: PeerGroup, keys: np.ndarray, w: np.ndarray):
    if group.world == 1:
        return keys, w
    import torch.distributed as dist

    parts = [None] * group.world
    dist.all_gather_object(parts, (keys, w), group=group.group)
    k = np.concatenate([p[0] for p in parts])
    v = np.concatenate([p[1] for p in parts])
    order = np.argsort(k, kind="stable")
    return k[order], v[order]


def predict_csr(off, keys, vals, mk: np.ndarray, mw: np.ndarray) -> torch.Tensor:
    """X·w for CSR rows against a sorted (key, weight) model."""
    dev = off.device
    sign = -(1 << 63)
    mks = torch.from_numpy(mk.view(np.int64).copy()).to(dev) ^ sign
    mwt = torch.from_numpy(mw.astype(np.float32)).to(dev)
    ks = keys ^ sign
    if mks.numel() == 0:
        return torch.zeros(off.numel() - 1, device=dev)
    pos = torch.searchsorted(mks, ks).clamp_(max=mks.numel() - 1)
    hit = mks[pos] == ks
    wv = torch.where(hit, mwt[pos], torch.zeros((), device=dev))
    if vals is not None:
        wv = wv * vals
    rows = off.numel() - 1
    row_of = torch.repeat_interleave(torch.arange(rows, device=dev), off[1:] - off[:-1])
    return torch.zeros(rows, device=dev).index_add_(0, row_of, wv)


def validation_auc(group: PeerGroup, conf_data, flags, cache: str, mk, mw, goodness: int) -> Optional[float]:
    """AUC over the validation files, histograms merged across ranks (src/base/auc.h, batch_solver.cc:114-123)."""
    H = host()
    files = _my_files(conf_data, group, 0)
    auc = H.AUC()
    auc.set_goodness(int(goodness))
    if files:
        off, keys, vals, y, _ = load_csr(conf_data, files, flags, cache + "valid/", group.device)
        xw = predict_csr(off, keys, vals, mk, mw)
        from ..ops.evalops import auc_histogram

        auc.merge_data(*auc_histogram(y, xw, int(goodness)))     # binned on the device: only the occupied bins come back
    if group.world > 1:
        import torch.distributed as dist

        parts = [None] * group.world
        dist.all_gather_object(parts, auc.data(), group=group.group)
        auc = H.AUC()
        auc.set_goodness(int(goodness))
        for p in parts:
            auc.merge_data(*p)
    return auc.evaluate()


def run_gpu_job(flags: cfg.Flags) -> dict:
    group = PeerGroup.from_env()
    conf = cfg.load_app_config(flags.app)
    if conf.has("neural_network"):
        from ..models.nn import run_nn_job

        return run_nn_job(conf, flags, group)
    lm = conf.linear_method
    cache = (lm.local_cache.file[0] if lm.local_cache.file else "/tmp/psb200_cache/") + f"rank{group.rank}/"
    out: dict = {}
    if not lm.has("solver") and lm.has("validation_data") and lm.has("model_input"):
        from .model_evaluation import evaluate_model

        return evaluate_model(lm, flags, group)
    if lm.solver.minibatch_size <= 0:
        from ..models.darlin import DarlinConfig, DarlinSolver

        files = _my_files(lm.training_data, group, int(flags.load_limit))
        off, keys, vals, y, info = load_csr(lm.training_data, files, flags, cache, group.device)
        d, s = lm.darling, lm.solver
        lam = lm.penalty.get("lambda")
        dc = DarlinConfig(lambda1=lam[0] if lam else 0.0, eta=lm.learning_rate.eta, delta_init=d.delta_init_value,
                          delta_max=d.delta_max_value, kkt_ratio=d.kkt_filter_threshold_ratio, max_pass=s.max_pass_of_data,
                          epsilon=s.epsilon, feature_block_ratio=s.feature_block_ratio,
                          random_block_order=s.random_feature_block_order, max_block_delay=s.max_block_delay,
                          seed=int(flags.seed), tail_feature_freq=int(s.tail_feature_freq),
                          countmin_k=int(s.countmin_k), countmin_n_ratio=float(s.countmin_n_ratio),
                          # TERAFEA keys carry their feature group in their top 10 bits: blocks are cut group by group
                          feature_group_bits=10 if (lm.training_data.has("text") and lm.training_data.text == "TERAFEA") else 0,
                          prior_fea_group=tuple(int(g) for g in s.prior_fea_group),
                          num_iter_for_prior_fea_group=int(s.num_iter_for_prior_fea_group))
        if lm.has("darling"):
            impl = flags.impl if flags.impl in ("fused", "nccl") else "fused"
            # -mmap_training_data: the column blocks stay in pinned host memory and are streamed per pass
            # (FeatureStation's out-of-core mode, src/linear_method/feature_station.cc:70-109); every rank streams
            # the blocks of its own rows
            ooc = bool(flags.mmap_training_data) and impl == "fused" and lm.init_w.type != "FILE"
            sol = DarlinSolver(group, dc, timeout_s=float(flags.timeout_s), impl=impl, out_of_core=ooc)
            from ..utils.trace import ChromeTrace, MetricsLog

            if flags.trace_file:
                sol.trace = ChromeTrace(f"{flags.trace_file}.rank{group.rank}.json", pid=group.rank)
            if flags.metrics_file:
                sol.metrics = MetricsLog(flags.metrics_file)
            if group.world > 1 and float(flags.report_interval) > 0:
                from ..parallel.monitor import RankMonitor

                sol.monitor = RankMonitor(group.rank, group.world, deadline_s=max(10.0, 5.0 * float(flags.report_interval)))
            sol.preprocess(off, keys, vals, y)
            if lm.init_w.type == "FILE":      # warm start from a model dump (one file, or the parts <name>_S<i>)
                from ..utils.modelio import model_arrays, model_files, read_model_text

                paths = model_files(lm.init_w.file_name)
                if not paths:
                    raise FileNotFoundError(f"init_w: no model file at {lm.init_w.file_name}")
                sol.warm_start(*model_arrays(read_model_text(*paths)))
            t0 = time.time()
            if flags.checkpoint_dir:
                from ..utils.checkpoint import run_with_checkpoints

                prog = run_with_checkpoints(sol, flags.checkpoint_dir, int(flags.checkpoint_interval) or 1, verbose=bool(flags.verbose) or True)
            elif flags.gpu_scheduler:
                # the passes run under a scheduler node of the host control plane (apps/gpu_control.py)
                from .gpu_control import run_scheduled

                ctl = run_scheduled(group, flags, conf.app_name or "linear_method", sol,
                                    lm.model_output.file[0] if lm.model_output.file else "", verbose=True)
                prog = sol.progress
                if ctl.get("model"):
                    out["model"] = ctl["model"]               # written by the SAVE_MODEL task
                out["scheduler_progress"] = ctl.get("scheduler")
                if "dashboard" in ctl:
                    out["dashboard"] = ctl["dashboard"]
            else:
                prog = sol.run(verbose=True)
        else:
            from ..models.batch import ProxGradientSolver

            sol = ProxGradientSolver(group, dc, loss=lm.loss.type, penalty=lm.penalty.type,
                                     learner=lm.learner.type if lm.has("learner") else "PROXIMAL_GRADIENT")
            sol.preprocess(off, keys, vals, y)
            t0 = time.time()
            prog = sol.run(verbose=True)
        out["seconds"] = time.time() - t0
        out["progress"] = [p.__dict__ for p in prog]
        if getattr(sol, "trace", None) is not None:
            out["trace"] = sol.trace.save()
        if lm.model_output.file and "model" not in out:
            out["model"] = sol.save_model(lm.model_output.file[0])
        if lm.has("validation_data"):
            mk, mw = _gather_model(group, *sol.model())
            out["validation_auc"] = validation_auc(group, lm.validation_data, flags, cache, mk, mw, s.auc_goodness)
            if group.rank == 0:
                print(f"validation AUC: {out['validation_auc']:.6f}", file=sys.stderr)
        return out
    if not lm.has("ftrl"):
        raise ValueError("online solver requested (solver.minibatch_size > 0) but no ftrl{} section")
    return run_ftrl_job(lm, flags, group, cache)


def run_ftrl_job(lm, flags: cfg.Flags, group: PeerGroup, cache: str) -> dict:
    """FTRL::run + FTRL::updateModel (src/linear_method/ftrl.cc:38-152): stream minibatches, print progress."""
    from ..models.ftrl import FTRLEngine, FTRLHyper
    from ..models.ftrl_trainer import FTRLTrainer, HostMinibatch

    H = host()
    s = lm.solver
    lam = list(lm.penalty.get("lambda")) + [0.0, 0.0]
    hyper = FTRLHyper(alpha=lm.learning_rate.alpha, beta=lm.learning_rate.beta, lambda1=lam[0], lambda2=lam[1],
                      tail_feature_freq=int(s.tail_feature_freq), countmin_n=int(s.countmin_n),
                      countmin_k=int(s.countmin_k))
    files = _my_files(lm.training_data, group, int(flags.load_limit))
    fmt = getattr(H.TextFormat, lm.training_data.text if lm.training_data.has("text") else "LIBSVM")
    reader = H.StreamReader()
    reader.init(files, fmt, True, bool(flags.shuffle_fea_id))
    mb = int(s.minibatch_size)
    max_nnz = mb * 256
    eng = FTRLEngine(group, hyper, table_capacity=max(int(s.countmin_n) // max(group.world, 1), 1 << 16), max_rows=mb,
                     max_nnz=max_nnz, local_capacity=min(max_nnz, 1 << 24), timeout_s=float(flags.timeout_s),
                     impl="nccl" if flags.impl == "nccl" else "fused")
    trainer = FTRLTrainer(eng)

    def batches():
        # every rank must run the same number of steps: ranks that run out of data feed empty minibatches.
        # The ranks agree on "anybody still has data" over a host-side (gloo) group, so that the question never
        # waits for, or holds up, the kernels of the step in flight.
        import torch.distributed as dist

        ctl = dist.new_group(backend="gloo") if group.world > 1 else None
        while True:
            out = reader.read(mb)
            have = torch.tensor([0 if out is None else 1])
            if ctl is not None:
                dist.all_reduce(have, group=ctl)
            if have.item() == 0:
                return
            if out is None:
                yield HostMinibatch(torch.zeros(1, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), torch.zeros(0)).pin()
                continue
            slots, info = out
            sl = slots.get(1, {"offset": np.zeros(info["num_ex"] + 1, np.uint64), "index": np.zeros(0, np.uint64), "value": np.zeros(0, np.float32)})
            y = torch.from_numpy(np.where(slots[0]["value"] > 0, 1.0, -1.0).astype(np.float32))
            v = torch.from_numpy(sl["value"]) if len(sl["value"]) else None
            yield HostMinibatch(torch.from_numpy(sl["offset"].astype(np.int64)), torch.from_numpy(sl["index"].view(np.int64)), y, v).pin()

    t0 = time.time()
    seen = 0
    last = time.time()
    # checkpoint / resume: the shard tables are saved every checkpoint_interval minibatches; a restarted job
    # reloads the newest step all ranks have and skips the minibatches that were applied before it
    ckdir, ckint = flags.checkpoint_dir, int(flags.checkpoint_interval)
    start_step, step = 0, 0
    if ckdir:
        from ..utils.checkpoint import load_ftrl, save_ftrl

        start_step = max(load_ftrl(eng, ckdir), 0)
        if start_step and group.rank == 0:
            print(f"resuming after minibatch {start_step} from {ckdir}", file=sys.stderr)
    # -report_interval > 0 (the reference's heartbeat switch): every rank heartbeats into the job's store and
    # looks at the others before launching; a rank that left or went silent stops the job with RankLost
    mon = None
    if group.world > 1 and float(flags.report_interval) > 0:
        from ..parallel.monitor import RankMonitor

        mon = RankMonitor(group.rank, group.world, deadline_s=max(10.0, 5.0 * float(flags.report_interval)))

    rows_of: list = []

    def stream():
        # minibatches that a checkpoint already covers are read and skipped; the rest go to the trainer, which
        # uploads minibatch i+1 while step i computes
        nonlocal step, seen
        for hb in batches():
            step += 1
            if mon is not None:
                mon.tick(step, float(flags.report_interval))
            seen += hb.y.numel()
            if step > start_step:
                rows_of.append(int(hb.y.numel()))       # rows of the trainer's step len(rows_of) - 1
                yield hb

    def after_step(i):
        at = start_step + i + 1
        if ckdir and ckint > 0 and at % ckint == 0:
            torch.cuda.synchronize(group.device)        # the model as of minibatch `at`
            save_ftrl(eng, ckdir, at)

    def on_loss(i, loss):
        nonlocal last
        if group.rank == 0 and time.time() - last >= s.eval_interval:
            st = eng.read_stats(reset=False)
            print("%10d examples, loss %.5e, penalty %.5e, |w|_0 %8d" % (seen * group.world, loss, eng.penalty(st), int(st["nnz_w"])))
            last = time.time()

    ctl = None
    if flags.gpu_scheduler:
        # the stream runs as the one UPDATE_MODEL task of a scheduler node (apps/gpu_control.py); every rank reports
        # its loss and examples, and the penalty and non-zeros of its shard, every eval_interval
        from .gpu_control import run_scheduled_online

        total = {"loss": 0.0}                                    # sum of the steps' loss sums (the trainer gives means)

        def run_training(report):
            mark = {"t": time.time(), "seen": 0, "loss": 0.0}

            def on_loss_report(i, loss):
                n = rows_of[i]                                    # the step's mean loss times its rows = its loss sum
                mark["loss"] += loss * n
                mark["seen"] += n
                total["loss"] += loss * n
                if time.time() - mark["t"] >= s.eval_interval:
                    st_ = eng.read_stats(reset=False)
                    report(mark["loss"], mark["seen"], eng.penalty(st_), int(st_["nnz_w"]))
                    mark.update(t=time.time(), seen=0, loss=0.0)

            return trainer.train(stream(), after_step=after_step, on_loss=on_loss_report)

        def final_progress():
            st_ = eng.read_stats(reset=False)
            return total["loss"] + eng.penalty(st_), int(st_["nnz_w"]), seen

        ctl = run_scheduled_online(group, flags, cfg.load_app_config(flags.app), run_training, final_progress,
                                   lambda: eng.save_model(lm.model_output.file[0]) if lm.model_output.file else None)
        losses = ctl["result"] or []
    else:
        losses = trainer.train(stream(), after_step=after_step, on_loss=on_loss)
    st = eng.read_stats(reset=False)
    out = {"seconds": time.time() - t0, "examples": seen, "mean_logloss_last": losses[-1] if losses else None,
           "nnz_w": st["nnz_w"], "penalty": eng.penalty(st)}
    if group.rank == 0:
        print("%10d examples, loss %.5e, penalty %.5e, |w|_0 %8d" % (seen * group.world, out["mean_logloss_last"] or 0.0,
                                                                   out["penalty"], int(st["nnz_w"])))
    if ctl is not None:
        out["scheduler_progress"] = ctl.get("scheduler")
        if ctl.get("model"):
            out["model"] = ctl["model"]                   # written by the SAVE_MODEL task
    if lm.model_output.file and "model" not in out:
        out["model"] = eng.save_model(lm.model_output.file[0])
    group.barrier()
    return out
