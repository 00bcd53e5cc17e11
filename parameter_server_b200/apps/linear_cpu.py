"""The linear-method application on CPU nodes, driven through the control-plane runtime.

This is the multi-process form of the job: a scheduler, S servers and W workers that talk only
through messages (push / pull on a shared parameter, task calls with logical timestamps), the way
the reference runs it.  It is used for CPU-only deployments, for the plumbing configuration
(1 scheduler + 2 servers + 2 workers on localhost) and as the protocol-level test bed; the GPU
engines in ``models/`` implement the same solvers on peer memory.

Reference roles: LinearMethod::process / startSystem / mergeProgress
(src/linear_method/linear_method.cc:62-179), BatchSolver::run / loadData / preprocessData /
saveModel (src/linear_method/batch_solver.cc:23-127, 202-426), Darling::updateModel
(src/linear_method/darling.cc:155-273), SharedParameter::process
(src/parameter/shared_parameter.h:90-149), KVVector (src/parameter/kv_vector.h).
"""
from __future__ import annotations

import math
import os
import shutil
import sys
import threading
import time
import zlib
from typing import Dict, List

import numpy as np
import scipy.sparse as sp

from .. import config as cfg
from ..runtime import host
from ..runtime.node import NodeContext
from ..utils.modelio import write_model_text
from ..utils.pbtext import dumps, parse

PUSH, PULL = 1, 2
F_INSERT_KEY_FREQ, F_INSERT_KEY = 1, 2
K_PACE = 10                       # parameter timestamps per scheduler task (batch_solver.h:15)
U64 = np.uint64
NAN_SENTINEL = np.float64(np.nan)


def _call(cmd: str, **kw) -> bytes:
    m = cfg.LMCall(cmd=cmd)
    for k, v in kw.items():
        if k == "key":
            m.key = cfg.PbRange(begin=v[0], end=v[1])
        else:
            m.set(k, v)
    return dumps(m, oneline=True).encode()


class SharedParam:
    """The shared parameter ``w``.  Push and pull are served by the native customer ``SharedParamCustomer``
    (csrc/host/shared_param.h) on its executor thread; this class is the handle the solver code talks to."""

    class _Filter:
        def __init__(self, cust):
            self._c = cust

        def clear(self) -> None:
            self._c.clear_filter()

    def __init__(self, ctx: NodeContext, name: str, solver):
        H = host()
        self.H, self.ctx, self.solver = H, ctx, solver
        # -parallel_match: the server's merge-join of a push into its key list runs on -num_threads threads
        # (src/parameter/kv_vector.h:77-137)
        fl = getattr(solver, "flags", None)
        threads = max(int(fl.num_threads), 1) if fl is not None and bool(fl.parallel_match) else 1
        s = solver.conf.solver
        self.cust = H.SharedParamCustomer(ctx.po, name, threads, max(int(ctx.num_workers), 1), int(s.countmin_k), float(s.countmin_n_ratio))
        self.kv = self.cust                      # keys / values / received / set_values... of the channel store, under its lock
        self.filter = SharedParam._Filter(self.cust)

    def take_pulled(self, t: int):
        """The replies of pull ``t`` concatenated in server (= key) order: (keys, values)."""
        return self.cust.take_pulled(t, self.cust.group(self.H.kServerGroup))


class LinearMethodNode:
    """Worker or server side of the batch DARLIN solver (one instance per non-scheduler node)."""

    def __init__(self, ctx: NodeContext, app_conf, flags: cfg.Flags):
        H = host()
        self.H, self.ctx, self.flags = H, ctx, flags
        self.app_conf = app_conf
        self.conf = app_conf.linear_method
        self.param = SharedParam(ctx, app_conf.parameter_name[0], self)
        self.cust = H.Customer(ctx.po, app_conf.app_name, self.process, False)
        self.kkt_threshold = 1e20
        self.violation = 0.0
        self.busy = 0.0
        self.ch = 1               # single feature group channel (all slots merged), like LIBSVM data
        self.station = None       # feature store on disk (-mmap_training_data)

    # ------------------------------------------------------------------ dispatch
    def process(self, msg) -> None:
        if not msg.request:
            return
        call = parse(msg.payload.decode(), cfg.LMCall)
        t0 = time.time()
        if self.ctx.hb_state is not None:
            self.ctx.hb_state["task"] = msg.time          # the task this node is at, for the scheduler's table
        reply = b""
        if call.cmd == "LOAD_DATA":
            reply = self.load_data()
        elif call.cmd == "PREPROCESS_DATA":
            self.preprocess(msg.time)
        elif call.cmd == "UPDATE_MODEL":
            self.update_model(msg, call)
            self.busy += time.time() - t0
            self.ctx.add_busy(time.time() - t0)
            return
        elif call.cmd == "EVALUATE_PROGRESS":
            reply = self.evaluate()
        elif call.cmd == "SAVE_MODEL":
            self.save_model()
        elif call.cmd == "COMPUTE_VALIDATION_AUC":
            reply = self.validation_auc(msg.time)
        elif call.cmd == "RECOVER":
            pass                      # "FIXME" in the reference (linear_method.cc:90-93); recovery here = restart from a dump
        self.busy += time.time() - t0
        self.ctx.add_busy(time.time() - t0)
        self.cust.reply(msg, payload=reply)

    # ------------------------------------------------------------------ LOAD_DATA
    def load_data(self) -> bytes:
        if not self.ctx.is_worker:
            return b""
        td = self.conf.training_data
        fmt = getattr(self.H.TextFormat, td.text if td.has("text") else "LIBSVM")
        cache = self.conf.local_cache.file[0] if self.conf.local_cache.file else "/tmp/psb200_cache/"
        r = self.H.SlotReader()
        r.init(cfg.data_files(td, self.H), fmt, cache + f"{self.ctx.node_id}/", True, bool(self.flags.shuffle_fea_id),
               bool(self.flags.add_beta_feature), int(self.flags.line_limit), int(self.flags.load_data_max_mb_per_thread))
        info, hits = r.read(max(int(self.flags.num_threads), 1))
        self.y = r.value(0).astype(np.float64)
        self.off, self.idx = r.offset(1).astype(np.int64), r.index(1)
        v = r.value(1)
        self.binary = len(v) == 0
        self.val = np.ones(len(self.idx)) if self.binary else v.astype(np.float64)
        if td.has("text") and td.text == "TERAFEA":
            return self._group_info(info).encode()
        return info["text"].encode()

    def _group_info(self, info: dict) -> str:
        """TERAFEA keys carry their feature group in their top 10 bits.  The keys of all groups stay in one key space
        (the groups' key ranges cannot overlap), but the scheduler cuts every group into blocks of its own, so it gets
        one slot per group: id, key range, non-zeros, examples in which the group occurs (src/proto/example.proto)."""
        gid = (self.idx >> U64(54)).astype(np.int64)
        row_of = np.repeat(np.arange(len(self.off) - 1, dtype=np.int64), np.diff(self.off))
        out = cfg.ExampleInfo(num_ex=int(info["num_ex"]))
        slots = [cfg.SlotInfo(format="DENSE", id=0, min_key=0, max_key=1, nnz_ele=len(self.y), nnz_ex=len(self.y))]
        for g in np.unique(gid).tolist():
            m = gid == g
            k = self.idx[m]
            slots.append(cfg.SlotInfo(format="SPARSE_BINARY" if self.binary else "SPARSE", id=int(g), min_key=int(k.min()),
                                      max_key=int(k.max()) + 1, nnz_ele=int(m.sum()), nnz_ex=int(len(np.unique(row_of[m])))))
        out.slot = slots
        return dumps(out)

    # ------------------------------------------------------------------ PREPROCESS_DATA
    def preprocess(self, T: int) -> None:
        H, P, t = self.H, self.param, T * K_PACE
        solver = self.conf.solver
        allr = (0, 2**64 - 1)
        freq = solver.tail_feature_freq
        if self.ctx.is_worker:
            # localisation in the native runtime (csrc/host/localizer.h): unique keys with counts, local column ids,
            # column-major storage
            T_ = max(int(self.flags.num_threads), 1)
            ukeys, cnt, loc = H.localize(self.idx)
            if freq > 0:      # tail-feature filter through the servers' count-min sketch
                P.cust.submit(H.kServerGroup, cmd=PUSH, key=ukeys.tobytes(), values=[cnt.astype(np.uint32).tobytes()],
                              time=t, key_range=allr, channel=self.ch, flags=F_INSERT_KEY_FREQ, wait=True)
                P.cust.submit(H.kServerGroup, cmd=PULL, key=ukeys.tobytes(), time=t + 2, wait_time=t + 1, key_range=allr,
                              channel=self.ch, aux=freq, erase_key_cache=True, wait=True)
                ukeys, _ = P.take_pulled(t + 2)           # the surviving keys, ascending (servers answer in key order)
                loc = H.remap_keys(self.idx, ukeys, T_)   # ids among the survivors, -1: dropped by the filter
            self.keys = ukeys
            indptr, rix, cval = H.csr_to_csc(self.off, loc, None if self.binary else self.val, len(ukeys), T_)
            self._csc_cache = (indptr, rix, cval, np.ascontiguousarray(self.y, dtype=np.float64))
            self.idx = self.val = self.off = None
            t2 = t + 4
            P.cust.submit(H.kServerGroup, cmd=PUSH, key=ukeys.tobytes(), time=t2, key_range=allr, channel=self.ch,
                          flags=F_INSERT_KEY, erase_key_cache=True, wait=True)
            P.cust.submit(H.kServerGroup, cmd=PULL, key=ukeys.tobytes(), time=t2 + 2, wait_time=t2 + 1, key_range=allr,
                          channel=self.ch, erase_key_cache=True, wait=True)
            _, w0 = P.take_pulled(t2 + 2)
            n = len(ukeys)
            self.w = w0.copy() if len(w0) == n else np.zeros(n)
            xw = np.zeros(len(self.y))
            if np.any(self.w != 0):
                wcol = np.repeat(self.w, np.diff(indptr))
                xw = np.bincount(rix, weights=wcol if cval is None else wcol * cval, minlength=len(self.y))
            self.dual = np.exp(self.y * xw)
            self.delta = np.full(n, self.conf.darling.delta_init_value)
            self.active = np.ones(n, dtype=np.uint8)
            if bool(self.flags.mmap_training_data):
                self._to_station()
        else:
            if freq > 0:
                P.cust.wait_in(H.kWorkerGroup, t)
                P.cust.finish_in(H.kWorkerGroup, t + 1)
            t2 = t + 4
            P.cust.wait_in(H.kWorkerGroup, t2)
            P.filter.clear()
            init = self.conf.init_w
            P.kv.init_values(self.ch, init.constant if init.type == "CONSTANT" else 0.0)
            if init.type == "GAUSSIAN":
                rng = np.random.default_rng(int(self.flags.seed) + zlib.crc32(self.ctx.node_id.encode()))
                P.kv.set_values(self.ch, rng.normal(init.mean, init.std, len(P.kv.keys(self.ch))))
            elif init.type == "FILE":
                self._init_from_model(init.file_name)
            n = len(P.kv.keys(self.ch))
            self.delta = np.full(n, self.conf.darling.delta_init_value)
            self.active = np.ones(n, dtype=np.uint8)
            P.cust.finish_in(H.kWorkerGroup, t2 + 1)

    def _init_from_model(self, name: str) -> None:
        """``init_w { type: FILE file_name: ... }``: start from a model dump (``key<TAB>value`` lines).  ``name`` is one
        file, or the ``model_output`` prefix of an earlier job, whose per-server parts ``<name>_S<i>`` are all read: the
        key ranges of the two jobs need not agree.  Keys of the dump that this job's data lacks are ignored.  (The
        reference declares the FILE type and aborts on it: src/base/shared_array_inl.h:115-123.)"""
        from ..utils.modelio import lookup_model, model_arrays, model_files, read_model_text

        paths = model_files(name)
        if not paths:
            raise FileNotFoundError(f"init_w: no model file at {name} or {name}_*")
        mk, mv = model_arrays(read_model_text(*paths))
        w = lookup_model(mk, mv, self.param.kv.keys(self.ch))
        self.param.kv.set_values(self.ch, w)

    # ------------------------------------------------------------------ UPDATE_MODEL
    def update_model(self, msg, call) -> None:
        H, P = self.H, self.param
        t = msg.time * K_PACE
        if call.has("kkt_filter_threshold"):
            self.kkt_threshold = call.kkt_filter_threshold
            self.violation = 0.0
        if call.has("kkt_filter_reset") and call.kkt_filter_reset:
            self.active[:] = 1
            if self.ctx.is_server:
                w = P.kv.values(self.ch)
                P.kv.set_values(self.ch, np.nan_to_num(w, nan=0.0))
        rng = (call.key.begin, call.key.end)
        if self.ctx.is_worker:
            c0, c1 = np.searchsorted(self.keys, [U64(rng[0]), U64(rng[1])])
            if self.station is not None:
                self._prefetch_ahead(msg.time)
            G, Uu = self._gradients(c0, c1, msg.time)
            gu = np.stack([G, Uu], 1).ravel()
            P.cust.submit(H.kServerGroup, cmd=PUSH, key=self.keys[c0:c1].tobytes(), values=[gu.tobytes()], time=t,
                          key_range=rng, channel=self.ch)
            msg.defer()
            sender, T = msg.sender, msg.time

            def on_pull():
                _, wn = P.take_pulled(t + 2)
                self._update_dual(c0, c1, wn, T)
                if self.station is not None:
                    self.station.drop(T)
                self.cust.finish_in(sender, T)
                self.cust.reply(msg)

            P.cust.submit(H.kServerGroup, cmd=PULL, key=self.keys[c0:c1].tobytes(), time=t + 2, wait_time=t + 1,
                          key_range=rng, channel=self.ch, on_finish=on_pull)
        else:
            lo, hi = self.ctx.po.my_node.key
            if max(lo, rng[0]) < min(hi, rng[1]):
                P.cust.wait_in(H.kWorkerGroup, t)
                s0, s1, nval, vals = P.kv.received(t)
                if nval and s1 > s0:
                    self._update_weight(s0, s1, vals.reshape(-1, nval))
                P.cust.finish_in(H.kWorkerGroup, t + 1)
            self.cust.reply(msg)

    # The three block steps run in the native runtime (csrc/host/darlin_cpu.h): threaded column gradients, the
    # server's proximal-Newton update, the worker's dual update.
    def _csc(self):
        return self._csc_cache            # (offsets per column, row ids, values or None, labels), built in preprocess

    def _to_station(self) -> None:
        """-mmap_training_data: the column-major features go to the local cache directory and leave memory;
        column ranges come back through the station's prefetch threads (csrc/host/feature_station.h)."""
        indptr, indices, data, y = self._csc()
        base = self.conf.local_cache.file[0] if self.conf.local_cache.file else "/tmp/psb200_cache/"
        self._station_dir = f"{base}{self.ctx.node_id}_features_{os.getpid()}"
        self.station = self.H.FeatureStation(self._station_dir, self.ctx.node_id,
                                             int(self.flags.prefetch_mem_limit_kb), max(int(self.flags.num_threads), 1),
                                             int(self.flags.prefetch_job_limit), bool(self.flags.prefetch_detail))
        self.station.add_group(self.ch, len(y), indptr, indices, data)
        self._y = y
        self._csc_cache = None

    def _prefetch_ahead(self, now: int) -> None:
        """Queue reads for the UPDATE_MODEL tasks that have arrived but not started, up to 4 (τ + 1) tasks ahead of
        the newest one seen (the reference's window: src/linear_method/darling.cc:175-200)."""
        st, tau = self.station, int(self.conf.solver.max_block_delay)
        if st.pending() >= tau + 8:
            return
        horizon = max(st.max_task(), now) + 4 * max(tau, 1)
        for m in self.cust.pending_requests():
            if m.time > horizon or st.task_used(m.time):
                continue
            try:
                call = parse(m.payload.decode(), cfg.LMCall)
            except Exception:
                continue
            if call.cmd != "UPDATE_MODEL":
                continue
            c0, c1 = np.searchsorted(self.keys, [U64(call.key.begin), U64(call.key.end)])
            st.prefetch(m.time, self.ch, int(c0), int(c1))

    def _gradients(self, c0: int, c1: int, task: int = 0):
        if self.station is not None:
            return self.station.block_gradient(task, self.ch, int(c0), int(c1), self._y, self.dual, self.delta, self.active,
                                               max(int(self.flags.num_threads), 1))
        indptr, indices, data, y = self._csc()
        return self.H.darlin_block_gradient(indptr, indices, data, y, self.dual, self.delta, self.active, c0, c1,
                                            max(int(self.flags.num_threads), 1))

    def _update_weight(self, s0: int, s1: int, GU: np.ndarray) -> None:
        P, d = self.param, self.conf.darling
        w = P.kv.values(self.ch)
        seg = np.ascontiguousarray(w[s0:s1], dtype=np.float64).copy()
        dl = np.ascontiguousarray(self.delta[s0:s1]).copy()
        ac = np.ascontiguousarray(self.active[s0:s1]).copy()
        vio = self.H.darlin_update_weight(seg, dl, ac, np.ascontiguousarray(GU[:, 0]), np.ascontiguousarray(GU[:, 1]),
                                          float(self.conf.penalty.get("lambda")[0]), float(self.conf.learning_rate.eta),
                                          float(self.kkt_threshold), float(d.delta_max_value))
        self.delta[s0:s1] = dl
        self.active[s0:s1] = ac
        self.violation = max(self.violation, vio)
        P.kv.set_values_range(self.ch, s0, seg)

    def _update_dual(self, c0: int, c1: int, w_new: np.ndarray, task: int = 0) -> None:
        if self.station is not None:
            self.station.block_update_dual(task, self.ch, int(c0), int(c1), self._y, self.dual, self.w, self.delta, self.active,
                                           np.ascontiguousarray(w_new, dtype=np.float64), float(self.conf.darling.delta_max_value))
            return
        indptr, indices, data, y = self._csc()
        self.H.darlin_update_dual(indptr, indices, data, y, self.dual, self.w, self.delta, self.active,
                                  np.ascontiguousarray(w_new, dtype=np.float64), c0, c1, float(self.conf.darling.delta_max_value))

    # ------------------------------------------------------------------ EVALUATE_PROGRESS / SAVE_MODEL
    def evaluate(self) -> bytes:
        p = cfg.Progress()
        if self.ctx.is_worker:
            p.objv = float(np.sum(np.log1p(1.0 / self.dual)))
            p.busy_time = [self.busy]
            self.busy = 0.0
        else:
            w = np.nan_to_num(self.param.kv.values(self.ch), nan=0.0)
            p.objv = float(np.abs(w).sum() * self.conf.penalty.get("lambda")[0])
            p.nnz_w = int((w != 0).sum())
            p.violation = float(self.violation)
            p.nnz_active_set = int(self.active.sum())
        return dumps(p, oneline=True).encode()

    def validation_auc(self, T: int) -> bytes:
        """COMPUTE_VALIDATION_AUC on a worker: read its validation files, pull the weights of their keys from the
        servers, predict, and reply the histogram form of the AUC that the scheduler merges.  (The reference dispatches
        the command and merges the replies, batch_solver.cc:114-123; its worker side is a commented-out sketch,
        batch_solver.cc:437-480.)"""
        data = cfg.AUCData()
        vd = self.conf.validation_data
        if not self.ctx.is_worker or not vd.file:
            return dumps(data, oneline=True).encode()
        H, P = self.H, self.param
        fmt = getattr(H.TextFormat, vd.text if vd.has("text") else "LIBSVM")
        cache = self.conf.local_cache.file[0] if self.conf.local_cache.file else "/tmp/psb200_cache/"
        r = H.SlotReader()
        r.init(cfg.data_files(vd, H), fmt, cache + f"{self.ctx.node_id}_valid/", True, bool(self.flags.shuffle_fea_id),
               bool(self.flags.add_beta_feature), int(self.flags.line_limit), int(self.flags.load_data_max_mb_per_thread))
        r.read(max(int(self.flags.num_threads), 1))
        y = r.value(0).astype(np.float32)
        off, idx, v = r.offset(1).astype(np.int64), r.index(1), r.value(1)
        ukeys, inv = np.unique(idx, return_inverse=True)
        t = T * K_PACE
        P.cust.submit(H.kServerGroup, cmd=PULL, key=ukeys.tobytes(), time=t, key_range=(0, 2**64 - 1), channel=self.ch,
                      erase_key_cache=True, wait=True)
        _, w = P.take_pulled(t)
        w = np.nan_to_num(w, nan=0.0) if len(w) == len(ukeys) else np.zeros(len(ukeys))
        X = sp.csr_matrix((np.ones(len(idx)) if len(v) == 0 else v.astype(np.float64), inv, off), shape=(len(y), len(ukeys)))
        auc = H.AUC()
        auc.set_goodness(int(self.conf.solver.auc_goodness))
        auc.add(y, (X @ w).astype(np.float32))
        data.tp_key, data.tp_count, data.fp_key, data.fp_count = (list(a) for a in auc.data())
        return dumps(data, oneline=True).encode()

    def save_model(self) -> None:
        if not self.ctx.is_server or not self.conf.model_output.file:
            return
        keys = self.param.kv.keys(self.ch)
        w = self.param.kv.values(self.ch)
        write_model_text(f"{self.conf.model_output.file[0]}_{self.ctx.node_id}", keys, w)

    def stop(self) -> None:
        # the job is over; a handler may still wait for a node that is gone (a worker that died): call the waits off
        # first, so that the executor threads can be joined
        self.param.cust.abort_waits()
        self.cust.abort_waits()
        self.cust.stop()
        self.param.cust.stop()
        if self.station is not None:
            if bool(self.flags.verbose):
                print(f"[{self.ctx.node_id}] feature station: {self.station.stats()}", flush=True)
            self.station = None               # joins the prefetch threads, closes the files
            shutil.rmtree(self._station_dir, ignore_errors=True)


class BatchScheduler:
    """Scheduler side: ``BatchSolver::run`` + ``Darling::runIteration``."""

    def __init__(self, ctx: NodeContext, app_conf, flags: cfg.Flags):
        H = host()
        self.H, self.ctx, self.flags, self.app_conf = H, ctx, flags, app_conf
        self.conf = app_conf.linear_method
        self.param = H.Customer(ctx.po, app_conf.parameter_name[0], None, True)
        self.cust = H.Customer(ctx.po, app_conf.app_name, None, False)
        self.progress: List[dict] = []

    def _submit(self, payload: bytes, wait: bool = True, wait_time: int = -1) -> int:
        t = self.cust.submit(self.H.kActiveGroup, payload=payload, wait_time=wait_time)
        if wait:
            self._wait(t)
        return t

    def _wait(self, t: int) -> None:
        """Wait for every node's reply to task ``t``; with heartbeats on (``-report_interval``) a node that stopped
        reporting ends the job with an error instead of holding the scheduler for ever."""
        hb = float(self.flags.report_interval)
        deadline_s = max(5.0 * hb, 2.0) if hb > 0 else 0.0
        while not self.cust.wait_out(self.H.kActiveGroup, t, 0.2):
            if deadline_s > 0:
                dead = self.ctx.po.dead_nodes(deadline_s)
                if dead:
                    raise RuntimeError(f"no heartbeat from {', '.join(dead)} for {deadline_s:g} s")

    def run(self, verbose: bool = True) -> List[dict]:
        from ..models.darlin import Progress, block_order, print_progress

        H, conf, sol = self.H, self.conf, self.conf.solver
        # LOAD_DATA, merge ExampleInfo
        t = self._submit(_call("LOAD_DATA"))
        num_ex = nnz = 0
        kmin, kmax = 2**64 - 1, 0
        per_slot: dict = {}
        for text in self.cust.take_replies(t).values():
            info = parse(text.decode(), cfg.ExampleInfo)
            num_ex += info.num_ex
            for s in info.slot:
                if s.id == 0:
                    continue
                nnz += s.nnz_ele
                kmin, kmax = min(kmin, s.min_key), max(kmax, s.max_key)
                a = per_slot.setdefault(int(s.id), [2**64 - 1, 0, 0, 0])
                a[0], a[1], a[2], a[3] = min(a[0], s.min_key), max(a[1], s.max_key), a[2] + s.nnz_ele, a[3] + s.nnz_ex
        self.num_ex = num_ex
        # feature blocks (batch_solver.cc:48-66): every feature group (slot) is cut by its own density over its own
        # key range; data that comes as one slot is cut as one group over [min_key, max_key)
        if len(per_slot) > 1:
            from ..models.darlin import group_blocks

            cut = group_blocks([(g, a[0], a[1], a[2], a[3]) for g, a in sorted(per_slot.items())], sol.feature_block_ratio)
            self.blocks = [(b, e) for _, b, e in cut]
            self.block_group = [g for g, _, _ in cut]
        else:
            per_row = nnz / max(num_ex, 1)
            nblk = max(int(math.ceil(per_row * sol.feature_block_ratio)), 1) if per_row > 1 + 1e-6 and sol.feature_block_ratio > 0 else 1
            span = kmax - kmin
            bounds = [kmin + span * i // nblk for i in range(nblk)] + [kmax]
            self.blocks = [(bounds[i], bounds[i + 1]) for i in range(nblk)]
            self.block_group = None
        nblk = len(self.blocks)
        self._submit(_call("PREPROCESS_DATA"))
        # iterations
        tau = sol.max_block_delay
        orders = block_order(nblk, sol.max_pass_of_data, sol.random_feature_block_order, int(self.flags.seed))
        # blocks of the important feature groups come first in the first pass, num_iter_for_prior_fea_group times
        # each and with zero delay (batch_solver.cc:89-107, darling.cc:39-50).  A TERAFEA key carries its group in
        # its top 10 bits, so a group's blocks are those whose key range meets the group's.
        prior: List[int] = []
        prng = np.random.RandomState(int(self.flags.seed) + 1)
        if self.block_group is not None:
            from ..models.darlin import prior_block_order

            prior = prior_block_order(self.block_group, [int(g) for g in sol.prior_fea_group],
                                      int(sol.num_iter_for_prior_fea_group), bool(sol.random_feature_block_order), int(self.flags.seed))
        for g in ([] if self.block_group is not None else sol.prior_fea_group):
            glo, ghi = int(g) << 54, (int(g) + 1) << 54
            tmp = [k for k, (b0, b1) in enumerate(self.blocks) if max(b0, glo) < min(b1, ghi)]
            for _ in range(int(sol.num_iter_for_prior_fea_group) if tmp else 0):
                if sol.random_feature_block_order:
                    prng.shuffle(tmp)
                prior += list(tmp)
        self.prior_blocks = prior
        kkt, reset = 1e20, False
        first_task = None
        tm = None
        t_start = time.time()
        for it in range(sol.max_pass_of_data):
            t_it = time.time()
            order = (prior if it == 0 else []) + orders[it].tolist()
            for i, b in enumerate(order):
                kw = dict(key=self.blocks[b], fea_grp=[1 if self.block_group is None else int(self.block_group[b])])
                if i == 0:
                    kw["kkt_filter_threshold"] = kkt
                    if reset:
                        kw["kkt_filter_reset"] = True
                wait_time = -1
                if tm is not None and first_task is not None and (tm + 1) - tau > first_task:
                    wait_time = tm if (it == 0 and i < len(prior)) else tm - tau       # zero delay for the prior blocks
                tm = self._submit(_call("UPDATE_MODEL", **kw), wait=False, wait_time=wait_time)
                if first_task is None:
                    first_task = tm
            wt = tm - tau if tm - tau >= first_task else first_task
            te = self._submit(_call("EVALUATE_PROGRESS"), wait=True, wait_time=wt)
            tm = te
            objv, nnz_w, nnz_as, vio, busy = 0.0, 0, 0, 0.0, []
            for text in self.cust.take_replies(te).values():
                p = parse(text.decode(), cfg.Progress)
                objv += p.objv
                nnz_w += p.nnz_w
                nnz_as += p.nnz_active_set
                vio = max(vio, p.violation)
                busy += list(p.busy_time)
            rel = 1.0 if not self.progress else self.progress[-1]["objv"] / objv - 1.0
            rec = dict(objv=objv, relative_objv=rel, nnz_w=nnz_w, violation=vio, nnz_active_set=nnz_as,
                       kkt_threshold=kkt, total_time=time.time() - t_start, busy_time=busy)
            self.progress.append(rec)
            if verbose:
                print_progress(it, Progress(objv, rel, nnz_w, vio, nnz_as, kkt, time.time() - t_it), file=sys.stderr, busy=busy or None)
            kkt = vio / max(num_ex, 1) * conf.darling.kkt_filter_threshold_ratio
            if 0 < rel <= sol.epsilon:
                if reset:
                    break
                reset = True
            else:
                reset = False
        if conf.has("validation_data") and conf.validation_data.file:
            tv = self._submit(_call("COMPUTE_VALIDATION_AUC"))
            auc = self.H.AUC()
            auc.set_goodness(int(sol.auc_goodness))
            for text in self.cust.take_replies(tv).values():
                d = parse(text.decode(), cfg.AUCData)
                auc.merge_data(list(d.tp_key), list(d.tp_count), list(d.fp_key), list(d.fp_count))
            self.validation = dict(auc=auc.evaluate(), accuracy=auc.accuracy(0.0))
            if self.progress:
                self.progress[-1]["validation_auc"] = self.validation["auc"]
                self.progress[-1]["validation_accuracy"] = self.validation["accuracy"]
            if verbose:
                print(f"\tEvaluation accuracy: {self.validation['accuracy']:.6g}, auc: {self.validation['auc']:.6g}", file=sys.stderr)
        self._submit(_call("SAVE_MODEL"))
        return self.progress

    def stop(self) -> None:
        self.cust.stop()
        self.param.stop()
