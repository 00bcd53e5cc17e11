"""Online FTRL on CPU nodes, driven through the control-plane runtime (scheduler, servers, workers).

The multi-process form of the reference's online solver for deployments without GPUs and as the
protocol-level twin of the GPU engine (``models/ftrl.py``).  Reference roles: ``FTRL::run`` (scheduler
starts the system, sends UPDATE_MODEL to everybody, saves the model; src/linear_method/ftrl.cc:38-59),
``FTRL::updateModel`` (worker loop: read a minibatch, count keys, tail filter through the servers'
count-min sketch, pull the working set, loss + gradient + pos/neg counts, push;
src/linear_method/ftrl.cc:61-152), ``FTRLModel::setValue / getValue`` (per-key server update with the
count-based learning rate; src/linear_method/ftrl_model.h:60-112).

Consistency: like the reference, pushes are not waited for (eventual consistency); a worker's pull
of minibatch t only waits for its own filter round trip.  With one worker the run is deterministic
and equals the fp64 oracle step by step.
"""
from __future__ import annotations

import math
import sys
import threading
import time
from typing import Dict, List

import numpy as np

from .. import config as cfg
from ..runtime import host
from ..runtime.node import NodeContext
from ..utils.modelio import write_model_text
from ..utils.pbtext import dumps, parse
from .linear_cpu import F_INSERT_KEY_FREQ, PULL, PUSH, U64, _call

ALL_KEYS = (0, 2**64 - 1)


class FTRLNode:
    """Worker or server side of the online solver (one instance per non-scheduler node)."""

    def __init__(self, ctx: NodeContext, app_conf, flags: cfg.Flags):
        H = host()
        self.H, self.ctx, self.flags, self.app_conf = H, ctx, flags, app_conf
        self.conf = app_conf.linear_method
        lam = list(self.conf.penalty.get("lambda")) + [0.0, 0.0]
        lr = self.conf.learning_rate
        # the shared parameter: a native customer that keeps this server's FTRL model (key -> {pos, neg, w, z}), applies
        # pushes as they arrive and answers pulls on its executor thread (csrc/host/shared_param.h::FTRLParamCustomer)
        s = self.conf.solver
        self.param = H.FTRLParamCustomer(ctx.po, app_conf.parameter_name[0], lr.alpha, lr.beta, lam[0], lam[1],
                                         max(int(s.countmin_n) // max(ctx.num_servers, 1), 64), int(s.countmin_k))
        self.store = self.param
        self.cust = H.Customer(ctx.po, app_conf.app_name, self.process, False)
        self.examples, self.loss_sum, self.steps = 0, 0.0, 0
        self._reporting = threading.Event()       # set when the periodic server reports must end
        self._stopping = threading.Event()        # set when the job is over: a stream still running is abandoned

    def _take(self, t: int):
        """The replies of pull ``t`` concatenated in server (= key) order: (keys, values)."""
        return self.param.take_pulled(t, self.param.group(self.H.kServerGroup))

    # ---- application calls from the scheduler
    def process(self, msg) -> None:
        if not msg.request:
            return
        call = parse(msg.payload.decode(), cfg.LMCall)
        reply = b""
        if call.cmd == "UPDATE_MODEL":
            if self.ctx.is_worker:
                self.update_model()
            else:
                self._start_server_reports()
        elif call.cmd == "EVALUATE_PROGRESS":
            self._reporting.set()                 # training is over: the periodic reports end
            reply = self.progress()
        elif call.cmd == "SAVE_MODEL":
            self.save_model()
        self.cust.reply(msg, payload=reply)

    def _penalty(self):
        n1, n2, nnz = self.store.stats()
        lam = list(self.conf.penalty.get("lambda")) + [0.0, 0.0]
        return lam[0] * n1 + 0.5 * lam[1] * math.sqrt(max(n2, 0.0)), nnz

    def _start_server_reports(self) -> None:
        """A server returns from UPDATE_MODEL at once and keeps reporting the penalty and the non-zeros of its shard
        every ``eval_interval`` seconds while the workers train (FTRL::updateModel / evalProgress, ftrl.cc:61-69,184-197)."""
        every = float(self.conf.solver.eval_interval)
        if every <= 0:
            return

        def loop():
            while not self._reporting.wait(every):
                pen, nnz = self._penalty()
                self.cust.submit("H", payload=_call("REPORT_PROGRESS", progress=cfg.Progress(objv=pen, nnz_w=int(nnz))))

        threading.Thread(target=loop, name=f"{self.ctx.node_id}-progress", daemon=True).start()

    def update_model(self) -> None:
        """FTRL::updateModel: one pass over this worker's files in minibatches."""
        H, P, s = self.H, self.param, self.conf.solver
        td = self.conf.training_data
        files = H.search_files(cfg.data_files(td, H))
        if not files:
            return
        reader = H.StreamReader()
        reader.init(files, getattr(H.TextFormat, td.text if td.has("text") else "LIBSVM"), True, bool(self.flags.shuffle_fea_id))
        mb, freq = int(s.minibatch_size), int(s.tail_feature_freq)
        ch = 0
        last_push = None
        last_report, reported = time.time(), [0.0, 0]
        # a reader thread parses ahead of the solver into a bounded buffer (FTRL::run's reader thread and
        # threadsafeLimitedQueue, src/linear_method/ftrl.cc:38-59); parsing runs without the interpreter lock
        import queue

        ahead: "queue.Queue" = queue.Queue(maxsize=max(int(self.flags.num_threads), 2))

        def read_ahead():
            try:
                while True:
                    out = reader.read(mb)
                    ahead.put(out)
                    if out is None:
                        return
            except BaseException as e:          # hand the error to the solver thread instead of dying silently
                ahead.put(e)

        threading.Thread(target=read_ahead, name=f"{self.ctx.node_id}-reader", daemon=True).start()
        while not self._stopping.is_set():
            out = ahead.get()
            if isinstance(out, BaseException):
                raise out
            if out is None:
                break
            slots, info = out
            rows = info["num_ex"]
            y = np.where(slots[0]["value"] > 0, 1.0, -1.0)
            sl = slots.get(1)
            if sl is None or len(sl["index"]) == 0:
                continue
            off = sl["offset"].astype(np.int64)
            idx = sl["index"]
            val = sl["value"].astype(np.float64) if len(sl["value"]) else np.ones(len(idx))
            # the minibatch's keys: unique with counts (FTRL::countKeys, ftrl.cc:154-174) and the local id of every
            # non-zero, in the native runtime (csrc/host/localizer.h)
            T_ = max(int(self.flags.num_threads), 1)
            ukeys, cnt, inv = H.localize(idx)
            ch += 1
            if freq > 0:      # tail filter: insert this minibatch's key counts, keep the keys above the threshold
                P.submit(H.kServerGroup, cmd=PUSH, key=ukeys.tobytes(), values=[cnt.astype(np.uint32).tobytes()],
                         key_range=ALL_KEYS, channel=ch, flags=F_INSERT_KEY_FREQ, wait=True)
                t = P.submit(H.kServerGroup, cmd=PULL, key=ukeys.tobytes(), key_range=ALL_KEYS, channel=ch, aux=freq,
                             erase_key_cache=True, wait=True)
                kept, _ = self._take(t)
            else:
                kept = ukeys
            t = P.submit(H.kServerGroup, cmd=PULL, key=kept.tobytes(), key_range=ALL_KEYS, channel=ch, wait=True)
            _, wk = self._take(t)
            if len(wk) != len(kept):
                wk = np.zeros(len(kept))
            pos_k = np.searchsorted(kept, ukeys)
            in_set = (pos_k < len(kept)) & (kept[np.minimum(pos_k, max(len(kept) - 1, 0))] == ukeys) if len(kept) else np.zeros(len(ukeys), bool)
            w_u = np.where(in_set, wk[np.minimum(pos_k, max(len(kept) - 1, 0))] if len(kept) else 0.0, 0.0)
            # margins, loss, per-key gradient and label counts in the native runtime (csrc/host/ftrl_cpu.h)
            loss, g, pos, neg = H.ftrl_minibatch(off, inv, val if len(sl["value"]) else None, y, w_u, T_)
            self.loss_sum += float(loss)
            self.examples += rows
            self.steps += 1
            last_push = P.submit(H.kServerGroup, cmd=PUSH, key=ukeys[in_set].tobytes(),
                                 values=[g[in_set].tobytes(), pos[in_set].tobytes(), neg[in_set].tobytes()],
                                 key_range=ALL_KEYS, channel=ch, erase_key_cache=True)
            # periodic progress report to the scheduler (FTRL::evalProgress / showProgress, ftrl.cc:184-219)
            if time.time() - last_report >= float(s.eval_interval):
                last_report = time.time()
                rep = cfg.Progress(objv=self.loss_sum - reported[0], num_ex_trained=self.examples - reported[1])
                reported = [self.loss_sum, self.examples]
                self.cust.submit("H", payload=_call("REPORT_PROGRESS", progress=rep))   # "H" = the scheduler's node id
        # pushes are not waited for while training; before reporting back, the last one must have been applied
        # (a server handles one sender's messages in order, so that covers the earlier ones too)
        if last_push is not None:
            P.wait_out(H.kServerGroup, last_push)

    def progress(self) -> bytes:
        pen, nnz = self._penalty() if self.ctx.is_server else (0.0, 0)
        p = cfg.Progress(objv=self.loss_sum + pen, nnz_w=nnz, num_ex_trained=self.examples)
        return dumps(p, oneline=True).encode()

    def save_model(self) -> None:
        mo = self.conf.model_output
        if self.ctx.is_server and mo.file:
            k, v = self.store.nonzero()
            write_model_text(f"{mo.file[0]}_{self.ctx.node_id}", k, v)

    def stop(self) -> None:
        self._reporting.set()
        self._stopping.set()
        self.param.abort_waits()          # a handler may still wait for a node that is gone
        self.cust.abort_waits()
        self.cust.stop()
        self.param.stop()


class FTRLScheduler:
    """Scheduler side: ``FTRL::run``."""

    def __init__(self, ctx: NodeContext, app_conf, flags: cfg.Flags):
        H = host()
        self.H, self.ctx, self.flags, self.app_conf = H, ctx, flags, app_conf
        self.param = H.Customer(ctx.po, (list(app_conf.parameter_name) or [app_conf.app_name + "_w"])[0], None, True)
        self.verbose = True
        self.reports: List[dict] = []          # periodic worker reports, in arrival order
        self._seen, self._loss = 0, 0.0
        self._mu = threading.Lock()
        self._window = [0.0, 0]                # workers' loss sum and examples since the last printed line
        self._servers: Dict[str, tuple] = {}   # server id -> its latest (penalty, non-zeros)
        self.lines: List[str] = []             # the progress lines printed so far
        self.cust = H.Customer(ctx.po, app_conf.app_name, self.process, False)
        self.progress: List[dict] = []

    def process(self, msg) -> None:
        """Workers' REPORT_PROGRESS calls: running totals and the mean loss since the previous report."""
        if not msg.request or not msg.payload:
            return
        call = parse(msg.payload.decode(), cfg.LMCall)
        if call.cmd != "REPORT_PROGRESS":
            return
        p = call.progress
        with self._mu:
            if not p.has("num_ex_trained"):        # a server: penalty and non-zeros of its shard
                self._servers[msg.sender] = (p.objv, int(p.nnz_w))
                return
            self._seen += p.num_ex_trained
            self._loss += p.objv
            self._window[0] += p.objv
            self._window[1] += p.num_ex_trained
            rec = dict(worker=msg.sender, examples=self._seen, mean_loss=p.objv / max(p.num_ex_trained, 1))
            self.reports.append(rec)
        if float(self.app_conf.linear_method.solver.eval_interval) <= 0:
            self.show_progress()                   # every report is shown when there is no interval

    def show_progress(self) -> None:
        """FTRL::showProgress (ftrl.cc:203-219): examples so far, the workers' mean loss since the last line, the servers'
        penalty and non-zeros as last reported."""
        with self._mu:
            loss, n = self._window
            self._window = [0.0, 0]
            pen = sum(v[0] for v in self._servers.values())
            nnz = sum(v[1] for v in self._servers.values())
            line = "%10d examples, loss %.5e, penalty %.5e, |w|_0 %8d" % (self._seen, loss / max(n, 1), pen, nnz)
            self.lines.append(line)
        if self.verbose:
            print(line, file=sys.stderr)

    def run(self, verbose: bool = True) -> List[dict]:
        H = self.H
        self.verbose = verbose
        t0 = time.time()
        every = float(self.app_conf.linear_method.solver.eval_interval)
        done = threading.Event()
        if every > 0:                                    # the thread that shows the merged progress (ftrl.cc:41-48)
            def shower():
                while not done.wait(every):
                    self.show_progress()

            threading.Thread(target=shower, name="H-progress", daemon=True).start()
        t = self.cust.submit(H.kActiveGroup, payload=_call("UPDATE_MODEL"))
        # workers return when their data is exhausted and applied; servers return at once and report while the workers
        # train.  The wait is not for ever: a node's error reply (a GPU rank's training loop that failed,
        # apps/gpu_control.py) ends it at once, and with heartbeats on so does a node that stopped reporting.
        hb = float(self.flags.report_interval)
        deadline_s = max(5.0 * hb, 2.0) if hb > 0 else 0.0
        replies: dict = {}
        try:
            while True:
                finished = self.cust.wait_out(H.kActiveGroup, t, 0.2)
                replies.update(self.cust.take_replies(t))
                for nid, text in replies.items():
                    if bytes(text).startswith(b"ERROR: "):
                        raise RuntimeError(f"{nid}: {bytes(text)[7:].decode()}")
                if finished:
                    break
                if deadline_s > 0:
                    dead = self.ctx.po.dead_nodes(deadline_s)
                    if dead:
                        raise RuntimeError(f"no heartbeat from {', '.join(dead)} for {deadline_s:g} s")
        finally:
            done.set()
        t = self.cust.submit(H.kActiveGroup, payload=_call("EVALUATE_PROGRESS"))
        self.cust.wait_out(H.kActiveGroup, t)
        objv, nnz_w, examples = 0.0, 0, 0
        for text in self.cust.take_replies(t).values():
            p = parse(text.decode(), cfg.Progress)
            objv += p.objv
            nnz_w += p.nnz_w
            examples += p.num_ex_trained
        rec = dict(objv=objv, nnz_w=nnz_w, examples=examples, seconds=time.time() - t0, reports=list(self.reports), lines=list(self.lines))
        self.progress.append(rec)
        if verbose:
            print("%10d examples, objective %.5e, |w|_0 %8d, %.2f s" % (examples, objv, nnz_w, rec["seconds"]), file=sys.stderr)
        t = self.cust.submit(H.kActiveGroup, payload=_call("SAVE_MODEL"))
        self.cust.wait_out(H.kActiveGroup, t)
        return self.progress

    def stop(self) -> None:
        self.cust.stop()
        self.param.stop()
