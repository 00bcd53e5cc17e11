"""A scheduler node for GPU jobs: the host control plane drives the passes of a batch job on GPU ranks.

In the reference the scheduler owns the loop of a batch job (src/linear_method/batch_solver.cc:69-132,
src/linear_method/darling.cc:30-101): it submits tasks to the workers and servers, merges their ``Progress`` replies,
prints the table, applies the stopping rule and finally asks for the model; a monitor thread prints the heartbeat
table of all nodes (src/system/postoffice.cc:271-374).  GPU ranks by default run that loop themselves, in lock step,
with ``torch.distributed`` as the only control plane.  With ``-gpu_scheduler`` the loop moves to a scheduler node:

* rank 0 also runs the scheduler node ``H`` (post office + TCP van on the loopback); every rank runs a worker node
  ``W<rank>`` whose server half lives in the same process (the data plane stays inside the kernels, over NVLink);
* a task covers a whole pass, not one block: a pass is one kernel launch here, and the block order of the pass
  (with the zero-delay sweeps over the important groups in front) travels in the task (``block_order``,
  ``num_prior``) — one message per block would cost more than the block;
* every rank answers with the ``Progress`` of the pass (already merged on the device); the scheduler checks that the
  ranks agree, prints the table, applies the reference's stopping rule and sends ``SAVE_MODEL``;
* with ``-report_interval`` the workers' heartbeats carry the device and its memory in use, and the scheduler prints
  the dashboard.

The solver only needs ``nblk``, ``cfg``, ``block_group``, ``progress``, ``run_pass(order, reset, prior)`` and
``save_model(prefix)``, which is what the CPU test's stand-in provides.

Online (FTRL) jobs follow ``FTRL::run`` (src/linear_method/ftrl.cc:38-59) the same way: one UPDATE_MODEL task runs a
rank's whole training loop, the ranks send the reference's worker and server progress reports while they train, and
the scheduler (the one of the CPU-node job, ``apps/ftrl_cpu.py::FTRLScheduler``) shows the merged line every
``eval_interval``, collects the final progress and sends SAVE_MODEL (:func:`run_scheduled_online`).
"""
from __future__ import annotations

import copy
import socket
import sys
import threading
import time
from typing import List, Optional

import numpy as np

from .. import config as cfg
from ..runtime import host
from ..runtime.node import NodeContext, dashboard, start_node
from ..utils.pbtext import dumps, parse


def _call(cmd: str, **kw) -> bytes:
    m = cfg.LMCall(cmd=cmd)
    for k, v in kw.items():
        m.set(k, v)
    return dumps(m, oneline=True).encode()


ERROR_PREFIX = b"ERROR: "


class GpuWorkerNode:
    """Worker + server of one GPU rank: runs the scheduler's tasks on the solver, on the node's executor thread."""

    def __init__(self, ctx: NodeContext, app_name: str, sol, model_prefix: str = "", device=None):
        self.ctx, self.sol, self.model_prefix, self.device = ctx, sol, model_prefix, device
        self.saved: Optional[str] = None
        self.failed: Optional[str] = None
        if ctx.hb_state is not None:
            ctx.hb_state["where"] = self._where()        # the first heartbeat already names the device
        self.cust = host().Customer(ctx.po, app_name, self.process, False)

    def _where(self) -> str:
        if self.device is None or getattr(self.device, "type", "cpu") != "cuda":
            return ""
        import torch

        free, total = torch.cuda.mem_get_info(self.device)
        return f" {self.device} hbm {(total - free) / 2**30:.1f}/{total / 2**30:.0f}GB"

    def process(self, msg) -> None:
        if not msg.request:
            return
        t0 = time.time()
        reply = b""
        try:
            if self.device is not None and getattr(self.device, "type", "cpu") == "cuda":
                import torch

                torch.cuda.set_device(self.device)           # the executor thread has no current device of its own
            call = parse(msg.payload.decode(), cfg.LMCall)
            if self.ctx.hb_state is not None:
                self.ctx.hb_state["task"] = msg.time
            if call.cmd == "UPDATE_MODEL":
                order = np.asarray(list(call.block_order), dtype=np.int32)
                n_prior = int(call.num_prior)
                prior = order[:n_prior].tolist() if n_prior > 0 else None
                p = self.sol.run_pass(order[n_prior:], bool(call.kkt_filter_reset), prior)
                reply = dumps(cfg.Progress(objv=float(p.objv), relative_objv=float(p.relative_objv), nnz_w=int(p.nnz_w),
                                           violation=float(p.violation), nnz_active_set=int(p.nnz_active),
                                           total_time=float(p.seconds), kkt_threshold=float(p.kkt_threshold)),
                               oneline=True).encode()
            elif call.cmd == "SAVE_MODEL":
                if self.model_prefix:
                    self.saved = self.sol.save_model(self.model_prefix)
                    reply = self.saved.encode()
            # LOAD_DATA / PREPROCESS_DATA are done before the control plane starts (they are collective set-up);
            # RECOVER does nothing, as in the reference
            if self.ctx.hb_state is not None:
                self.ctx.hb_state["where"] = self._where()
        except Exception as e:  # noqa: BLE001 - the scheduler must hear about it instead of waiting forever
            import traceback

            self.failed = traceback.format_exc()
            reply = ERROR_PREFIX + f"{type(e).__name__}: {e}".encode()
        self.ctx.add_busy(time.time() - t0)
        self.cust.reply(msg, payload=reply)

    def stop(self) -> None:
        self.cust.stop()


class GpuBatchScheduler:
    """Scheduler side of a batch job on GPU ranks: one UPDATE_MODEL task per pass."""

    def __init__(self, ctx: NodeContext, app_name: str, solver_cfg, nblk: int, block_group, verbose: bool = True,
                 deadline_s: float = 0.0):
        self.H, self.ctx, self.deadline_s = host(), ctx, float(deadline_s)
        self.cfg, self.nblk, self.block_group, self.verbose = solver_cfg, nblk, block_group, verbose
        self.cust = self.H.Customer(ctx.po, app_name, None, False)
        self.progress: List[dict] = []
        self.saved: List[str] = []

    def _round(self, payload: bytes) -> dict:
        """One task to every rank; returns their replies.  Does not wait for ever: a rank's error reply ends the round
        at once, and with heartbeats on (``-report_interval``) so does a rank that stopped reporting."""
        t = self.cust.submit(self.H.kWorkerGroup, payload=payload)
        replies: dict = {}

        def check():
            replies.update(self.cust.take_replies(t))
            for nid, text in replies.items():
                if bytes(text).startswith(ERROR_PREFIX):
                    raise RuntimeError(f"{nid}: {bytes(text)[len(ERROR_PREFIX):].decode()}")

        while not self.cust.wait_out(self.H.kWorkerGroup, t, 0.2):
            check()
            if self.deadline_s > 0:
                dead = self.ctx.po.dead_nodes(self.deadline_s)
                if dead:
                    raise RuntimeError(f"no heartbeat from {', '.join(dead)} for {self.deadline_s:g} s")
        check()
        return replies

    def run(self) -> List[dict]:
        from ..models.darlin import Progress, block_order, print_progress, prior_block_order

        c = self.cfg
        orders = block_order(self.nblk, c.max_pass, c.random_block_order, c.seed)
        prior = prior_block_order(self.block_group, c.prior_fea_group, c.num_iter_for_prior_fea_group, c.random_block_order, c.seed)
        reset = False
        t_start = time.time()
        for it in range(c.max_pass):
            first = prior if it == 0 else []
            t_it = time.time()
            replies = self._round(_call("UPDATE_MODEL", block_order=[int(b) for b in first] + orders[it].tolist(),
                                        num_prior=len(first), kkt_filter_reset=reset))
            ps = {nid: parse(bytes(text).decode(), cfg.Progress) for nid, text in replies.items()}
            p0 = next(iter(ps.values()))
            for nid, p in ps.items():      # the ranks merged their parts on the device: they must report the same pass
                if abs(p.objv - p0.objv) > 1e-9 * max(abs(p0.objv), 1.0) or p.nnz_w != p0.nnz_w:
                    raise RuntimeError(f"pass {it}: {nid} reports objective {p.objv} / {p.nnz_w} non-zeros, others {p0.objv} / {p0.nnz_w}")
            rec = dict(objv=p0.objv, relative_objv=p0.relative_objv, nnz_w=int(p0.nnz_w), violation=p0.violation,
                       nnz_active_set=int(p0.nnz_active_set), kkt_threshold=p0.kkt_threshold, total_time=time.time() - t_start,
                       busy_time=[p.total_time for p in ps.values()])
            self.progress.append(rec)
            if self.verbose:
                print_progress(it, Progress(p0.objv, p0.relative_objv, int(p0.nnz_w), p0.violation, int(p0.nnz_active_set),
                                            p0.kkt_threshold, time.time() - t_it), file=sys.stderr, busy=rec["busy_time"] or None)
            if 0 < p0.relative_objv <= c.epsilon:
                if reset:
                    break
                reset = True
            else:
                reset = False
        self.saved = sorted(bytes(t).decode() for t in self._round(_call("SAVE_MODEL")).values() if bytes(t))
        return self.progress

    def stop(self) -> None:
        self.cust.stop()


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _start_nodes(group, flags: cfg.Flags):
    """The nodes of a scheduled GPU job: every rank starts its worker node ``W<rank>``; rank 0 also starts the scheduler
    ``H`` (in a thread of its own: it waits for all workers to register) on a free loopback port that the ranks
    learn over the process group.  Returns (worker context, {"ctx": scheduler context} on rank 0, the boot thread)."""
    import torch.distributed as dist

    W = int(group.world)
    port = [_free_port() if group.rank == 0 else 0]
    if W > 1:
        dist.broadcast_object_list(port, src=0, group=group.group)
    f = copy.copy(flags)
    f.num_workers, f.num_servers, f.num_unused, f.num_replicas = W, 0, 0, 0
    f.scheduler = f"role:SCHEDULER,hostname:'127.0.0.1',port:{int(port[0])},id:'H'"
    f.interface = ""
    sched_ctx: dict = {}
    th = None
    if group.rank == 0:
        def boot():
            try:
                sched_ctx["ctx"] = start_node(0, f)
            except Exception as e:  # noqa: BLE001
                sched_ctx["error"] = e

        th = threading.Thread(target=boot, name="H-boot", daemon=True)
        th.start()
    ctx = start_node(group.rank + 1, f)
    return ctx, sched_ctx, th


def run_scheduled(group, flags: cfg.Flags, app_name: str, sol, model_prefix: str = "", verbose: bool = True) -> dict:
    """Run the passes of ``sol`` (already preprocessed, on every rank) under a scheduler node on rank 0.

    Collective over ``group`` (``rank``, ``world``, ``group`` = the torch.distributed group, ``device``,
    ``barrier()``).  Returns on every rank ``{"progress": solver.progress, "model": path or None}``; rank 0 adds the
    scheduler's own records under ``"scheduler"`` and the last dashboard under ``"dashboard"``."""
    ctx, sched_ctx, th = _start_nodes(group, flags)
    node = GpuWorkerNode(ctx, app_name, sol, model_prefix, getattr(group, "device", None))
    out: dict = {}
    try:
        if th is not None:
            th.join()
            if "error" in sched_ctx:
                raise sched_ctx["error"]
        group.barrier()                                   # every rank's customer exists before the first task goes out
        if group.rank == 0:
            hctx = sched_ctx["ctx"]
            every = float(flags.report_interval)
            sched = GpuBatchScheduler(hctx, app_name, sol.cfg, sol.nblk, sol.block_group, verbose,
                                      deadline_s=max(5.0 * every, 2.0) if every > 0 else 0.0)
            stop_monitor = threading.Event()
            if float(flags.report_interval) > 0:
                def monitor():
                    while not stop_monitor.wait(float(flags.report_interval)):
                        print(dashboard(hctx.po), file=sys.stderr, flush=True)

                threading.Thread(target=monitor, name="H-monitor", daemon=True).start()
            try:
                out["scheduler"] = sched.run()
                out["saved"] = sched.saved
                if float(flags.report_interval) > 0:
                    # a short job can end before the first report is due: wait for every worker's first one (bounded)
                    deadline = time.time() + 3.0 * float(flags.report_interval) + 1.0
                    while time.time() < deadline and not all(text for _, text in hctx.po.heartbeats().values()):
                        time.sleep(0.01)
                    out["dashboard"] = dashboard(hctx.po)
            finally:
                stop_monitor.set()
                hctx.po.stop_all()                        # TERMINATE to every node, this process's worker included
                sched.stop()
        ctx.po.wait_terminate(1e9)
    finally:
        node.stop()
        ctx.stop()
        if "ctx" in sched_ctx:
            sched_ctx["ctx"].stop()
    if node.failed:
        raise RuntimeError(f"rank {group.rank}: a task failed\n{node.failed}")
    out["progress"] = sol.progress
    out["model"] = node.saved
    return out


# ---------------------------------------------------------------------------------------------------------------
# online jobs: one UPDATE_MODEL task for the whole stream, periodic progress reports to the scheduler
class GpuOnlineWorkerNode:
    """Worker + server of one GPU rank of an online (FTRL) job.  The scheduler's single UPDATE_MODEL task runs the
    rank's whole training loop on the node's executor thread; the loop calls :meth:`report` now and then, which
    sends the reference's two kinds of REPORT_PROGRESS to the scheduler: the worker's (loss and examples since its
    last report) and the server's (penalty and non-zeros of its shard) — src/linear_method/ftrl.cc:184-201."""

    def __init__(self, ctx: NodeContext, app_name: str, run_training, final_progress, save_model, device=None):
        self.ctx, self.device = ctx, device
        self.run_training, self.final_progress, self.save_model = run_training, final_progress, save_model
        self.result = None
        self.saved: Optional[str] = None
        self.failed: Optional[str] = None
        self.cust = host().Customer(ctx.po, app_name, self.process, False)

    def report(self, loss_sum: float, examples: int, penalty: float, nnz_w: int) -> None:
        self.cust.submit("H", payload=_call("REPORT_PROGRESS", progress=cfg.Progress(objv=float(loss_sum), num_ex_trained=int(examples))))
        self.cust.submit("H", payload=_call("REPORT_PROGRESS", progress=cfg.Progress(objv=float(penalty), nnz_w=int(nnz_w))))

    def process(self, msg) -> None:
        if not msg.request:
            return
        t0 = time.time()
        reply = b""
        try:
            if self.device is not None and getattr(self.device, "type", "cpu") == "cuda":
                import torch

                torch.cuda.set_device(self.device)
            call = parse(msg.payload.decode(), cfg.LMCall)
            if self.ctx.hb_state is not None:
                self.ctx.hb_state["task"] = msg.time
            if call.cmd == "UPDATE_MODEL":
                self.result = self.run_training(self.report)
            elif call.cmd == "EVALUATE_PROGRESS":
                objv, nnz_w, examples = self.final_progress()
                reply = dumps(cfg.Progress(objv=float(objv), nnz_w=int(nnz_w), num_ex_trained=int(examples)), oneline=True).encode()
            elif call.cmd == "SAVE_MODEL":
                self.saved = self.save_model()
                reply = (self.saved or "").encode()
        except Exception as e:  # noqa: BLE001 - the scheduler must hear about it instead of waiting forever
            import traceback

            self.failed = traceback.format_exc()
            reply = ERROR_PREFIX + f"{type(e).__name__}: {e}".encode()
        self.ctx.add_busy(time.time() - t0)
        self.cust.reply(msg, payload=reply)

    def stop(self) -> None:
        self.cust.stop()


def run_scheduled_online(group, flags: cfg.Flags, app_conf, run_training, final_progress, save_model, verbose: bool = True) -> dict:
    """An online job under a scheduler node on rank 0 (``FTRL::run``, src/linear_method/ftrl.cc:38-59): UPDATE_MODEL to
    every rank, the merged progress line every ``eval_interval`` while the ranks train, EVALUATE_PROGRESS, SAVE_MODEL.

    ``run_training(report)`` is the rank's whole training loop (``report(loss_sum, examples, penalty, nnz_w)`` at its
    own pace), ``final_progress()`` returns ``(objective part, non-zeros, examples)`` of this rank, ``save_model()``
    the path it wrote.  Collective over ``group``.  Returns ``{"result": run_training's value, "model": path}``; rank 0
    adds ``"scheduler"`` (the scheduler's record: totals, worker reports, printed lines)."""
    from .ftrl_cpu import FTRLScheduler

    ctx, sched_ctx, th = _start_nodes(group, flags)
    node = GpuOnlineWorkerNode(ctx, app_conf.app_name or "linear_method", run_training, final_progress, save_model,
                               getattr(group, "device", None))
    out: dict = {}
    try:
        if th is not None:
            th.join()
            if "error" in sched_ctx:
                raise sched_ctx["error"]
        group.barrier()
        if group.rank == 0:
            hctx = sched_ctx["ctx"]
            sched = FTRLScheduler(hctx, app_conf, flags)
            try:
                out["scheduler"] = sched.run(verbose=verbose)
            finally:
                hctx.po.stop_all()
                sched.stop()
        ctx.po.wait_terminate(1e9)
    finally:
        node.stop()
        ctx.stop()
        if "ctx" in sched_ctx:
            sched_ctx["ctx"].stop()
    if node.failed:
        raise RuntimeError(f"rank {group.rank}: a task failed\n{node.failed}")
    out["result"] = node.result
    out["model"] = node.saved
    return out
