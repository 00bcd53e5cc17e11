"""Run one node of a job (scheduler, server or worker) from flags + an app config file.

Equivalent of ``Postoffice::run`` in the reference (src/system/postoffice.cc:34-84): the scheduler
reads ``-app``, assigns the training files to the workers, ships the configuration to every node,
runs the application and finally tells everybody to terminate; the other nodes create the
application when its configuration arrives and serve until TERMINATE.
"""
from __future__ import annotations

import threading
from typing import Optional

from .. import config as cfg
from ..runtime import host
from ..runtime.node import NodeContext, start_node
from ..utils.pbtext import dumps, parse


def make_app(ctx: NodeContext, app_conf, flags: cfg.Flags):
    """LinearMethod::create (src/linear_method/linear_method.cc:20-39) for CPU nodes."""
    lm = app_conf.linear_method
    if not app_conf.has("linear_method"):
        raise ValueError("only linear_method apps run on CPU nodes")
    if not lm.has("solver") and lm.has("validation_data") and lm.has("model_input"):
        from .model_evaluation import ModelEvaluationNode

        return ModelEvaluationNode(ctx, app_conf, flags)
    if lm.solver.minibatch_size <= 0:
        if not lm.has("darling"):
            raise ValueError("batch solver without darling{} is not available on CPU nodes; use the GPU engine")
        from .linear_cpu import BatchScheduler, LinearMethodNode

        return BatchScheduler(ctx, app_conf, flags) if ctx.is_scheduler else LinearMethodNode(ctx, app_conf, flags)
    if not lm.has("ftrl"):
        raise ValueError("online solver requested (solver.minibatch_size > 0) but no ftrl{} section")
    from .ftrl_cpu import FTRLNode, FTRLScheduler

    return FTRLScheduler(ctx, app_conf, flags) if ctx.is_scheduler else FTRLNode(ctx, app_conf, flags)


def run_node(rank: int, flags: cfg.Flags, hub=None, app_text: Optional[str] = None, verbose: bool = True):
    """Blocking: returns the scheduler's progress list on rank 0, None elsewhere."""
    H = host()
    ctx = start_node(rank, flags, hub)
    try:
        if ctx.is_scheduler:
            boot = H.Customer(ctx.po, "default", None, False)
            text = app_text if app_text is not None else open(flags.app).read()
            conf = parse(text, cfg.AppConfig)
            lm = conf.linear_method
            files = H.search_files(cfg.data_files(lm.training_data, H))
            if lm.training_data.file and not files:
                raise FileNotFoundError(f"no training file matches {list(lm.training_data.file)}")
            parts = H.divide_files(files, max(flags.num_workers, 1), int(flags.load_limit))
            vparts = None
            if lm.has("validation_data") and lm.validation_data.file:       # linear_method.cc:154-172
                vfiles = H.search_files(cfg.data_files(lm.validation_data, H))
                vparts = H.divide_files(vfiles, max(flags.num_workers, 1), int(flags.load_limit))
            workers = boot.group(H.kWorkerGroup)
            for nid in boot.group(H.kActiveGroup):
                c = conf.copy()
                if nid in workers:
                    c.linear_method.mutable("training_data").file = list(parts[workers.index(nid)])
                    if vparts is not None:
                        c.linear_method.mutable("validation_data").file = list(vparts[workers.index(nid)])
                t = boot.submit(nid, payload=dumps(c).encode())
                boot.wait_out(nid, t)
            app = make_app(ctx, conf, flags)
            stop_monitor = threading.Event()
            if float(flags.report_interval) > 0:
                # the scheduler's monitor thread: the heartbeat table every report interval (postoffice.cc:271-290)
                import sys

                from ..runtime.node import dashboard

                def monitor():
                    while not stop_monitor.wait(float(flags.report_interval)):
                        print(dashboard(ctx.po), file=sys.stderr, flush=True)

                threading.Thread(target=monitor, name="H-monitor", daemon=True).start()
            try:
                return app.run(verbose=verbose)
            finally:
                stop_monitor.set()
                ctx.po.stop_all()
                app.stop()
                boot.stop()
        else:
            holder = {}

            def on_conf(msg):
                if msg.request and msg.payload:
                    holder["app"] = make_app(ctx, parse(msg.payload.decode(), cfg.AppConfig), flags)

            boot = H.Customer(ctx.po, "default", on_conf, False)
            ctx.po.wait_terminate(1e9)
            if "app" in holder:
                holder["app"].stop()
            boot.stop()
            return None
    finally:
        ctx.stop()


def run_local_threads(flags: cfg.Flags, app_text: str, verbose: bool = False):
    """All roles as threads of this process over the in-process van (tests, notebooks)."""
    H = host()
    hub = H.InprocHub()
    n = 1 + flags.num_workers + flags.num_servers
    out, errs = {}, []

    def target(r):
        try:
            out[r] = run_node(r, flags, hub, app_text, verbose)
        except Exception as e:  # noqa: BLE001
            import traceback

            errs.append((r, traceback.format_exc()))

    threads = [threading.Thread(target=target, args=(r,), daemon=True) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(600)
    if errs:
        raise RuntimeError(f"rank {errs[0][0]} failed:\n{errs[0][1]}")
    return out[0]
