"""Tracing and metrics.

The reference has no tracer: it offers a per-message van log (``-print_van``), ``-verbose`` narration
and per-iteration busy/total times in ``Progress`` (src/system/van.cc:170-172,
src/linear_method/darling.cc:206-210).  Here:

* :class:`ChromeTrace` records spans (host wall clock, optionally bracketed by CUDA events for device
  time) and writes a Chrome / Perfetto ``traceEvents`` JSON file (``-trace_file``);
* :func:`nvtx_range` opens an NVTX range around a phase so that profilers show load / preprocess /
  block pass / push / pull phases by name;
* :class:`MetricsLog` appends one JSON object per line (``-metrics_file``): examples/s, objective,
  kernel phase times, bytes moved.
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from typing import Optional


class ChromeTrace:
    def __init__(self, path: Optional[str] = None, pid: int = 0):
        self.path, self.pid = path, pid
        self.events = []
        self._lock = threading.Lock()
        self._cuda = []

    def enabled(self) -> bool:
        return bool(self.path)

    @contextlib.contextmanager
    def span(self, name: str, cat: str = "host", device_timed: bool = False, **args):
        """Record ``name`` from entry to exit; with ``device_timed`` the span also carries the GPU time between two
        CUDA events recorded on the current stream (resolved when the trace is saved)."""
        if not self.enabled():
            yield
            return
        ev = None
        if device_timed:
            import torch

            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        t0 = time.perf_counter_ns()
        try:
            yield
        finally:
            t1 = time.perf_counter_ns()
            if ev is not None:
                ev[1].record()
            rec = {"name": name, "cat": cat, "ph": "X", "pid": self.pid, "tid": threading.get_ident() % 100000,
                   "ts": t0 / 1e3, "dur": (t1 - t0) / 1e3, "args": dict(args)}
            with self._lock:
                self.events.append(rec)
                if ev is not None:
                    self._cuda.append((rec, ev))

    def instant(self, name: str, **args) -> None:
        if self.enabled():
            with self._lock:
                self.events.append({"name": name, "ph": "i", "s": "p", "pid": self.pid, "tid": 0,
                                    "ts": time.perf_counter_ns() / 1e3, "args": dict(args)})

    def save(self) -> Optional[str]:
        if not self.enabled():
            return None
        for rec, (e0, e1) in self._cuda:
            try:
                e1.synchronize()
                rec["args"]["device_ms"] = e0.elapsed_time(e1)
            except Exception:
                pass
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        with open(self.path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
        return self.path


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch

        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
            try:
                yield
            finally:
                torch.cuda.nvtx.range_pop()
            return
    except Exception:
        pass
    yield


class MetricsLog:
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self._lock = threading.Lock()

    def log(self, **fields) -> None:
        if not self.path:
            return
        fields.setdefault("time", time.time())
        with self._lock, open(self.path, "a") as f:
            f.write(json.dumps(fields) + "\n")
