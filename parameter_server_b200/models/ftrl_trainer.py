"""Streaming driver for online FTRL: host-resident minibatches → device steps → per-step loss.

This is the user-facing loop of the FTRL app (the reference's reader thread + bounded
``data_buf_`` + minibatch loop, src/linear_method/ftrl.cc:74-151).  Minibatches live in pinned
host memory; each is uploaded with ``cudaMemcpyAsync`` on a side stream into one of two device
staging buffers while the previous step computes, and each step's loss sum is read back to the
host (device→host copy into pinned memory) one step behind the compute stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Iterator, List, Optional

import torch

from .ftrl import DeviceMinibatch, FTRLEngine


@dataclass
class HostMinibatch:
    """CSR minibatch in (preferably pinned) host memory.  Keys are uint64 bit patterns in int64, or 32-bit
    feature ids in int32 with ``key_mode`` KEY_U32 / KEY_U32_HASHED (see ``DeviceMinibatch``); offsets are
    int64 or int32.  The compact forms halve the bytes that cross the host link."""
    offsets: torch.Tensor
    keys: torch.Tensor
    y: torch.Tensor
    vals: Optional[torch.Tensor] = None
    key_mode: int = 0

    def pin(self) -> "HostMinibatch":
        f = lambda t: None if t is None else (t if t.is_pinned() else t.pin_memory())
        return HostMinibatch(f(self.offsets), f(self.keys), f(self.y), f(self.vals), self.key_mode)

    def nbytes(self) -> int:
        n = (self.offsets.numel() * self.offsets.element_size() + self.keys.numel() * self.keys.element_size()
             + self.y.numel() * 4)
        return n + (self.vals.numel() * 4 if self.vals is not None else 0)


class _Staging:
    def __init__(self, eng: FTRLEngine, with_vals: bool):
        d = eng.dev
        self.max_nnz, self.dev = eng.max_nnz, d
        self.offsets = torch.empty((eng.max_rows + 1,), dtype=torch.int64, device=d)
        self.keys = torch.empty((eng.max_nnz,), dtype=torch.int64, device=d)
        self.y = torch.empty((eng.max_rows,), dtype=torch.float32, device=d)
        # feature values: allocated up front on request, else when the first valued minibatch arrives
        self.vals = torch.empty((eng.max_nnz,), dtype=torch.float32, device=d) if with_vals else None
        self.ready = torch.cuda.Event()
        self.free = torch.cuda.Event()

    def upload(self, hb: HostMinibatch) -> DeviceMinibatch:
        r, n = hb.y.numel(), hb.keys.numel()
        # the staging buffers are sized for 64-bit entries; narrower inputs use a prefix of the same memory
        off = self.offsets.view(hb.offsets.dtype)[: r + 1]
        keys = self.keys.view(hb.keys.dtype)[:n]
        off.copy_(hb.offsets, non_blocking=True)
        keys.copy_(hb.keys, non_blocking=True)
        self.y[:r].copy_(hb.y, non_blocking=True)
        v = None
        if hb.vals is not None:
            if self.vals is None:
                self.vals = torch.empty((self.max_nnz,), dtype=torch.float32, device=self.dev)
            self.vals[:n].copy_(hb.vals, non_blocking=True)
            v = self.vals[:n]
        return DeviceMinibatch(off, keys, self.y[:r], v, hb.key_mode)


class FTRLTrainer:
    """Host→device streaming around :class:`FTRLEngine` through a ring of ``depth`` staging buffers."""

    def __init__(self, engine: FTRLEngine, with_vals: bool = False, depth: int = 3):
        self.eng = engine
        self.copy_stream = torch.cuda.Stream(device=engine.dev)
        self.stages = [_Staging(engine, with_vals) for _ in range(depth)]
        self.loss_host = torch.zeros((depth, 8), dtype=torch.float64).pin_memory()
        self.loss_events = [torch.cuda.Event() for _ in range(depth)]
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def train(self, batches: Iterable[HostMinibatch], after_step=None, on_loss=None) -> List[float]:
        """Run one step per minibatch; returns the mean logistic loss of every step.

        ``batches`` may be a generator: the next minibatch is fetched and uploaded while the current step
        computes.  ``after_step(i)`` runs on the host right after step ``i`` (0-based) was enqueued — a
        caller that needs the model as of that step (a checkpoint) synchronises there.  ``on_loss(i, loss)``
        runs when step ``i``'s loss has arrived on the host, ``depth`` steps behind the launches."""
        eng, depth = self.eng, len(self.stages)
        compute = torch.cuda.current_stream(eng.dev)
        it: Iterator[HostMinibatch] = iter(batches)
        losses: List[float] = []
        pending: List[int] = []

        def upload(i: int, hb: HostMinibatch) -> DeviceMinibatch:
            st = self.stages[i % depth]
            with torch.cuda.stream(self.copy_stream):
                self.copy_stream.wait_event(st.free)   # the step that last used this buffer is done
                mb = st.upload(hb)
                st.ready.record(self.copy_stream)
            self.h2d_bytes += hb.nbytes()
            return mb

        def collect(j: int) -> None:
            self.loss_events[j % depth].synchronize()
            st = self.loss_host[j % depth].tolist()
            losses.append(st[0] / max(st[1], 1.0))
            eng.maybe_grow(st[6])      # the shard table doubles before it fills up (entries as of step j)
            if on_loss is not None:
                on_loss(j, losses[-1])

        nxt = next(it, None)
        i = 0
        cur = upload(0, nxt) if nxt is not None else None
        while cur is not None:
            nxt = next(it, None)
            nxt_dev = upload(i + 1, nxt) if nxt is not None else None
            st = self.stages[i % depth]
            compute.wait_event(st.ready)
            if len(pending) >= depth:
                collect(pending.pop(0))
            eng.stats[0:2].zero_()
            eng.step(cur)
            st.free.record(compute)
            self.loss_host[i % depth].copy_(eng.stats, non_blocking=True)   # loss sum, rows, ..., table entries
            self.loss_events[i % depth].record(compute)
            self.d2h_bytes += 64
            pending.append(i)
            if after_step is not None:
                after_step(i)
            cur, i = nxt_dev, i + 1
        for j in pending:
            collect(j)
        eng.check_status()
        return losses
