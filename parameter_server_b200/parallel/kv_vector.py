"""Key-range sharded key→value vector on peer memory (``KVVector`` + ``SharedParameter`` push/pull).

Reference: src/parameter/kv_vector.h (per-channel sorted keys + aligned values; pushes from several
workers are summed on the server, pulls look values up by key) and
src/parameter/shared_parameter.h:14-26.  Here a shard's keys and values live in symmetric buffers;
``resolve`` turns a worker's key list into ``(owner, slot)`` once, ``pull`` / ``push`` are single
kernels that read / reduce into the owners' memory over NVLink.  ``impl="nccl"`` exchanges the
same rows with ``all_to_all_single`` and is the comparison baseline.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from ..ops import _native as N
from ..ops import sparse
from ..utils.range import Range
from .peer import PeerGroup

_P8 = C.c_void_p * N.MAX_RANKS


class KvPeers(C.Structure):
    _fields_ = [("keys", _P8), ("vals", _P8), ("nkeys", C.c_int64 * N.MAX_RANKS), ("seps", N.KeySeps), ("k", C.c_int), ("pad", C.c_int)]


class DeviceKVVector:
    def __init__(self, group: PeerGroup, k: int = 1, key_range: Optional[Range] = None, impl: str = "fused"):
        self.group, self.k, self.impl = group, int(k), impl
        self.dev = group.device
        self.key_range = key_range or Range.all()
        self.seps = self.key_range.separators(group.world)
        self._lib = N.lib()

    # ------------------------------------------------------------------ server side
    def set_keys(self, keys: torch.Tensor, capacity: Optional[int] = None) -> None:
        """Install this shard's sorted unique keys (all inside its key range) and zero values.  Collective."""
        g, W = self.group, self.group.world
        n = keys.numel()
        sizes = [n]
        if W > 1:
            import torch.distributed as dist

            sizes = [None] * W
            dist.all_gather_object(sizes, n, group=g.group)
        cap = max(capacity or 0, max(sizes), 1)
        self.nkeys = sizes
        self.keys = g.alloc((cap,), torch.int64, fill=-1)
        self.vals = g.alloc((cap, self.k), torch.float32, fill=0)
        self.keys.local[:n] = keys
        P = KvPeers()
        for r in range(W):
            P.keys[r], P.vals[r], P.nkeys[r] = self.keys.ptrs[r], self.vals.ptrs[r], sizes[r]
        for i, s in enumerate(self.seps):
            P.seps.sep[i] = s
        for i in range(len(self.seps), N.MAX_RANKS + 1):
            P.seps.sep[i] = N.EMPTY_KEY
        P.seps.world = W
        P.k = self.k
        self._P = P
        g.barrier()

    def merge_keys(self, worker_keys: torch.Tensor) -> torch.Tensor:
        """Union of every rank's keys restricted to this shard's range (key-only push); returns them sorted."""
        g = self.group
        parts = [worker_keys]
        if g.world > 1:
            import torch.distributed as dist

            sizes = [None] * g.world
            dist.all_gather_object(sizes, worker_keys.numel(), group=g.group)
            pad = torch.full((max(sizes),), -1, dtype=torch.int64, device=self.dev)
            pad[: worker_keys.numel()] = worker_keys
            bufs = [torch.empty_like(pad) for _ in range(g.world)]
            dist.all_gather(bufs, pad, group=g.group)
            parts = [b[:n] for b, n in zip(bufs, sizes)]
        allk, _ = sparse.count_unique(torch.cat(parts))
        start, pk, _ = sparse.partition_by_key_range(allk, None, self.seps)
        s = start.tolist()
        mine, _ = sparse.sort_pairs(pk[s[g.rank]: s[g.rank + 1]].contiguous())
        return mine

    @property
    def local_keys(self) -> torch.Tensor:
        return self.keys.local[: self.nkeys[self.group.rank]]

    @property
    def local_values(self) -> torch.Tensor:
        return self.vals.local[: self.nkeys[self.group.rank]]

    # ------------------------------------------------------------------ worker side
    def resolve(self, keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(owner int32, slot int32) of every key; slot is -1 for keys no shard holds."""
        n = keys.numel()
        owner = torch.empty(n, dtype=torch.int32, device=self.dev)
        slot = torch.empty(n, dtype=torch.int32, device=self.dev)
        N.check(self._lib.psb_kv_resolve(C.byref(self._P), N.ptr(keys), C.c_size_t(n), N.ptr(owner), N.ptr(slot), N.stream_ptr()), "kv_resolve")
        if self.impl == "nccl":
            self._plan(owner, slot)
        return owner, slot

    def pull(self, owner: torch.Tensor, slot: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = owner.numel()
        if out is None:
            out = torch.empty((n, self.k), dtype=torch.float32, device=self.dev)
        if self.impl == "nccl":
            return self._pull_nccl(out)
        N.check(self._lib.psb_kv_pull(C.byref(self._P), N.ptr(owner), N.ptr(slot), C.c_size_t(n), N.ptr(out), N.stream_ptr()), "kv_pull")
        return out

    def push(self, owner: torch.Tensor, slot: torch.Tensor, vals: torch.Tensor) -> None:
        """Add ``vals[i]`` to the owner's row of key i (sums over all pushing ranks)."""
        if self.impl == "nccl":
            return self._push_nccl(vals)
        N.check(self._lib.psb_kv_push(C.byref(self._P), N.ptr(owner), N.ptr(slot), C.c_size_t(owner.numel()), N.ptr(vals.contiguous()),
                                      N.stream_ptr()), "kv_push")

    # ------------------------------------------------------------------ NCCL-only baseline
    def _plan(self, owner: torch.Tensor, slot: torch.Tensor) -> None:
        import torch.distributed as dist

        W = self.group.world
        _, dest = sparse.bucket_order(owner, W)
        self._perm = torch.empty_like(dest)
        self._perm[dest] = torch.arange(dest.numel(), device=self.dev)       # position → original index, grouped by owner
        counts = torch.bincount(owner.long(), minlength=W)
        self._out_counts = counts.tolist()
        cin = torch.empty_like(counts)
        if W > 1:
            dist.all_to_all_single(cin, counts, group=self.group.group)
        else:
            cin = counts
        self._in_counts = cin.tolist()
        send_slots = slot[self._perm].contiguous()
        self._recv_slots = torch.empty(sum(self._in_counts), dtype=torch.int32, device=self.dev)
        if W > 1:
            dist.all_to_all_single(self._recv_slots, send_slots, self._in_counts, self._out_counts, group=self.group.group)
        else:
            self._recv_slots = send_slots

    def _pull_nccl(self, out: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        nr = self._recv_slots.numel()
        rows = torch.empty((nr, self.k), dtype=torch.float32, device=self.dev)
        N.check(self._lib.psb_rows_gather(N.ptr(self.vals.local), N.ptr(self._recv_slots), C.c_size_t(nr), self.k, N.ptr(rows), N.stream_ptr()), "rows_gather")
        got = torch.empty((self._perm.numel(), self.k), dtype=torch.float32, device=self.dev)
        if self.group.world > 1:
            dist.all_to_all_single(got, rows, [c for c in self._out_counts], [c for c in self._in_counts], group=self.group.group)
        else:
            got = rows
        out[self._perm] = got
        return out

    def _push_nccl(self, vals: torch.Tensor) -> None:
        import torch.distributed as dist

        send = vals[self._perm].contiguous()
        nr = self._recv_slots.numel()
        rows = torch.empty((nr, self.k), dtype=torch.float32, device=self.dev)
        if self.group.world > 1:
            dist.all_to_all_single(rows, send, self._in_counts, self._out_counts, group=self.group.group)
        else:
            rows = send
        N.check(self._lib.psb_rows_scatter_add(N.ptr(self.vals.local), N.ptr(self._recv_slots), C.c_size_t(nr), self.k, N.ptr(rows), N.stream_ptr()),
                "rows_scatter_add")
