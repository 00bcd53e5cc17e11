"""Online FTRL-proximal logistic regression on key-range sharded device tables.

Role map to the reference: :class:`FTRLEngine` is worker + server of one rank —
``FTRL::updateModel`` (src/linear_method/ftrl.cc:61-152) on the worker side and
``FTRLModel`` (src/linear_method/ftrl_model.h) on the server side.  A step is
two cooperative kernels (see ``csrc/ftrl_kernels.cu``):

* pull-fused SpMV  — dedup keys, gather weights from the owner shards over NVLink,
  ``Xw``, logistic loss, per-row coefficient;
* push-fused update — ``Xᵀ·coef`` + pos/neg counts per unique key, key-range
  routing into the owners' inboxes, owner-side FTRL update on arrival.

``impl="nccl"`` runs the same arithmetic with stand-alone kernels and
``all_to_all_single`` exchanges; it is the comparison baseline, not the product.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import _native as N
from ..parallel.peer import PeerGroup
from ..utils.range import Range


@dataclass
class FTRLHyper:
    alpha: float = 0.1
    beta: float = 1.0
    lambda1: float = 1.0
    lambda2: float = 0.1
    rule: str = "count"  # "count": reference's sqrt(pos*neg/(pos+neg)); "sumsq": Σg²
    # tail-feature filter (LearnerConfig tail_feature_freq, countmin_n, countmin_k): a key is updated only
    # once its count-min estimate of rows seen exceeds tail_feature_freq; 0 = off
    tail_feature_freq: int = 0
    countmin_n: int = 1 << 20   # sketch width summed over all servers (src/linear_method/ftrl.cc:14-16)
    countmin_k: int = 2

    def native(self) -> N.FtrlHyper:
        return N.FtrlHyper(self.alpha, self.beta, self.lambda1, self.lambda2, 0 if self.rule == "count" else 1, 0,
                           None, 0, 0, 0, 0)


@dataclass
class DeviceMinibatch:
    """CSR minibatch resident on the device. ``keys`` holds uint64 bit patterns in int64."""
    offsets: torch.Tensor            # int64 [rows+1]
    keys: torch.Tensor               # int64 [nnz]
    y: torch.Tensor                  # float32 [rows], ±1
    vals: Optional[torch.Tensor] = None  # float32 [nnz]; None = binary features

    @property
    def rows(self) -> int:
        return self.y.numel()

    @property
    def nnz(self) -> int:
        return self.keys.numel()

    def nbytes(self) -> int:
        n = self.offsets.numel() * 8 + self.keys.numel() * 8 + self.y.numel() * 4
        return n + (self.vals.numel() * 4 if self.vals is not None else 0)


def _pow2_at_least(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


class FTRLEngine:
    """Worker + server shard of one rank for online FTRL (see module docstring)."""

    def __init__(self, group: PeerGroup, hyper: FTRLHyper, *, table_capacity: int, max_rows: int, max_nnz: int,
                 local_capacity: Optional[int] = None, timeout_s: float = 2.0, max_probe: int = 512,
                 key_range: Optional[Range] = None, impl: str = "fused", track_counts: Optional[bool] = None):
        """``track_counts``: keep the per-key pos/neg row counts of FTRL::countKeys
        (src/linear_method/ftrl.cc:154-174).  The count rule needs them; the Σg² rule does not, and
        without them the fused kernels use a 4-byte-per-value split layout of the minibatch table and
        12-byte push records.  Default: on for ``rule="count"``, off for ``rule="sumsq"``."""
        if group.world > N.MAX_RANKS:
            raise ValueError(f"at most {N.MAX_RANKS} ranks per box")
        needs_counts = hyper.rule == "count" or hyper.tail_feature_freq > 0
        if track_counts is None:
            track_counts = needs_counts or impl != "fused"
        if needs_counts and not track_counts:
            raise ValueError('rule="count" and the tail-feature filter need track_counts')
        self.track_counts = bool(track_counts) or impl != "fused"
        self.group, self.hyper, self.impl = group, hyper, impl
        self.dev = group.device
        self.cap = _pow2_at_least(table_capacity)
        self.lcap = _pow2_at_least(local_capacity or max_nnz)
        if self.lcap >= (1 << 32) - 1:
            raise ValueError("local table too large")
        self.in_cap = self.lcap
        self.max_rows, self.max_nnz = max_rows, max_nnz
        self.epoch = 0
        self.key_range = key_range or Range.all()
        self.seps = self.key_range.separators(group.world)
        W = group.world
        i64, f32 = torch.int64, torch.float32

        # --- server side: shard table + inbox + flags (peer-addressable)
        # one 32-byte slot per key: [key, (w,z), (pos,neg), reserved] viewed as 4 x int64
        self.tab = group.alloc((self.cap, 4), i64, fill=0)
        self.tab.local[:, 0] = -1
        self.in_keys = group.alloc((W * self.in_cap,), i64, fill=-1)
        self.in_g = group.alloc((W * self.in_cap,), f32)
        self.in_cnt = group.alloc((W * self.in_cap,), i64)
        # the per-minibatch table is cut into chunks of 1024 slots; chunk c of sender s owns the fixed inbox
        # segment [s * in_cap + c * 1024, ...) and reports its fill level in in_chunk[s * nchunks + c]
        self.nchunks = (self.lcap + 1023) // 1024
        self.in_chunk = group.alloc((W * self.nchunks,), torch.int32)
        self.in_flag = group.alloc((N.MAX_RANKS,), i64)
        self.applied = group.alloc((N.MAX_RANKS,), i64)

        # --- worker side: per-minibatch scratch (local only)
        d = self.dev
        self.lt_keys = torch.full((self.lcap,), -1, dtype=i64, device=d)
        self.lt_val = torch.zeros((self.lcap, 4), dtype=f32, device=d)
        self.slot_of = torch.empty((max_nnz,), dtype=torch.int32, device=d)
        self.coef = torch.empty((max_rows,), dtype=f32, device=d)
        self.xw = torch.empty((max_rows,), dtype=f32, device=d)
        self.send_cnt = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        self.recv_cnt = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        self.stats = torch.zeros((8,), dtype=torch.float64, device=d)
        self.status = torch.zeros((8,), dtype=torch.int32, device=d)

        self._seps = N.KeySeps()
        for i, s in enumerate(self.seps):
            self._seps.sep[i] = s
        for i in range(len(self.seps), N.MAX_RANKS + 1):
            self._seps.sep[i] = N.EMPTY_KEY
        self._seps.world = W

        P = N.FtrlPeers()
        P.seps = self._seps
        P.rank, P.max_probe, P.tab_mask = group.rank, max_probe, self.cap - 1
        for r in range(W):
            P.tab[r] = self.tab.ptrs[r]
            P.in_keys[r] = self.in_keys.ptrs[r]
            P.in_g[r] = self.in_g.ptrs[r]
            P.in_cnt[r] = self.in_cnt.ptrs[r]
            P.in_flag[r] = self.in_flag.ptrs[r]
            P.in_chunk[r] = self.in_chunk.ptrs[r]
            P.applied[r] = self.applied.ptrs[r]
        P.timeout_ns = int(timeout_s * 1e9)
        P.in_cap = self.in_cap
        P.nchunks = self.nchunks
        P.tab_shift = 64 - (self.cap.bit_length() - 1)
        self._P = P
        L = N.LocalScratch()
        L.lt_keys, L.lt_val, L.lt_mask = self.lt_keys.data_ptr(), self.lt_val.data_ptr(), self.lcap - 1
        L.lt_shift = 64 - (self.lcap.bit_length() - 1)
        L.slot_of, L.coef, L.xw = self.slot_of.data_ptr(), self.coef.data_ptr(), self.xw.data_ptr()
        L.send_cnt, L.recv_cnt = self.send_cnt.data_ptr(), self.recv_cnt.data_ptr()
        L.stats, L.status = self.stats.data_ptr(), self.status.data_ptr()
        self.trace = torch.zeros((16,), dtype=torch.int64, device=d)
        L.trace = self.trace.data_ptr()
        if not self.track_counts:
            self.lt_w = torch.zeros((self.lcap,), dtype=f32, device=d)
            self.lt_g = torch.zeros((self.lcap,), dtype=f32, device=d)
            L.lt_w, L.lt_g, L.soa = self.lt_w.data_ptr(), self.lt_g.data_ptr(), 1
        self._L = L
        self._H = hyper.native()
        if hyper.tail_feature_freq > 0:
            # this server's share of the sketch (FTRL::init sizes it countmin_n / num_servers)
            self.cm_width = max(int(hyper.countmin_n) // W, 64)
            self.cm = torch.zeros((self.cm_width,), dtype=torch.int32, device=d)
            self._H.cm, self._H.cm_width = self.cm.data_ptr(), self.cm_width
            self._H.cm_k, self._H.tail_freq = max(int(hyper.countmin_k), 1), int(hyper.tail_feature_freq)
        self._lib = N.lib()
        self.kernel_launches = 0
        if impl == "nccl":
            self._u_keys = torch.empty((self.lcap,), dtype=i64, device=d)
            self._u_slot = torch.empty((self.lcap,), dtype=torch.int32, device=d)
            self._counts = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        group.barrier()

    # ----------------------------------------------------------------- helpers
    def _mb(self, mb: DeviceMinibatch) -> N.Minibatch:
        if mb.rows > self.max_rows or mb.nnz > self.max_nnz:
            raise ValueError(f"minibatch {mb.rows}x{mb.nnz} exceeds engine limits {self.max_rows}x{self.max_nnz}")
        return N.Minibatch(mb.offsets.data_ptr(), mb.keys.data_ptr(),
                           0 if mb.vals is None else mb.vals.data_ptr(), mb.y.data_ptr(), mb.nnz, mb.rows, 0)

    def check_status(self) -> None:
        """Raise if a kernel recorded an error (bounded wait ran out, table full, ...)."""
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"rank {self.group.rank}: {N.STATUS_NAMES.get(st[0], st[0])} (peer/arg={st[1]}, phase={st[2]})")

    # -------------------------------------------------------------------- step
    def step(self, mb: DeviceMinibatch) -> None:
        """Enqueue one training step on the current stream (no host synchronisation)."""
        if self.impl == "nccl":
            return self._step_nccl(mb)
        self.epoch += 1
        M, s = self._mb(mb), N.stream_ptr()
        N.check(self._lib.psb_ftrl_pull_spmv(C.byref(self._P), C.byref(M), C.byref(self._L), C.c_uint32(self.epoch), s),
                "ftrl_pull_spmv")
        N.check(self._lib.psb_ftrl_push_update(C.byref(self._P), C.byref(M), C.byref(self._L), C.byref(self._H),
                                               C.c_uint32(self.epoch), s), "ftrl_push_update")
        self.kernel_launches += 2

    def predict(self, mb: DeviceMinibatch) -> torch.Tensor:
        """X·w for a minibatch with the current model (collective: every rank calls it between steps).

        The pull runs with the next step's epoch without consuming it, so it waits for exactly the
        updates of the last completed step and leaves the epoch protocol untouched.
        """
        M, s = self._mb(mb), N.stream_ptr()
        saved = self.stats.clone()
        if self.impl == "nccl":
            self.group.barrier()   # every owner's last apply kernel has finished
            self._pull_nccl(M)
        else:
            N.check(self._lib.psb_ftrl_pull_spmv(C.byref(self._P), C.byref(M), C.byref(self._L),
                                                 C.c_uint32(self.epoch + 1), s), "ftrl_pull_spmv")
        N.check(self._lib.psb_ftrl_clear_local(C.byref(self._L), s), "clear_local")
        self.kernel_launches += 2
        out = self.xw[: mb.rows].clone()
        self.stats.copy_(saved)
        return out

    # ------------------------------------------------------- NCCL-only baseline
    def _step_nccl(self, mb: DeviceMinibatch) -> None:
        self.epoch += 1
        M = self._mb(mb)
        ctx = self._pull_nccl(M)
        self._push_nccl(M, *ctx)

    def _pull_nccl(self, M):
        """Unfused pull: localize, pack unique keys by owner, all_to_all keys, lookup, all_to_all weights, SpMV."""
        import torch.distributed as dist

        lib, L, s = self._lib, self._L, N.stream_ptr()
        W = self.group.world
        N.check(lib.psb_ftrl_localize(C.byref(M), C.byref(L), self._P.max_probe, s), "localize")
        self._counts.zero_()
        N.check(lib.psb_ftrl_count_owner(C.byref(self._seps), C.byref(L), N.ptr(self._counts), s), "count_owner")
        counts = self._counts[:W].tolist()
        total = sum(counts)
        bases = [0] * N.MAX_RANKS
        for i in range(1, W):
            bases[i] = bases[i - 1] + counts[i - 1]
        cursors = torch.tensor(bases, dtype=torch.int32, device=self.dev)
        N.check(lib.psb_ftrl_pack_keys(C.byref(self._seps), C.byref(L), N.ptr(cursors), N.ptr(self._u_keys),
                                       N.ptr(self._u_slot), s), "pack_keys")
        self.kernel_launches += 3
        ukeys = self._u_keys[:total]
        if W > 1:
            cnt_out = torch.tensor(counts, dtype=torch.int64, device=self.dev)
            cnt_in = torch.empty_like(cnt_out)
            dist.all_to_all_single(cnt_in, cnt_out, group=self.group.group)
            in_counts = cnt_in.tolist()
            rkeys = torch.empty((sum(in_counts),), dtype=torch.int64, device=self.dev)
            dist.all_to_all_single(rkeys, ukeys, in_counts, counts, group=self.group.group)
        else:
            in_counts, rkeys = counts, ukeys
        nr = rkeys.numel()
        rw = torch.empty((nr,), dtype=torch.float32, device=self.dev)
        if nr:
            N.check(lib.psb_ftrl_lookup(N.ptr(self.tab.local), C.c_uint64(self.cap - 1),
                                        C.c_uint32(self._P.tab_shift), self._P.max_probe, N.ptr(rkeys), C.c_uint32(nr), N.ptr(rw), s), "lookup")
            self.kernel_launches += 1
        if W > 1:
            uw = torch.empty((total,), dtype=torch.float32, device=self.dev)
            dist.all_to_all_single(uw, rw, counts, in_counts, group=self.group.group)
        else:
            uw = rw
        if total:
            N.check(lib.psb_ftrl_scatter_w(N.ptr(self._u_slot), N.ptr(uw), C.c_uint32(total), C.byref(L), s), "scatter_w")
        N.check(lib.psb_ftrl_spmv_loss(C.byref(M), C.byref(L), s), "spmv_loss")
        self.kernel_launches += 2
        return counts, in_counts, rkeys

    def _push_nccl(self, M, counts, in_counts, rkeys) -> None:
        """Unfused push: gradient, pack by owner, all_to_all (g, counts), owner update sender by sender."""
        import torch.distributed as dist

        lib, L, s = self._lib, self._L, N.stream_ptr()
        W, total, nr = self.group.world, sum(counts), rkeys.numel()
        N.check(lib.psb_ftrl_grad(C.byref(M), C.byref(L), s), "grad")
        ug = torch.empty((total,), dtype=torch.float32, device=self.dev)
        uc = torch.empty((total,), dtype=torch.int64, device=self.dev)
        if total:
            N.check(lib.psb_ftrl_pack_push(N.ptr(self._u_slot), C.c_uint32(total), C.byref(L), N.ptr(ug), N.ptr(uc), s),
                    "pack_push")
        self.kernel_launches += 2
        if W > 1:
            rg = torch.empty((nr,), dtype=torch.float32, device=self.dev)
            rc = torch.empty((nr,), dtype=torch.int64, device=self.dev)
            dist.all_to_all_single(rg, ug, in_counts, counts, group=self.group.group)
            dist.all_to_all_single(rc, uc, in_counts, counts, group=self.group.group)
        else:
            rg, rc = ug, uc
        off = 0
        for n in in_counts:
            if n:
                N.check(lib.psb_ftrl_apply(N.ptr(self.tab.local),
                                           C.c_uint64(self.cap - 1), C.c_uint32(self._P.tab_shift), self._P.max_probe,
                                           N.ptr(rkeys[off:off + n]),
                                           N.ptr(rg[off:off + n]), N.ptr(rc[off:off + n]), C.c_uint32(n),
                                           C.byref(self._H), N.ptr(self.stats), N.ptr(self.status), s), "apply")
                self.kernel_launches += 1
            off += n

    # ------------------------------------------------------------------- stats
    def read_stats(self, reset: bool = True) -> dict:
        """Device→host read of the running statistics (synchronises the stream)."""
        v = self.stats.tolist()
        if reset:
            self.stats[0:2].zero_()
            self.stats[5].zero_()
        return {"loss_sum": v[0], "rows": v[1], "norm1": v[2], "norm2_sq": v[3], "nnz_w": v[4],
                "unique_keys": v[5], "table_entries": v[6]}

    def phase_times_us(self) -> dict:
        """Durations (µs) of the phases of the last fused step, from in-kernel globaltimer marks."""
        t = self.trace.tolist()
        d = lambda a, b: (t[b] - t[a]) / 1e3
        return {"localize": d(0, 1), "gather": d(1, 2), "spmv_loss": d(2, 3), "kernel_gap": d(3, 4), "grad": d(4, 5),
                "route_send": d(5, 6), "wait_senders": d(6, 7), "apply": d(7, 8), "step": d(0, 8)}

    def penalty(self, st: dict) -> float:
        """λ₁‖w‖₁ + ½λ₂·sqrt(‖w‖₂²) exactly as FTRLModel::objv (src/linear_method/ftrl_model.h:31)."""
        return st["norm1"] * self.hyper.lambda1 + 0.5 * self.hyper.lambda2 * max(st["norm2_sq"], 0.0) ** 0.5

    # -------------------------------------------------------------- model dump
    def dump_model(self):
        """(keys uint64 as int64 bit patterns, w) of this shard's non-zero weights, key-ascending."""
        out_k = torch.empty((self.cap,), dtype=torch.int64, device=self.dev)
        out_w = torch.empty((self.cap,), dtype=torch.float32, device=self.dev)
        cnt = torch.zeros((1,), dtype=torch.int64, device=self.dev)
        N.check(self._lib.psb_ftrl_dump_nonzero(N.ptr(self.tab.local),
                                                C.c_uint64(self.cap - 1), N.ptr(out_k), N.ptr(out_w), N.ptr(cnt),
                                                N.stream_ptr()), "dump_nonzero")
        n = int(cnt.item())
        k, w = out_k[:n].cpu().numpy().view("uint64"), out_w[:n].cpu().numpy()
        order = k.argsort(kind="stable")
        return k[order], w[order]

    def save_model(self, file_prefix: str) -> str:
        """Write ``<file>_S<rank>`` with one ``key<TAB>weight`` line per non-zero weight
        (format of FTRLModel::writeToFile, src/linear_method/ftrl_model.h:24-29)."""
        from ..utils.modelio import write_model_text

        k, w = self.dump_model()
        path = f"{file_prefix}_S{self.group.rank}"
        write_model_text(path, k, w)
        return path
