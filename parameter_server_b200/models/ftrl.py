"""Online FTRL-proximal logistic regression on key-range sharded device tables.

Role map to the reference: :class:`FTRLEngine` is worker + server of one rank —
``FTRL::updateModel`` (src/linear_method/ftrl.cc:61-152) on the worker side and
``FTRLModel`` (src/linear_method/ftrl_model.h) on the server side.  A step is
two cooperative kernels (see ``csrc/ftrl_kernels.cu``):

* pull-fused SpMV  — dedup keys into a table laid out by owner; every owner reads its region
  of every worker's table over NVLink, looks the keys up in its shard and stores the weights
  into the worker's weight array; ``Xw``, logistic loss, per-row coefficient;
* push-fused update — ``Xᵀ·coef`` + pos/neg counts per unique key into the worker's
  accumulators; every owner reads its region of them over NVLink and applies the FTRL update
  to the shard slots it resolved during the pull.

``impl="nccl"`` runs the same arithmetic with stand-alone kernels and
``all_to_all_single`` exchanges; it is the comparison baseline, not the product.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import _native as N
from ..parallel.peer import PeerGroup, SymmetricBuffer
from ..utils.range import Range

KEY_U64, KEY_U32, KEY_U32_HASHED = 0, 1, 2


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
    """CSR minibatch resident on the device.

    ``keys``: uint64 bit patterns in int64 (``key_mode`` KEY_U64), or 32-bit feature ids in int32 that the
    kernels widen on the fly: KEY_U32 uses the id itself as the key, KEY_U32_HASHED the 64-bit mix of the id
    (``data.synthetic.mix64``) — half the bytes per non-zero for jobs whose feature space fits 32 bits.
    ``offsets``: int64 or int32."""
    offsets: torch.Tensor            # [rows+1]
    keys: torch.Tensor               # [nnz]
    y: torch.Tensor                  # float32 [rows], ±1
    vals: Optional[torch.Tensor] = None  # float32 [nnz]; None = binary features
    key_mode: int = KEY_U64

    @property
    def rows(self) -> int:
        return self.y.numel()

    @property
    def nnz(self) -> int:
        return self.keys.numel()

    def nbytes(self) -> int:
        n = (self.offsets.numel() * self.offsets.element_size() + self.keys.numel() * self.keys.element_size()
             + self.y.numel() * 4)
        return n + (self.vals.numel() * 4 if self.vals is not None else 0)


def _pow2_at_least(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


class FTRLEngine:
    """Worker + server shard of one rank for online FTRL (see module docstring)."""

    GROW_AT = 0.75    # share of the shard table's slots that may be taken after a worst-case step

    def __init__(self, group: PeerGroup, hyper: FTRLHyper, *, table_capacity: int, max_rows: int, max_nnz: int,
                 local_capacity: Optional[int] = None, timeout_s: float = 2.0, max_probe: int = 512,
                 key_range: Optional[Range] = None, impl: str = "fused", track_counts: Optional[bool] = None):
        """``table_capacity``: initial slots of this rank's shard table (it grows by doubling, see
        :meth:`maybe_grow`).  ``local_capacity``: slots of the per-minibatch table over all owners; it should
        hold about 1.5 x the unique keys of a minibatch, evenly spread over the owners' key ranges.
        ``track_counts``: keep the per-key pos/neg row counts of FTRL::countKeys
        (src/linear_method/ftrl.cc:154-174).  The count rule needs them; the Σg² rule does not, and
        without them an accumulator is one float instead of four.  Default: on for ``rule="count"``,
        off for ``rule="sumsq"``."""
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
        W = group.world
        # one region of 2^region_log2 slots per owner
        lcap = _pow2_at_least(local_capacity or max_nnz)
        self.region_log2 = max((lcap // _pow2_at_least(W)).bit_length() - 1, 2)    # at least 4 slots: 16-byte rows
        self.lcap = W << self.region_log2
        if self.lcap >= (1 << 32) - 2:
            raise ValueError("local table too large")
        self.max_rows, self.max_nnz, self.max_probe = max_rows, max_nnz, max_probe
        self.epoch = 0          # training steps taken
        self.pull_seq = 0       # pulls launched (steps and predictions): sequence of the ready / replied flags
        self.push_seq = 0       # pushes launched: sequence of the grads flags, parity of the accumulator buffers
        self.key_range = key_range or Range.all()
        self.seps = self.key_range.separators(W)
        i64, f32 = torch.int64, torch.float32
        d = self.dev

        # --- worker side, readable / writable by the owners: per-minibatch table, weights, accumulators, flags
        self.lt_keys = group.alloc((self.lcap,), i64, fill=-1)
        self.lt_w = group.alloc((self.lcap,), f32)
        self.lt_acc = group.alloc((2, self.lcap, 4) if self.track_counts else (2, self.lcap), f32)
        self.ready = group.alloc((N.MAX_RANKS,), i64)
        self.replied = group.alloc((N.MAX_RANKS,), i64)
        self.grads = group.alloc((N.MAX_RANKS,), i64)
        # --- worker side, private
        self.slot_of = torch.empty((max_nnz,), dtype=torch.int32, device=d)
        self.coef = torch.empty((max_rows,), dtype=f32, device=d)
        self.xw = torch.empty((max_rows,), dtype=f32, device=d)
        self.send_cnt = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        self.recv_cnt = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        self.stats = torch.zeros((8,), dtype=torch.float64, device=d)
        self.status = torch.zeros((8,), dtype=torch.int32, device=d)
        self.trace = torch.zeros((16,), dtype=torch.int64, device=d)
        # --- server side, private: shard slot of every request of the current step (and the keys, for the filter)
        self.in_slot = torch.full((self.lcap,), -1, dtype=torch.int32, device=d)
        self.in_keys = torch.full((self.lcap,), -1, dtype=i64, device=d) if hyper.tail_feature_freq > 0 else None

        self._seps = N.KeySeps()
        for i, s in enumerate(self.seps):
            self._seps.sep[i] = s
        for i in range(len(self.seps), N.MAX_RANKS + 1):
            self._seps.sep[i] = N.EMPTY_KEY
        self._seps.world = W

        P = N.FtrlPeers()
        P.seps = self._seps
        P.rank, P.max_probe = group.rank, max_probe
        for r in range(W):
            P.lt_keys[r] = self.lt_keys.ptrs[r]
            P.lt_w[r] = self.lt_w.ptrs[r]
            P.lt_acc[r] = self.lt_acc.ptrs[r]
            P.ready[r] = self.ready.ptrs[r]
            P.replied[r] = self.replied.ptrs[r]
            P.grads[r] = self.grads.ptrs[r]
        P.in_slot = self.in_slot.data_ptr()
        P.in_keys = 0 if self.in_keys is None else self.in_keys.data_ptr()
        P.timeout_ns = int(timeout_s * 1e9)
        P.region_log2 = self.region_log2
        self._P = P
        # --- server side: the shard table, one 32-byte slot per key: [key, (w,z), (pos,neg), reserved] as 4 x int64
        self._set_table(self._empty_table(_pow2_at_least(table_capacity)))

        L = N.LocalScratch()
        L.lt_keys, L.lt_w, L.lt_acc = self.lt_keys.local.data_ptr(), self.lt_w.local.data_ptr(), self.lt_acc.local.data_ptr()
        L.lt_slots = self.lcap
        L.slot_of, L.coef, L.xw = self.slot_of.data_ptr(), self.coef.data_ptr(), self.xw.data_ptr()
        L.send_cnt, L.recv_cnt = self.send_cnt.data_ptr(), self.recv_cnt.data_ptr()
        L.stats, L.status = self.stats.data_ptr(), self.status.data_ptr()
        L.trace = self.trace.data_ptr()
        L.soa = 0 if self.track_counts else 1
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
        self.grown = 0
        if impl == "nccl":
            self._u_keys = torch.empty((self.lcap,), dtype=i64, device=d)
            self._u_slot = torch.empty((self.lcap,), dtype=torch.int32, device=d)
            self._counts = torch.zeros((N.MAX_RANKS,), dtype=torch.int32, device=d)
        self.maybe_grow(0.0)      # a table too small for even one step's keys starts larger
        self.grown = 0
        group.barrier()

    # ------------------------------------------------------------- shard table
    def _empty_table(self, cap: int) -> torch.Tensor:
        t = torch.zeros((cap, 4), dtype=torch.int64, device=self.dev)
        t[:, 0] = -1
        return t

    def _set_table(self, t: torch.Tensor) -> None:
        """Make ``t`` this rank's shard table.  Only the owner ever touches its table, so no other rank has
        to know; the shard slots remembered between the two kernels of a step do not outlive the step."""
        cap = t.shape[0]
        if cap & (cap - 1) or cap >= (1 << 32) - 2:
            raise ValueError("shard table capacity must be a power of two below 2^32")
        self.cap = cap
        self.tab = SymmetricBuffer(t, [t.data_ptr()])
        self._P.tab = t.data_ptr()
        self._P.tab_mask = cap - 1
        self._P.tab_shift = 64 - (cap.bit_length() - 1)

    def maybe_grow(self, table_entries: Optional[float] = None) -> bool:
        """Double the shard table before it can fill up (the reference's model is an ``unordered_map`` that
        grows, src/linear_method/ftrl_model.h:57).  One step creates at most one entry per slot of the
        per-minibatch tables' regions for this owner, so the table grows as soon as that many new keys
        would take it beyond ``GROW_AT`` of its slots.  Call between steps; reads the entry count from the
        device unless the caller has it.  Local to this rank."""
        if table_entries is None:
            table_entries = float(self.stats[6].item())
        worst_step = min(self.lcap, self.max_nnz * self.group.world)
        if table_entries + worst_step <= self.GROW_AT * self.cap:
            return False
        new_cap = self.cap
        while table_entries + worst_step > self.GROW_AT * new_cap:
            new_cap *= 2
        new = self._empty_table(new_cap)
        N.check(self._lib.psb_ftrl_rehash(N.ptr(self.tab.local), C.c_uint64(self.cap - 1), N.ptr(new),
                                          C.c_uint64(new_cap - 1), C.c_uint32(64 - (new_cap.bit_length() - 1)),
                                          self.max_probe, N.ptr(self.status), N.stream_ptr()), "ftrl_rehash")
        self.kernel_launches += 1
        torch.cuda.current_stream(self.dev).synchronize()
        self._set_table(new)
        self.grown += 1
        return True

    def reset_protocol(self) -> None:
        """Bring the flag words and sequence numbers of all ranks back to zero (collective; used after a
        checkpoint was loaded, so that fresh and used engines continue in step)."""
        self.group.barrier()
        for f in (self.ready, self.replied, self.grads):
            f.local.zero_()
        self.pull_seq = self.push_seq = 0
        self.lt_keys.local.fill_(-1)
        self.lt_acc.local.zero_()
        self.group.barrier()

    # ----------------------------------------------------------------- helpers
    def _mb(self, mb: DeviceMinibatch) -> N.Minibatch:
        if mb.rows > self.max_rows or mb.nnz > self.max_nnz:
            raise ValueError(f"minibatch {mb.rows}x{mb.nnz} exceeds engine limits {self.max_rows}x{self.max_nnz}")
        off32 = 1 if mb.offsets.dtype == torch.int32 else 0
        if (mb.keys.dtype == torch.int32) != (mb.key_mode != KEY_U64):
            raise ValueError("32-bit keys need key_mode KEY_U32 or KEY_U32_HASHED (and 64-bit keys KEY_U64)")
        return N.Minibatch(mb.offsets.data_ptr(), mb.keys.data_ptr(),
                           0 if mb.vals is None else mb.vals.data_ptr(), mb.y.data_ptr(), mb.nnz, mb.rows, off32,
                           int(mb.key_mode))

    def check_status(self) -> None:
        """Raise if a kernel recorded an error (bounded wait ran out, table full, ...)."""
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"rank {self.group.rank}: {N.STATUS_NAMES.get(st[0], st[0])} (peer/arg={st[1]}, phase={st[2]})")

    # -------------------------------------------------------------------- step
    def _launch_pull(self, M, insert: bool) -> None:
        self.pull_seq += 1
        N.check(self._lib.psb_ftrl_pull_spmv(C.byref(self._P), C.byref(M), C.byref(self._L), C.c_uint32(self.pull_seq),
                                             C.c_uint32(1 if insert else 0), N.stream_ptr()), "ftrl_pull_spmv")
        self.kernel_launches += 1

    def step(self, mb: DeviceMinibatch) -> None:
        """Enqueue one training step on the current stream (no host synchronisation)."""
        if self.impl == "nccl":
            return self._step_nccl(mb)
        self.epoch += 1
        M = self._mb(mb)
        self._L.parity = (self.push_seq + 1) & 1
        # under the tail filter a key gets its entry only when it passes the filter, in the push
        self._launch_pull(M, insert=self.hyper.tail_feature_freq <= 0)
        self.push_seq += 1
        N.check(self._lib.psb_ftrl_push_update(C.byref(self._P), C.byref(M), C.byref(self._L), C.byref(self._H),
                                               C.c_uint32(self.push_seq), N.stream_ptr()), "ftrl_push_update")
        self.kernel_launches += 1

    def predict(self, mb: DeviceMinibatch) -> torch.Tensor:
        """X·w for a minibatch with the current model (collective: every rank calls it between steps).
        Creates no entries in the model."""
        M, s = self._mb(mb), N.stream_ptr()
        saved = self.stats.clone()
        if self.impl == "nccl":
            self.group.barrier()   # every owner's last apply kernel has finished
            self._pull_nccl(M)
        else:
            self._launch_pull(M, insert=False)
        N.check(self._lib.psb_ftrl_clear_local(C.byref(self._L), s), "clear_local")
        self.kernel_launches += 1
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
        N.check(lib.psb_ftrl_localize(C.byref(self._P), C.byref(M), C.byref(L), s), "localize")
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
        return {"localize": d(0, 1), "lookup_reply": d(1, 2), "spmv_loss": d(2, 3), "kernel_gap": d(3, 4), "grad": d(4, 5),
                "flag_reset": d(5, 6), "apply": d(6, 8), "step": d(0, 8)}

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
