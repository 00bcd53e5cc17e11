"""DARLIN — block-coordinate L1 logistic regression on key-range sharded GPUs.

Roles (reference → here): ``BatchSolver::run`` / ``Darling::runIteration`` scheduler loop
(src/linear_method/batch_solver.cc:23-127, src/linear_method/darling.cc:18-104) →
:meth:`DarlinSolver.run`; ``BatchSolver::preprocessData`` (unique keys, localisation, column-major
storage, key exchange with the servers; src/linear_method/batch_solver.cc:227-384) →
:meth:`DarlinSolver.preprocess`; the per-block worker/server step ``Darling::updateModel``
(src/linear_method/darling.cc:155-273) → the persistent pass kernel in ``csrc/darlin_kernels.cu``.

Every rank is worker r and server r.  After preprocessing the key set is fixed, so each local
column carries its resolved ``(owner, slot)`` and pushes/pulls move values only — the steady state
of the reference's sender/receiver key cache (src/system/remote_node.cc:96-184).
"""
from __future__ import annotations

import ctypes as C
import math
import sys
import time
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from ..ops import _native as N
from ..ops.reduce import reduce_sum
from ..parallel.peer import PeerGroup
from ..utils.range import Range

_SIGN = -(1 << 63)


def _ukey(t: torch.Tensor) -> torch.Tensor:
    """Map uint64 bit patterns (int64) to int64 values whose signed order is the unsigned order."""
    return t ^ _SIGN


@dataclass
class DarlinConfig:
    lambda1: float = 1.0
    eta: float = 1.0
    delta_init: float = 1.0
    delta_max: float = 5.0
    kkt_ratio: float = 10.0
    max_pass: int = 20
    epsilon: float = 1e-4
    feature_block_ratio: float = 4.0
    random_block_order: bool = True
    max_block_delay: int = 0          # tau: tau+1 consecutive blocks form a group whose gradients precede its updates
    seed: int = 0
    reset_nan_on_kkt_reset: bool = True
    # tail-feature filter of BatchSolver::preprocessData (src/linear_method/batch_solver.cc:227-290): features
    # whose count-min estimate of occurrences is <= tail_feature_freq are dropped before training; 0 = off
    tail_feature_freq: int = 0
    countmin_k: int = 2
    countmin_n_ratio: float = 2.0
    # Feature groups (src/linear_method/batch_solver.cc:48-66): with feature_group_bits = b > 0 the top b bits
    # of a key are its group (TERAFEA keys: b = 10); every group is cut into ceil(its non-zeros per row x
    # feature_block_ratio) blocks over its own key range.  0 = all keys form one group.
    feature_group_bits: int = 0
    # blocks of these groups are swept num_iter_for_prior_fea_group times at the start of the first pass, with
    # zero delay (src/linear_method/batch_solver.cc:88-108, src/linear_method/darling.cc:48-50)
    prior_fea_group: tuple = ()
    num_iter_for_prior_fea_group: int = 5


def group_blocks(groups, ratio: float):
    """Feature blocks of the reference's partition rule: ``groups`` = [(id, min_key, max_key_excl, nnz_ele, nnz_ex)],
    result = [(id, begin_key, end_key_excl)] with every group cut into n even key ranges, n = ceil(non-zeros per
    example x ratio) when a group has more than one non-zero per example, else 1; empty ranges are left out."""
    out = []
    for gid, lo, hi, nnz_ele, nnz_ex in groups:
        if hi <= lo or nnz_ex <= 0:
            continue
        per_row = nnz_ele / nnz_ex
        n = max(int(math.ceil(per_row * ratio)), 1) if per_row > 1 + 1e-6 and ratio > 0 else 1
        size = hi - lo
        for i in range(n):
            b, e = lo + size * i // n, lo + size * (i + 1) // n
            if e > b:
                out.append((gid, b, e))
    return out


def prior_block_order(block_groups, prior_groups, n_iter: int, random_order: bool, seed: int) -> List[int]:
    """Order of the extra sweeps over the blocks of the important groups (first pass only)."""
    rng = np.random.RandomState(seed + 1)
    out: List[int] = []
    for g in prior_groups:
        tmp = [k for k, bg in enumerate(block_groups) if bg == int(g)]
        for _ in range(int(n_iter) if tmp else 0):
            if random_order:
                rng.shuffle(tmp)
            out += list(tmp)
    return out


@dataclass
class Progress:
    objv: float
    relative_objv: float
    nnz_w: int
    violation: float
    nnz_active: int
    kkt_threshold: float
    seconds: float = 0.0


def block_order(nblk: int, n_pass: int, random_order: bool, seed: int) -> List[np.ndarray]:
    rng = np.random.RandomState(seed)
    out = []
    for _ in range(n_pass):
        o = np.arange(nblk, dtype=np.int32)
        if random_order:
            rng.shuffle(o)
        out.append(o)
    return out


def margins_from_weights(col_ptr: torch.Tensor, row_idx: torch.Tensor, vals: Optional[torch.Tensor], y: torch.Tensor,
                         w: torch.Tensor) -> torch.Tensor:
    """``y * (X w)`` for a column-major matrix (``col_ptr`` offsets, ``row_idx`` per non-zero, ``vals`` or None = binary)."""
    P = col_ptr.numel() - 1
    cols = torch.repeat_interleave(torch.arange(P, device=col_ptr.device), (col_ptr[1:] - col_ptr[:-1]).long())
    contrib = w.to(torch.float32)[cols]
    if vals is not None:
        contrib = contrib * vals.to(torch.float32)
    xw = torch.zeros(y.numel(), dtype=torch.float32, device=y.device).index_add_(0, row_idx.long(), contrib)
    return y.to(torch.float32) * xw


class DarlinSolver:
    """Worker + server of one rank; ``preprocess`` once, then ``run`` (or ``run_pass`` repeatedly)."""

    def __init__(self, group: PeerGroup, cfg: DarlinConfig, timeout_s: float = 2.0, impl: str = "fused",
                 out_of_core: bool = False, prefetch_depth: int = 3, blocks_per_launch: Optional[int] = None,
                 ctas_per_sm: Optional[int] = None, wide_block_cols: int = 0, gather_small_groups: bool = True,
                 list_block_cols: int = 0):
        """``out_of_core``: keep the column blocks (row ids, values) in pinned host memory and stream each
        block to the GPU on a side stream ahead of its turn in the block order — the role of the
        reference's ``FeatureStation`` in ``-mmap_training_data`` mode with its task-id keyed look-ahead
        prefetch (src/linear_method/feature_station.cc:212-279, src/linear_method/darling.cc:175-201)."""
        self.group, self.cfg, self.impl = group, cfg, impl
        # thread blocks of the pass kernel per SM (1 or 2): more blocks hide gather latency, fewer make the
        # per-group barriers cheaper; 2 measured best with and without bounded delay (5.1 against 5.8 ms per
        # pass on 677,399 x 47,236, one GPU)
        self.ctas_per_sm = ctas_per_sm
        # groups of blocks with more local columns than this fetch the owners' sums once per column instead of
        # once per non-zero, at the price of one more in-GPU barrier (0: the kernel's default, 16384)
        self.wide_block_cols = int(wide_block_cols)
        # groups of blocks with at most 2048 columns over all owners: gather every rank's partial sums on every
        # rank (one cross-GPU wait, no NVLink load in the margin update) instead of pushing into the owners
        self.gather_small_groups = bool(gather_small_groups)
        # several GPUs, groups with more columns over all owners than this: push and pull as bulk transfers over
        # the resolved column lists, two cross-GPU rounds per group (0: the kernel's default, 262144)
        self.list_block_cols = int(list_block_cols)
        self.out_of_core, self.prefetch_depth = out_of_core, max(int(prefetch_depth), 2)
        # out-of-core mode: blocks per kernel launch, rounded up to a multiple of max_block_delay + 1.  A launch
        # costs about 28 us, so small blocks are batched (up to 16); a batch is also the unit that must be on the
        # device before its kernel starts, so it is kept near 24 MB (chosen in _to_host_blocks when not given)
        if cfg.max_block_delay > 127:
            raise ValueError("max_block_delay above 127 is not supported by the pass kernel")
        self._launch_group = max(int(cfg.max_block_delay), 0) + 1
        self._blocks_per_launch_arg = blocks_per_launch
        self.blocks_per_launch = self._round_launch(16 if blocks_per_launch is None else blocks_per_launch)
        self.h2d_bytes = 0
        self.dev = group.device
        self.timeout_s = timeout_s
        self._lib = N.lib()
        self.progress: List[Progress] = []
        self.kkt_threshold = 1e20
        self.seq = 0
        self.bar = 0
        self.kernel_launches = 0

    # ------------------------------------------------------------------ preprocessing
    def _drop_tail_features(self, offsets: torch.Tensor, keys: torch.Tensor, vals: Optional[torch.Tensor]):
        """Tail-feature filter (src/linear_method/batch_solver.cc:250-290, src/parameter/shared_parameter.h:114-133).

        Every worker sends its unique keys with their occurrence counts to the servers (the whole key space
        split evenly); a server adds them to its count-min sketch worker by worker in rank order, then answers
        which keys have an estimate above ``tail_feature_freq``; the worker drops all other columns.  The
        sketch of a server is ``max(W · n · countmin_n_ratio / log(W+1), 64)`` wide, n = keys in the first
        non-empty message it got.  Returns the filtered CSR (offsets, keys, vals).  Collective.
        """
        import torch.distributed as dist

        from ..ops import sparse

        g, dev, W, cfg = self.group, self.dev, self.group.world, self.cfg
        keys = keys.contiguous()
        lkeys, cnt = sparse.count_unique(keys)
        P = lkeys.numel()
        i64 = torch.int64
        if W > 1:
            seps = Range.all().separators(W)
            sep_s = torch.tensor([s + _SIGN for s in seps[1:-1]], dtype=i64, device=dev)
            bounds = [0] + torch.searchsorted(_ukey(lkeys), sep_s).tolist() + [P]
            send = [bounds[i + 1] - bounds[i] for i in range(W)]
            recv_t = torch.empty(W, dtype=i64, device=dev)
            dist.all_to_all_single(recv_t, torch.tensor(send, dtype=i64, device=dev), group=g.group)
            recv = recv_t.tolist()
            rk = torch.empty(sum(recv), dtype=i64, device=dev)
            rc = torch.empty(sum(recv), dtype=torch.int32, device=dev)
            dist.all_to_all_single(rk, lkeys, recv, send, group=g.group)
            dist.all_to_all_single(rc, cnt, recv, send, group=g.group)
        else:
            send = recv = [P]
            rk, rc = lkeys, cnt
        n_first = next((n for n in recv if n > 0), 0)
        width = max(int(W * n_first * cfg.countmin_n_ratio / math.log(W + 1)), 64)
        sketch = sparse.CountMinDevice(width, cfg.countmin_k, dev)
        at = 0
        for n in recv:
            if n:
                sketch.insert(rk[at:at + n], rc[at:at + n])
            at += n
        est = sketch.query(rk) if rk.numel() else torch.zeros(0, dtype=torch.int32, device=dev)
        passed = (est > cfg.tail_feature_freq).to(torch.uint8)
        if W > 1:
            keep = torch.empty(P, dtype=torch.uint8, device=dev)
            dist.all_to_all_single(keep, passed, send, recv, group=g.group)
        else:
            keep = passed
        inv = sparse.remap(keys, lkeys)
        sel = keep[inv.long()].bool()
        rows = offsets.numel() - 1
        row_of = torch.repeat_interleave(torch.arange(rows, device=dev), offsets[1:] - offsets[:-1])
        new_off = torch.zeros(rows + 1, dtype=i64, device=dev)
        new_off[1:] = torch.cumsum(torch.bincount(row_of[sel], minlength=rows), 0)
        self.tail_filter_stats = {"features": P, "dropped": P - int(keep.sum().item()), "sketch_width": width}
        return new_off, keys[sel].contiguous(), None if vals is None else vals[sel].contiguous()

    def _group_info(self, offsets: torch.Tensor, keys: torch.Tensor, lkeys: torch.Tensor):
        """Per feature group (top ``feature_group_bits`` bits of the key): (id, min_key, max_key + 1, non-zeros,
        examples that have the group), summed / merged over all ranks — the slot statistics of the reference's
        ExampleInfo (src/proto/example.proto, merged in src/data/common.cc).  Collective."""
        import torch.distributed as dist

        dev, bits = self.dev, int(self.cfg.feature_group_bits)
        G, shift = 1 << bits, 64 - bits
        gid = (keys >> shift) & (G - 1)
        nnz_ele = torch.bincount(gid, minlength=G).to(torch.float64)
        rows = offsets.numel() - 1
        row_of = torch.repeat_interleave(torch.arange(rows, device=dev), offsets[1:] - offsets[:-1])
        pairs = torch.unique(row_of * G + gid)                    # one entry per (example, group) that occurs
        nnz_ex = torch.bincount(pairs % G, minlength=G).to(torch.float64)
        lg = (lkeys >> shift) & (G - 1)                           # group of every unique local key (ascending keys)
        big = (1 << 63) - 1
        kmin = torch.full((G,), big, dtype=torch.int64, device=dev).scatter_reduce_(0, lg, _ukey(lkeys), "amin")
        kmax = torch.full((G,), -big - 1, dtype=torch.int64, device=dev).scatter_reduce_(0, lg, _ukey(lkeys), "amax")
        if self.group.world > 1:
            cnt = torch.stack([nnz_ele, nnz_ex])
            dist.all_reduce(cnt, group=self.group.group)
            nnz_ele, nnz_ex = cnt[0], cnt[1]
            dist.all_reduce(kmin, op=dist.ReduceOp.MIN, group=self.group.group)
            dist.all_reduce(kmax, op=dist.ReduceOp.MAX, group=self.group.group)
        out = []
        for g in torch.nonzero(nnz_ele > 0).flatten().tolist():
            out.append((g, int(kmin[g].item()) - _SIGN, int(kmax[g].item()) - _SIGN + 1, float(nnz_ele[g].item()),
                        float(nnz_ex[g].item())))
        return out

    def preprocess(self, offsets: torch.Tensor, keys: torch.Tensor, vals: Optional[torch.Tensor], y: torch.Tensor):
        """Localise this rank's CSR rows shard, exchange key sets with the servers, build the CSC blocks.

        ``keys`` are uint64 bit patterns in int64.  Collective over the group.
        """
        import torch.distributed as dist

        g, dev, W = self.group, self.dev, self.group.world
        from ..ops import sparse

        if self.cfg.tail_feature_freq > 0:
            offsets, keys, vals = self._drop_tail_features(offsets, keys, vals)
        rows, nnz = y.numel(), keys.numel()
        # unique local keys in unsigned order + column id of every non-zero  (Localizer::countUniqIndex/remapIndex)
        lkeys, _ = sparse.count_unique(keys.contiguous())          # radix sort + run-length unique (unsigned order)
        uk = _ukey(lkeys)                                          # same keys as int64 values in that order
        P = lkeys.numel()
        inv = sparse.remap(keys.contiguous(), lkeys)               # local column id of every non-zero
        col_ptr, row_idx, cvals = sparse.csr_to_csc(offsets, inv, vals, P)   # CSR → CSC (SparseMatrix::alterStorage)
        # global statistics (ExampleInfo merge): rows, nnz, key range
        stats = g.all_reduce_sum([rows, nnz])
        self.total_rows, self.total_nnz = int(stats[0]), int(stats[1])
        kmin = int(uk.min().item()) if P else (1 << 62)
        kmax = int(uk.max().item()) if P else -(1 << 62)
        if W > 1:
            tmin = torch.tensor([kmin], dtype=torch.int64, device=dev)
            tmax = torch.tensor([kmax], dtype=torch.int64, device=dev)
            dist.all_reduce(tmin, op=dist.ReduceOp.MIN, group=g.group)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX, group=g.group)
            kmin, kmax = int(tmin.item()), int(tmax.item())
        self.key_min, self.key_max = kmin - _SIGN, kmax - _SIGN + 1   # unsigned [min, max+1)
        # servers take the union of the workers' keys in their range (KVVector::setValue key-only push)
        if W > 1:
            sizes = [None] * W
            dist.all_gather_object(sizes, P, group=g.group)
            mx = max(sizes)
            pad = torch.full((mx,), (1 << 63) - 1, dtype=torch.int64, device=dev)
            pad[:P] = uk
            allk = [torch.empty_like(pad) for _ in range(W)]
            dist.all_gather(allk, pad, group=g.group)
            # union of the workers' sorted key sets by ranking (bit patterns: unsigned order)
            gk = _ukey(sparse.set_union_many([_ukey(a[:n]) for a, n in zip(allk, sizes)]))
        else:
            gk = uk
        self.gkeys_sorted = gk                                     # ordered (sign-flipped) global keys
        r = g.rank
        gidx = torch.searchsorted(gk, uk)                          # every local column's position in that list
        # feature blocks (batch_solver.cc:48-66): every feature group is cut into even key sub-ranges of its own
        # key range; without groups all keys form one group over [min_key, max_key)
        groups = self._group_info(offsets, keys, lkeys) if self.cfg.feature_group_bits > 0 else \
            [(1, self.key_min, self.key_max, self.total_nnz, self.total_rows)]
        blocks = group_blocks(groups, self.cfg.feature_block_ratio)
        if not blocks:
            blocks = [(1, self.key_min, self.key_max)]
        nblk = len(blocks)
        self.block_group = [g for g, _, _ in blocks]
        self.block_keys = [(b, e) for _, b, e in blocks]
        to_s = lambda ks: torch.tensor([min(k, (1 << 64) - 1) + _SIGN for k in ks], dtype=torch.int64, device=dev)
        b_lo, b_hi = to_s([b for b, _ in self.block_keys]), to_s([e for _, e in self.block_keys])
        top = torch.tensor([e >= (1 << 64) for _, e in self.block_keys], device=dev)     # a range that ends at 2^64
        lc0, lc1 = torch.searchsorted(uk, b_lo), torch.where(top, P, torch.searchsorted(uk, b_hi))
        gc0, gc1 = torch.searchsorted(gk, b_lo), torch.where(top, gk.numel(), torch.searchsorted(gk, b_hi))
        # Ownership.  The reference gives server i the i-th even cut of the whole key range, so one feature block
        # (a key sub-range itself) lands on one server and the servers take turns.  Here every block's keys are cut
        # into W runs of equal key count, one per server: a server owns one key range per block, all servers work
        # on every block, and a shard's slots follow block order (ascending keys).
        nb = gc1 - gc0
        if nblk > 1 and not bool((gc0[1:] >= gc1[:-1]).all()):
            raise ValueError("feature blocks must be disjoint ascending key ranges")
        ow = torch.arange(W + 1, device=dev)
        own_lo = gc0[:, None] + (nb[:, None] * ow[None, :]) // W    # [nblk, W + 1] cuts in the global key list
        cnt = own_lo[:, 1:] - own_lo[:, :-1]                        # keys of block b on owner o
        base = torch.cumsum(cnt, 0) - cnt                           # ... and the first of their slots
        slots_all = cnt.sum(0)
        self.slots, max_slots = int(slots_all[r].item()), int(slots_all.max().item())
        starts = own_lo[:, :W].reshape(-1).contiguous()

        def owner_slot(pos):
            idx = (torch.searchsorted(starts, pos, right=True) - 1).clamp_(0, nblk * W - 1)
            b_, o_ = idx // W, idx % W
            inside = (pos >= gc0[b_]) & (pos < gc1[b_])             # keys of no block are never touched
            return torch.where(inside, o_, 0), torch.where(inside, base[b_, o_] + pos - own_lo[b_, o_], 0), inside

        owner, gslot, _ = owner_slot(gidx)
        all_o, _, all_in = owner_slot(torch.arange(gk.numel(), device=dev))
        self.skeys = _ukey(gk[(all_o == r) & all_in])              # this shard's keys (bit patterns), in slot order
        sl0 = base[:, r].contiguous()
        sl1 = sl0 + cnt[:, r]
        self.blk_gs0 = own_lo[:, r].contiguous()                   # global position of this shard's first slot per block
        # first local column of every owner's share of every block
        self._cb = torch.searchsorted(gidx.contiguous(), own_lo.reshape(-1).contiguous()).reshape(nblk, W + 1).contiguous()
        self.blk_lc = torch.stack([lc0, lc1], 1).contiguous()
        self.blk_sl = torch.stack([sl0, sl1], 1).contiguous()
        self.blk_gc = torch.stack([gc0, gc1], 1).contiguous()      # every block's range in the global sorted key list
        self.gcol = gidx.contiguous()                               # every local column's position in that list
        self.nblk = nblk
        # ---- worker state
        f32 = torch.float32
        self.rows, self.cols, self.nnz = rows, P, nnz
        self.lkeys = lkeys
        self.col_ptr, self.row_idx, self.vals, self.y = col_ptr, row_idx, cvals, y.contiguous()
        # label and margin of a row share 8 bytes: every non-zero gathers them with one access
        self.ym = torch.stack([y.to(f32), torch.zeros(rows, dtype=f32, device=dev)], 1).contiguous()
        self.margin = self.ym[:, 1]
        # column id of every non-zero (saves a column search per non-zero and phase); not kept in out-of-core
        # mode, where it would add 50 % to the bytes streamed from the host
        self.col_of = None if self.out_of_core else torch.repeat_interleave(
            torch.arange(P, dtype=torch.int32, device=dev), col_ptr[1:] - col_ptr[:-1]).contiguous()
        self.w = torch.zeros(P, dtype=f32, device=dev)
        self.delta = torch.full((P,), self.cfg.delta_init, dtype=f32, device=dev)
        self.active = torch.ones(P, dtype=torch.uint8, device=dev)
        self.gslot = gslot.to(torch.int32).contiguous()
        self.gowner = owner.to(torch.uint8).contiguous()
        self.dw = torch.zeros(P, dtype=f32, device=dev)
        # ---- server state (peer-addressable weights and accumulators)
        cap = max(max_slots, 1)
        self.srv_w = g.alloc((cap,), f32)
        # (G,U) accumulators, three buffers in rotation: a group of blocks sums into one while the previous
        # group's sums are still being read and the one before that is being zeroed
        self.srv_gu = g.alloc((3, cap, 2), f32)
        self._gu_stride = cap
        self._prev_tail = None          # blocks of the group that ran last (their accumulators are zeroed next)
        # small groups of blocks on several GPUs: every rank's partial sums are gathered on every rank instead of
        # pushed into the owners' accumulators (csrc/darlin_kernels.cu, kGatherCols = 2048)
        self.srv_part = g.alloc((3, W, 2048, 2), f32)
        self.part_mine = torch.zeros((2048, 2), dtype=f32, device=dev)
        # very wide groups of blocks on several GPUs: per local column its partial (G,U), its slot in the owner's
        # shard and the owner's answer, addressable by the owners; every rank's owner boundaries per block
        self._all_cb = self.srv_d_slot = None
        if W > 1:
            pmax = torch.tensor([P], dtype=torch.int64, device=dev)
            dist.all_reduce(pmax, op=dist.ReduceOp.MAX, group=g.group)
            pmax = max(int(pmax.item()), 1)
            self.col_gu = g.alloc((pmax, 2), f32)
            self.col_slot = g.alloc((pmax,), torch.int32)
            self.col_slot.local[:P] = self.gslot
            self.col_dw = g.alloc((pmax,), f32)
            self.arrive2 = g.alloc((1,), torch.int64)
            cbs = [torch.empty_like(self._cb) for _ in range(W)]
            dist.all_gather(cbs, self._cb, group=g.group)
            self._all_cb = torch.stack(cbs).contiguous()
            self.srv_d_slot = torch.zeros(cap, dtype=f32, device=dev)
        self.phase_ns = torch.zeros(12, dtype=torch.int64, device=dev)     # in-kernel phase timers (thread block 0)
        self.arrive = g.alloc((1,), torch.int64)
        self.srv_delta = torch.full((cap,), self.cfg.delta_init, dtype=f32, device=dev)
        self.srv_active = torch.ones(cap, dtype=torch.uint8, device=dev)
        self.violation = torch.zeros(1, dtype=torch.int32, device=dev)
        # monotone in-GPU counters: [0] barrier after the margin update, [1]/[2] this GPU's CTAs that finished
        # the gradient / update phase (the CTA completing a count notifies the other ranks)
        self.local_bar = torch.zeros(8, dtype=torch.int64, device=dev)
        self.abort = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)
        if self.out_of_core:
            self._to_host_blocks()
        self._build_structs()
        g.barrier()

    def _to_host_blocks(self) -> None:
        """Move the CSC payload to pinned host memory; only a small ring of block buffers stays on the device."""
        has_vals = self.vals is not None
        words = 2 if has_vals else 1
        cp = self.col_ptr[self.blk_lc.reshape(-1)].reshape(-1, 2).cpu()
        self.blk_nnz = np.ascontiguousarray(cp.numpy().astype(np.int64))   # [p0, p1) of every block in the CSC arrays
        # pinned host copy, packed per block as [row ids | values]: one copy per block brings both
        rows_h = self.row_idx.cpu()
        vals_h = self.vals.cpu().view(torch.int32) if has_vals else None
        self.h_pack = torch.empty(max(rows_h.numel() * words, 1), dtype=torch.int32).pin_memory()
        for p0, p1 in self.blk_nnz.tolist():
            n = p1 - p0
            self.h_pack[words * p0: words * p0 + n] = rows_h[p0:p1]
            if has_vals:
                self.h_pack[words * p0 + n: words * p1] = vals_h[p0:p1]
        cap = max(int((self.blk_nnz[:, 1] - self.blk_nnz[:, 0]).max()) if len(self.blk_nnz) else 1, 1)
        if self._blocks_per_launch_arg is None and len(self.blk_nnz):
            avg_bytes = max(float((self.blk_nnz[:, 1] - self.blk_nnz[:, 0]).mean()) * 4 * words, 1.0)
            self.blocks_per_launch = self._round_launch(min(16, max(1, int(24e6 // avg_bytes))))
        if self.group.world > 1:
            # every launch of the pass kernel synchronises with the other ranks' launches group by group, so all
            # ranks cut the block order into the same batches
            import torch.distributed as dist

            t = torch.tensor([self.blocks_per_launch], dtype=torch.int64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group.group)
            self.blocks_per_launch = self._round_launch(int(t.item()))
        d = min(self.prefetch_depth, 16)
        # a ring slot holds one launch's worth of blocks; stage_base gets every block's address for the kernel
        self.stage = [torch.empty(cap * words * self.blocks_per_launch, dtype=torch.int32, device=self.dev)
                      for _ in range(d)]
        self.stage_base = torch.zeros(max(len(self.blk_nnz), 1), dtype=torch.int64, device=self.dev)
        self._stage_ptrs = (C.c_void_p * d)(*[t.data_ptr() for t in self.stage])
        lib = self._lib
        lib.psb_darlin_streamer_create.restype = C.c_void_p
        self._streamer = C.c_void_p(lib.psb_darlin_streamer_create(d))
        if not self._streamer:
            raise RuntimeError("could not create the block streamer (copy stream / events)")
        self.row_idx = self.stage[0]                          # placeholders for the struct; replaced per block
        self.vals = self.stage[0].view(torch.float32) if has_vals else None

    def _round_launch(self, n: int) -> int:
        g = self._launch_group
        return (max(int(n), 1) + g - 1) // g * g

    def __del__(self):
        st = getattr(self, "_streamer", None)
        if st:
            try:
                self._lib.psb_darlin_streamer_destroy(st)
            except Exception:
                pass
            self._streamer = None

    def _pass_streamed(self, order: np.ndarray, order_t: torch.Tensor) -> None:
        """One pass with every block's rows/values copied host→device just ahead of its kernel: one native
        call issues the copies, events and launches of all blocks (``psb_darlin_pass_streamed``)."""
        n = len(order)
        H = self._hyper()
        order_h = np.ascontiguousarray(order, dtype=np.int32)
        group = max(int(self.cfg.max_block_delay), 0) + 1
        Q = self._sched(order_t, n, group)
        moved, launches = C.c_ulonglong(0), C.c_int(0)
        N.check(self._lib.psb_darlin_pass_streamed(
            self._streamer, C.byref(self._Wk), C.byref(self._P), C.byref(self._S), C.byref(Q), C.byref(H), self.grid,
            order_h.ctypes.data_as(C.c_void_p), n, self.blk_nnz.ctypes.data_as(C.c_void_p),
            C.c_void_p(self.h_pack.data_ptr()), 1 if self.vals is not None else 0, self._stage_ptrs,
            C.c_void_p(self.stage_base.data_ptr()), self.blocks_per_launch, N.stream_ptr(), C.byref(moved),
            C.byref(launches)), "darlin_pass_streamed")
        self.h2d_bytes += moved.value
        self.kernel_launches += launches.value
        # a launch of `blocks_per_launch` blocks (a multiple of the group size) runs ceil(blocks / group) groups
        ngroups = sum((min(self.blocks_per_launch, n - f) + group - 1) // group for f in range(0, n, self.blocks_per_launch))
        self.seq += ngroups
        self.bar += ngroups
        self._prev_tail = order_t[(n - 1) // group * group:]

    def _sched(self, order_t: torch.Tensor, n: int, group: int) -> N.DarlinSched:
        prev = self._prev_tail
        return N.DarlinSched(order_t.data_ptr(), self.blk_lc.data_ptr(), self.blk_sl.data_ptr(), n, group, self.seq,
                             self.local_bar.data_ptr(), self.bar, self.abort.data_ptr(), self.status.data_ptr(), None,
                             None if prev is None else prev.data_ptr(), 0 if prev is None else prev.numel(),
                             self.wide_block_cols, self.blk_gc.data_ptr(), self.blk_gs0.data_ptr(),
                             1 if self.gather_small_groups else 0, 0, self.phase_ns.data_ptr(),
                             None if self._all_cb is None else self._all_cb.data_ptr(), self.nblk, self.list_block_cols)

    def _build_structs(self):
        Wk = N.DarlinWorker(self.col_ptr.data_ptr(), self.row_idx.data_ptr(),
                            0 if self.vals is None else self.vals.data_ptr(), self.ym.data_ptr(),
                            0 if self.col_of is None else self.col_of.data_ptr(), self.w.data_ptr(), self.delta.data_ptr(),
                            self.active.data_ptr(),
                            self.gslot.data_ptr(), self.gowner.data_ptr(), self.dw.data_ptr(), self.cols, self.rows, 0,
                            self.gcol.data_ptr())
        P = N.DarlinPeers()
        for r in range(self.group.world):
            P.w[r], P.gu[r] = self.srv_w.ptrs[r], self.srv_gu.ptrs[r]
            P.arrive[r] = self.arrive.ptrs[r]
            P.part[r] = self.srv_part.ptrs[r]
            if self._all_cb is not None:
                P.colgu[r], P.colslot[r] = self.col_gu.ptrs[r], self.col_slot.ptrs[r]
                P.coldw[r], P.arrive2[r] = self.col_dw.ptrs[r], self.arrive2.ptrs[r]
        P.mine = self.part_mine.data_ptr()
        P.rank, P.world, P.timeout_ns = self.group.rank, self.group.world, int(self.timeout_s * 1e9)
        P.gu_stride = self._gu_stride
        S = N.DarlinServer(self.srv_delta.data_ptr(), self.srv_active.data_ptr(), self.violation.data_ptr(), self.slots,
                           None if self.srv_d_slot is None else self.srv_d_slot.data_ptr())
        self._Wk, self._P, self._S = Wk, P, S
        self._lib.psb_darlin_grid.restype = C.c_int
        grid = self._lib.psb_darlin_grid()
        sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        grid = min(grid, sms * (self.ctas_per_sm or 2))
        if self.group.world > 1:
            import torch.distributed as dist

            t = torch.tensor([grid], dtype=torch.int64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group.group)
            grid = int(t.item())
        self.grid = grid

    def _hyper(self) -> N.DarlinHyper:
        return N.DarlinHyper(self.cfg.lambda1, self.cfg.eta, self.cfg.delta_max, min(self.kkt_threshold, 1e30))

    # ------------------------------------------------------------------ passes
    def warm_start(self, mkeys: np.ndarray, mvals: np.ndarray) -> None:
        """Start from a model (ascending uint64 ``mkeys`` with weights ``mvals``, e.g. an earlier job's dump) instead of
        zero: owners take the weights of their keys, workers those of their columns, and the margins become ``y * Xw``.
        Keys that the data lacks are ignored.  Call it right after ``preprocess`` on every rank with the same model."""
        if self.out_of_core:
            raise NotImplementedError("warm start needs the column blocks on the device")
        from ..utils.modelio import lookup_model

        def look(keys_t: torch.Tensor) -> torch.Tensor:
            w = lookup_model(mkeys, mvals, keys_t.cpu().numpy().view(np.uint64))
            return torch.from_numpy(w.astype(np.float32)).to(self.dev)

        self.srv_w.local.zero_()
        self.srv_w.local[: self.slots].copy_(look(self.skeys)[: self.slots])
        self.w.copy_(look(self.lkeys))
        self.margin.copy_(margins_from_weights(self.col_ptr, self.row_idx, self.vals, self.y, self.w))
        self.group.barrier()

    def reset_active_sets(self) -> None:
        """KKT filter reset (src/linear_method/darling.cc:167-169): every key re-enters the active set."""
        self.active.fill_(1)
        self.srv_active.fill_(1)
        if self.cfg.reset_nan_on_kkt_reset:
            torch.nan_to_num_(self.srv_w.local, nan=0.0)

    def reset_state(self) -> None:
        """Back to the state right after ``preprocess``: zero weights and margins, initial trust regions,
        every key active, empty progress (the data and the key resolution are kept)."""
        self.margin.zero_()
        self.w.zero_()
        self.dw.zero_()
        self.delta.fill_(self.cfg.delta_init)
        self.active.fill_(1)
        self.srv_w.local.zero_()
        self.srv_gu.local.zero_()
        self.part_mine.zero_()
        if self._all_cb is not None:
            self.col_gu.local.zero_()
        self._prev_tail = None
        self.srv_delta.fill_(self.cfg.delta_init)
        self.srv_active.fill_(1)
        self.progress = []
        self.kkt_threshold = 1e20
        self.group.barrier()

    def launch_pass(self, order: np.ndarray, delay: Optional[int] = None, first: bool = True) -> None:
        """Enqueue one pass over the blocks in ``order`` on the current stream.  ``delay``: bounded delay for
        these blocks when it differs from the configured one; ``first``: this is the first launch of a pass
        (the maximal KKT violation restarts)."""
        if delay is not None and delay != self.cfg.max_block_delay:
            saved, self.cfg.max_block_delay = self.cfg.max_block_delay, delay
            try:
                return self.launch_pass(order, first=first)
            finally:
                self.cfg.max_block_delay = saved
        order_t = torch.as_tensor(order, dtype=torch.int32).to(self.dev, non_blocking=False)
        self._order_keepalive = order_t
        if first:
            self.violation.zero_()
        if self.impl == "nccl":
            return self._pass_unfused(order)
        if self.out_of_core:
            return self._pass_streamed(np.asarray(order), order_t)
        group = max(int(self.cfg.max_block_delay), 0) + 1        # bounded delay: tau+1 blocks share their sync points
        Q = self._sched(order_t, len(order), group)
        H = self._hyper()
        N.check(self._lib.psb_darlin_pass(C.byref(self._Wk), C.byref(self._P), C.byref(self._S), C.byref(Q),
                                          C.byref(H), self.grid, N.stream_ptr()), "darlin_pass")
        ngroups = (len(order) + group - 1) // group
        self.seq += ngroups
        self.bar += ngroups
        self.kernel_launches += 1
        self._prev_tail = order_t[(len(order) - 1) // group * group:]

    def _pass_unfused(self, order: np.ndarray) -> None:
        """Baseline: per block, stand-alone kernels + all_reduce of (G,U) + broadcast-free local update."""
        import torch.distributed as dist

        lib, s, H, W = self._lib, N.stream_ptr(), self._hyper(), self.group.world
        blk_lc, blk_sl = self.blk_lc.tolist(), self.blk_sl.tolist()
        gs0 = self.blk_gs0.tolist()
        nglobal = self.gkeys_sorted.numel()
        # global column index of each local column, for dense exchange buffers
        if not hasattr(self, "_gcol"):
            self._gcol = self.gcol
            self._gu_glob = torch.zeros((nglobal, 2), dtype=torch.float32, device=self.dev)
            self._w_glob = torch.zeros((nglobal,), dtype=torch.float32, device=self.dev)
            to_s = lambda ks: torch.tensor([min(k, (1 << 64) - 1) + _SIGN for k in ks], dtype=torch.int64, device=self.dev)
            g0s = torch.searchsorted(self.gkeys_sorted, to_s([b for b, _ in self.block_keys])).tolist()
            g1s = [nglobal if e >= (1 << 64) else v for (_, e), v in zip(
                self.block_keys, torch.searchsorted(self.gkeys_sorted, to_s([e for _, e in self.block_keys])).tolist())]
            self._blk_g = list(zip(g0s, g1s))
        r = self.group.rank
        for b in order.tolist():
            lc0, lc1 = blk_lc[b]
            g0, g1 = self._blk_g[b]
            if g1 <= g0:
                continue
            gu_loc = torch.zeros((max(lc1 - lc0, 1), 2), dtype=torch.float32, device=self.dev)
            nnz_b = int((self.col_ptr[lc1] - self.col_ptr[lc0]).item()) if lc1 > lc0 else 0
            if nnz_b:
                N.check(lib.psb_darlin_grad_local(C.byref(self._Wk), lc0, lc1, N.ptr(gu_loc), nnz_b, s), "grad_local")
                self.kernel_launches += 1
            gu = self._gu_glob[g0:g1]
            gu.zero_()
            if lc1 > lc0:
                gu.index_add_(0, self._gcol[lc0:lc1] - g0, gu_loc[: lc1 - lc0])
            if W > 1:
                dist.all_reduce(gu, group=self.group.group)          # push + server-side sum
            s0, s1 = blk_sl[b]
            if s1 > s0:
                self.srv_gu.local[0, s0:s1].copy_(gu[gs0[b] - g0: gs0[b] - g0 + s1 - s0])
                N.check(lib.psb_darlin_update_weight(C.byref(self._P), C.byref(self._S), C.byref(H), s0, s1, s), "update_weight")
                self.kernel_launches += 1
            wb = self._w_glob[g0:g1]
            wb.zero_()
            if s1 > s0:
                wb[gs0[b] - g0: gs0[b] - g0 + s1 - s0] = self.srv_w.local[s0:s1]
            if W > 1:
                wnan = torch.isnan(wb)
                wz = torch.nan_to_num(wb, nan=0.0)
                nanf = wnan.to(torch.float32)
                dist.all_reduce(wz, group=self.group.group)          # pull (all-gather of disjoint shards)
                dist.all_reduce(nanf, group=self.group.group)
                wb = torch.where(nanf > 0, torch.full_like(wz, float("nan")), wz)
            if lc1 > lc0:
                wn = wb[self._gcol[lc0:lc1] - g0].contiguous()
                N.check(lib.psb_darlin_apply_pull(C.byref(self._Wk), C.byref(H), lc0, lc1, N.ptr(wn), s), "apply_pull")
                if nnz_b:
                    N.check(lib.psb_darlin_update_margin(C.byref(self._Wk), lc0, lc1, nnz_b, s), "update_margin")
                self.kernel_launches += 2

    def phase_times_ms(self, reset: bool = True) -> dict:
        """Time thread block 0 spent per phase since the last reset, from in-kernel globaltimer reads."""
        t = (self.phase_ns.to(torch.float64) / 1e6).tolist()
        if reset:
            self.phase_ns.zero_()
        out = {"commit_grad": t[0], "arrive_wait": t[1], "update_margin": t[2], "gpu_barrier": t[3]}
        if t[4] > 0:     # very wide groups on several GPUs: the parts of "update_margin"
            out.update(list_sum=t[4], list_update=t[5], list_reply=t[6], list_wait=t[7], list_apply=t[8], list_margin=t[9])
        return out

    def evaluate(self) -> tuple:
        """(objective, nnz_w, nnz_active, violation) summed/maxed over ranks (Darling::evaluateProgress)."""
        loss = reduce_sum(self.margin.contiguous(), "sum_logistic")
        srv = self.srv_w.local[: max(self.slots, 0)]
        if self.slots > 0:
            pen = reduce_sum(srv, "sum_abs").clone()
            nz = reduce_sum(srv, "count_nonzero").clone()
            nact = self.srv_active[: self.slots].sum(dtype=torch.float64)
        else:
            pen = nz = nact = torch.zeros(1, dtype=torch.float64, device=self.dev)
        vals = torch.stack([loss.reshape(()), pen.reshape(()), nz.reshape(()), nact.reshape(())])
        vio = self.violation.view(torch.float32)
        if self.group.world > 1 and self.impl == "fused":
            # merged inside one small kernel over peer memory (in-switch reduction where the box has multicast)
            if getattr(self, "_scalars", None) is None:
                from ..parallel.scalar_reduce import ScalarAllReduce

                self._scalars = ScalarAllReduce(self.group, timeout_s=self.timeout_s)
            vals, vio = self._scalars(vals, vio)
        elif self.group.world > 1:
            import torch.distributed as dist

            vio = vio.to(torch.float64)
            dist.all_reduce(vals, group=self.group.group)
            dist.all_reduce(vio, op=dist.ReduceOp.MAX, group=self.group.group)
        v = vals.tolist()
        return v[0] + self.cfg.lambda1 * v[1], int(v[2]), int(v[3]), float(vio.item())

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"rank {self.group.rank}: {N.STATUS_NAMES.get(st[0], st[0])} (block={st[1]}, phase={st[2]})")

    def run_pass(self, order: np.ndarray, reset: bool = False, prior: Optional[List[int]] = None) -> Progress:
        """One pass; ``prior``: blocks swept before ``order`` with zero delay (first pass, important groups)."""
        from ..utils.trace import nvtx_range

        t0 = time.time()
        trace, metrics = getattr(self, "trace", None), getattr(self, "metrics", None)
        monitor = getattr(self, "monitor", None)     # parallel.monitor.RankMonitor: look at the other ranks before launching
        if monitor is not None:
            monitor.tick(len(self.progress))
        if reset:
            self.reset_active_sets()
        if prior:
            self.launch_pass(np.asarray(prior, dtype=np.int32), delay=0)
        with nvtx_range("darlin_pass"):
            if trace is not None:
                with trace.span("darlin_pass", cat="solver", device_timed=True, blocks=len(order), it=len(self.progress)):
                    self.launch_pass(order, first=not prior)
            else:
                self.launch_pass(order, first=not prior)
        with nvtx_range("evaluate_progress"):
            objv, nnz_w, nnz_as, vio = self.evaluate()
        self.check_status()
        if metrics is not None and self.group.rank == 0:
            metrics.log(event="pass", it=len(self.progress), objective=objv, nnz_w=nnz_w, active=nnz_as, violation=vio,
                        seconds=time.time() - t0, examples_per_s=self.total_rows / max(time.time() - t0, 1e-9),
                        h2d_bytes=self.h2d_bytes)
        rel = 1.0 if not self.progress else self.progress[-1].objv / objv - 1.0
        p = Progress(objv, rel, nnz_w, vio, nnz_as, self.kkt_threshold, time.time() - t0)
        self.progress.append(p)
        self.kkt_threshold = vio / max(self.total_rows, 1) * self.cfg.kkt_ratio
        return p

    def run(self, verbose: bool = False) -> List[Progress]:
        """All passes with the reference's stopping rule (src/linear_method/darling.cc:83-99)."""
        cfg = self.cfg
        orders = block_order(self.nblk, cfg.max_pass, cfg.random_block_order, cfg.seed)
        prior = prior_block_order(self.block_group, cfg.prior_fea_group, cfg.num_iter_for_prior_fea_group,
                                  cfg.random_block_order, cfg.seed)
        reset = False
        for it in range(cfg.max_pass):
            p = self.run_pass(orders[it], reset, prior if it == 0 else None)
            if verbose and self.group.rank == 0:
                print_progress(it, p, file=sys.stderr)
            if 0 < p.relative_objv <= cfg.epsilon:
                if reset:
                    break
                reset = True
            else:
                reset = False
        return self.progress

    # ------------------------------------------------------------------ model
    def model(self):
        """(keys uint64, w float32) of this shard's non-zero weights, ascending keys."""
        w = torch.nan_to_num(self.srv_w.local[: self.slots], nan=0.0)
        nz = w != 0
        return self.skeys[nz].cpu().numpy().view(np.uint64), w[nz].cpu().numpy()

    def save_model(self, file_prefix: str) -> str:
        """``<file>_S<rank>``: ``key<TAB>weight`` per non-zero weight (batch_solver.cc:403-426)."""
        from ..utils.modelio import write_model_text

        k, w = self.model()
        path = f"{file_prefix}_S{self.group.rank}"
        write_model_text(path, k, w)
        return path


def print_progress(it: int, p: Progress, file=sys.stderr, busy=None) -> None:
    """Progress table in the reference's layout (linear_method.cc:181-231, darling.cc:480-501).  ``busy``: the nodes'
    compute seconds of this pass; a scheduler that has them prints the reference's "(app:min max) total" columns."""
    if it == 0:
        print("     |        training        |  sparsity |      KKT filter     |" + ("    time (sec.)" if busy else "  time"), file=file)
        print("iter |  objective    relative |     |w|_0 | threshold  #activet |" + ("(app:min max) total" if busy else " (sec)"), file=file)
        print(" ----+------------------------+-----------+---------------------+" + ("-----------------" if busy else "-------"), file=file)
    tail = f"{min(busy):6.1f}{max(busy):6.1f}{p.seconds:6.1f}" if busy else f"{p.seconds:6.2f}"
    print(f"{it:4d} | {p.objv:.5e}  {p.relative_objv:.3e} |{p.nnz_w:10d} | {p.kkt_threshold:.1e} {p.nnz_active:11d} |{tail}", file=file)


def smoke(dev) -> None:
    """Tiny end-to-end run used by the build driver's smoke test."""
    from ..data.synthetic import zipf_sparse_matrix

    off, idx, vals, y, _ = zipf_sparse_matrix(2000, 4096, 24, seed=0, device=dev)
    sol = DarlinSolver(PeerGroup.single(dev), DarlinConfig(lambda1=0.5, max_pass=4))
    sol.preprocess(off, idx, vals, y)
    prog = sol.run()
    assert prog[-1].objv < prog[0].objv * 1.0001 and prog[-1].objv == prog[-1].objv
    print(f"smoke ok: DARLIN {len(prog)} passes, objective {prog[0].objv:.2f} -> {prog[-1].objv:.2f}, |w|_0 {prog[-1].nnz_w}")
