"""fp64 CPU restatement of DARLIN (delayed block proximal-Newton CD for L1 logistic regression).

Math and control flow of the reference: Darling::computeGradients / updateWeight / updateDual /
runIteration / evaluateProgress (src/linear_method/darling.cc:18-104, 306-477, 503-557) and the
feature-block partition of BatchSolver::run (src/linear_method/batch_solver.cc:48-66).  Workers
hold row shards; servers hold key ranges; blocks are processed strictly in order (bounded delay
τ = 0), which is the schedule the GPU engine implements.  Used as the oracle of the GPU kernels
and as the timed CPU baseline.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import scipy.sparse as sp


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
    seed: int = 0
    max_block_delay: int = 0              # tau: groups of tau+1 blocks compute all gradients before any update
    reset_nan_on_kkt_reset: bool = True   # reference leaves filtered weights NaN forever (quirk)
    feature_group_bits: int = 0           # b > 0: a key's top b bits are its feature group (batch_solver.cc:48-66)
    prior_fea_group: tuple = ()           # groups swept first, with zero delay, in the first pass (batch_solver.cc:88-108)
    num_iter_for_prior_fea_group: int = 5


def block_ranges(min_key: int, max_key_excl: int, nnz_per_row: float, ratio: float) -> List[Tuple[int, int]]:
    """Key ranges of the feature blocks of one group (batch_solver.cc:55-65)."""
    n = 1
    if nnz_per_row > 1 + 1e-6:
        n = max(int(math.ceil(nnz_per_row * ratio)), 1)
    size = max_key_excl - min_key
    out = []
    for i in range(n):
        b = min_key + size * i // n
        e = max_key_excl if i + 1 == n else min_key + size * (i + 1) // n
        out.append((b, e))
    return out


def block_order(nblk: int, n_pass: int, random_order: bool, seed: int) -> List[np.ndarray]:
    """Block visiting order of every pass (deterministic stand-in for std::random_shuffle)."""
    rng = np.random.RandomState(seed)
    out = []
    for _ in range(n_pass):
        o = np.arange(nblk, dtype=np.int32)
        if random_order:
            rng.shuffle(o)
        out.append(o)
    return out


@dataclass
class Progress:
    objv: float
    relative_objv: float
    nnz_w: int
    violation: float
    nnz_active: int
    kkt_threshold: float


class DarlinRef:
    """Single-process DARLIN over W row shards (list of CSR (offsets, cols, vals|None, y))."""

    def __init__(self, shards: Sequence[tuple], num_keys_hint: Optional[int], cfg: DarlinConfig):
        self.cfg = cfg
        self.X, self.y, self.dual = [], [], []
        keys_all = np.unique(np.concatenate([s[1] for s in shards]))
        self.keys = keys_all                         # sorted global unique keys
        P = len(keys_all)
        nnz = 0
        rows = 0
        self.binary = all(s[2] is None for s in shards)
        for off, cols, vals, y in shards:
            n = len(y)
            j = np.searchsorted(keys_all, cols)
            v = np.ones(len(cols)) if vals is None else vals.astype(np.float64)
            row_of = np.repeat(np.arange(n), np.diff(off))
            self.X.append(sp.csc_matrix((v, (row_of, j)), shape=(n, P)))
            self.y.append(y.astype(np.float64))
            self.dual.append(np.ones(n))
            nnz += len(cols)
            rows += n
        self.rows = rows
        self.w = np.zeros(P)
        self.delta = np.full(P, float(cfg.delta_init))
        self.active = np.ones(P, dtype=bool)
        self.wk_w = [np.zeros(P) for _ in shards]
        self.wk_delta = [np.full(P, float(cfg.delta_init)) for _ in shards]
        self.wk_active = [np.ones(P, dtype=bool) for _ in shards]
        self.violation = 0.0
        self.kkt_threshold = 1e20
        mn, mx = int(keys_all.min()), int(keys_all.max()) + 1
        if cfg.feature_group_bits > 0:
            # per group: key range, non-zeros, examples in which the group occurs; blocks group by group
            sh = np.uint64(64 - cfg.feature_group_bits)
            self.block_keys, self.block_group = [], []
            for g in np.unique(keys_all >> sh).tolist():
                gk = keys_all[(keys_all >> sh) == np.uint64(g)]
                ele = ex = 0
                for off, cols, _, y in shards:
                    m = (cols >> sh) == np.uint64(g)
                    ele += int(m.sum())
                    ex += len(np.unique(np.repeat(np.arange(len(y)), np.diff(off))[m]))
                for b, e in block_ranges(int(gk.min()), int(gk.max()) + 1, ele / max(ex, 1), cfg.feature_block_ratio):
                    if e > b:
                        self.block_keys.append((b, e))
                        self.block_group.append(int(g))
        else:
            self.block_keys = block_ranges(mn, mx, nnz / rows, cfg.feature_block_ratio)
            self.block_group = [1] * len(self.block_keys)
        self.blocks = [(int(np.searchsorted(keys_all, np.uint64(b))),
                        len(keys_all) if e >= (1 << 64) else int(np.searchsorted(keys_all, np.uint64(e)))) for b, e in self.block_keys]
        self.progress: List[Progress] = []

    # ------------------------------------------------------------------ block step
    def _gradients(self, k: int, c0: int, c1: int):
        X, y, dual = self.X[k], self.y[k], self.dual[k]
        G = np.zeros(c1 - c0)
        U = np.zeros(c1 - c0)
        tau = 1.0 / (1.0 + dual)
        t2 = tau * (1 - tau)
        for jj, j in enumerate(range(c0, c1)):
            if not self.wk_active[k][j]:
                continue
            s, e = X.indptr[j], X.indptr[j + 1]
            rows, v = X.indices[s:e], X.data[s:e]
            d = self.wk_delta[k][j]
            G[jj] = -np.sum(y[rows] * tau[rows] * v)
            if self.binary:
                U[jj] = np.sum(np.minimum(t2[rows] * math.exp(d), 0.25))
            else:
                U[jj] = np.sum(np.minimum(t2[rows] * np.exp(np.abs(v) * d), 0.25) * v * v)
        return G, U

    def _update_weight(self, c0: int, c1: int, G: np.ndarray, U: np.ndarray):
        cfg = self.cfg
        for jj, k in enumerate(range(c0, c1)):
            if not self.active[k]:
                continue
            g, u = G[jj], U[jj] / cfg.eta + 1e-10
            gp, gn = g + cfg.lambda1, g - cfg.lambda1
            w = self.w[k]
            d, vio = -w, 0.0
            if w == 0:
                if gp < 0:
                    vio = -gp
                elif gn > 0:
                    vio = gn
                elif gp > self.kkt_threshold and gn < -self.kkt_threshold:
                    self.active[k] = False
                    self.w[k] = np.nan
                    continue
            self.violation = max(self.violation, vio)
            if gp <= u * w:
                d = -gp / u
            elif gn >= u * w:
                d = -gn / u
            d = min(self.delta[k], max(-self.delta[k], d))
            self.delta[k] = min(cfg.delta_max, 2 * abs(d) + 0.1)
            self.w[k] = w + d

    def _update_dual(self, k: int, c0: int, c1: int):
        X, y = self.X[k], self.y[k]
        for j in range(c0, c1):
            if not self.wk_active[k][j]:
                continue
            wn = self.w[j]
            if wn != wn:
                self.wk_active[k][j] = False
                self.wk_w[k][j] = 0.0
                continue
            d = wn - self.wk_w[k][j]
            self.wk_delta[k][j] = min(self.cfg.delta_max, 2 * abs(d) + 0.1)
            self.wk_w[k][j] = wn
            if d != 0:
                s, e = X.indptr[j], X.indptr[j + 1]
                rows, v = X.indices[s:e], X.data[s:e]
                self.dual[k][rows] *= np.exp(y[rows] * v * d)

    def run_block(self, b: int) -> None:
        c0, c1 = self.blocks[b]
        if c1 <= c0:
            return
        G = np.zeros(c1 - c0)
        U = np.zeros(c1 - c0)
        for k in range(len(self.X)):
            g, u = self._gradients(k, c0, c1)
            G += g
            U += u
        self._update_weight(c0, c1, G, U)
        for k in range(len(self.X)):
            self._update_dual(k, c0, c1)

    def run_group(self, blocks) -> None:
        """Bounded delay: gradients of every block of the group first, then the updates, then the duals."""
        if len(blocks) == 1:
            return self.run_block(blocks[0])
        grads = []
        for b in blocks:
            c0, c1 = self.blocks[b]
            G, U = np.zeros(max(c1 - c0, 0)), np.zeros(max(c1 - c0, 0))
            if c1 > c0:
                for k in range(len(self.X)):
                    g, u = self._gradients(k, c0, c1)
                    G += g
                    U += u
            grads.append((c0, c1, G, U))
        for c0, c1, G, U in grads:
            if c1 > c0:
                self._update_weight(c0, c1, G, U)
        for c0, c1, _, _ in grads:
            for k in range(len(self.X)):
                if c1 > c0:
                    self._update_dual(k, c0, c1)

    # ------------------------------------------------------------------ passes
    def evaluate(self) -> Tuple[float, int, int]:
        loss = sum(float(np.sum(np.log1p(1.0 / d))) for d in self.dual)
        fin = np.nan_to_num(self.w, nan=0.0)
        return loss + self.cfg.lambda1 * float(np.abs(fin).sum()), int((fin != 0).sum()), int(self.active.sum())

    def prior_order(self) -> List[int]:
        """Extra sweeps over the blocks of the important groups (same draw as the solvers')."""
        rng = np.random.RandomState(self.cfg.seed + 1)
        out: List[int] = []
        for g in self.cfg.prior_fea_group:
            tmp = [k for k, bg in enumerate(self.block_group) if bg == int(g)]
            for _ in range(int(self.cfg.num_iter_for_prior_fea_group) if tmp else 0):
                if self.cfg.random_block_order:
                    rng.shuffle(tmp)
                out += list(tmp)
        return out

    def run_pass(self, order: np.ndarray, reset: bool, prior: Sequence[int] = ()) -> Progress:
        self.violation = 0.0
        if reset:
            self.active[:] = True
            for a in self.wk_active:
                a[:] = True
            if self.cfg.reset_nan_on_kkt_reset:
                self.w[np.isnan(self.w)] = 0.0
        g = max(int(self.cfg.max_block_delay), 0) + 1
        order = [int(b) for b in order]
        for b in prior:                       # zero delay: one block at a time
            self.run_block(int(b))
        for i in range(0, len(order), g):
            self.run_group(order[i:i + g])
        objv, nnz_w, nnz_as = self.evaluate()
        rel = 1.0 if not self.progress else self.progress[-1].objv / objv - 1.0
        p = Progress(objv, rel, nnz_w, self.violation, nnz_as, self.kkt_threshold)
        self.progress.append(p)
        self.kkt_threshold = self.violation / self.rows * self.cfg.kkt_ratio
        return p

    def run(self) -> List[Progress]:
        cfg = self.cfg
        orders = block_order(len(self.blocks), cfg.max_pass, cfg.random_block_order, cfg.seed)
        reset = False
        prior = self.prior_order()
        for it in range(cfg.max_pass):
            p = self.run_pass(orders[it], reset, prior if it == 0 else ())
            if 0 < p.relative_objv <= cfg.epsilon:
                if reset:
                    break
                reset = True
            else:
                reset = False
        return self.progress

    def model(self):
        m = np.nan_to_num(self.w, nan=0.0)
        nz = m != 0
        return self.keys[nz], m[nz]
