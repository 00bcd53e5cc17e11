"""fp64 CPU restatement of the reference's online FTRL (oracle + timed CPU baseline).

Server rule: FTRLModel::setValue (src/linear_method/ftrl_model.h:81-112); worker
minibatch: FTRL::updateModel (src/linear_method/ftrl.cc:88-151) with LogitLoss
(src/linear_method/loss.h:73-88) and countKeys (src/linear_method/ftrl.cc:154-174).

The schedule is bulk-synchronous over W workers: in step t every worker pulls the
model as of the end of step t-1, then the pushes are applied worker by worker in
rank order — one legal serialisation of the reference's asynchronous execution
and the one the GPU engine implements.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np


@dataclass
class Entry:
    pos: float = 0.0
    neg: float = 0.0
    w: float = 0.0
    z: float = 0.0


@dataclass
class FTRLRef:
    alpha: float = 0.1
    beta: float = 1.0
    lambda1: float = 1.0
    lambda2: float = 0.1
    rule: str = "count"
    model: Dict[int, Entry] = field(default_factory=dict)
    norm1: float = 0.0
    norm2: float = 0.0
    nnz: int = 0

    @staticmethod
    def _sqrt_n(pos: float, neg: float) -> float:
        a = pos + neg
        return 0.0 if a == 0 else math.sqrt(pos * neg / a)

    def get(self, key: int) -> float:
        e = self.model.get(key)
        return 0.0 if e is None else e.w

    def set_value(self, keys: Sequence[int], pos, neg, grad) -> None:
        for k, p, n, g in zip(keys, pos, neg, grad):
            e = self.model.setdefault(int(k), Entry())
            if self.rule == "count":
                sq = self._sqrt_n(e.pos, e.neg)
                e.pos += float(p)
                e.neg += float(n)
                sq_new = self._sqrt_n(e.pos, e.neg)
            else:
                sq = math.sqrt(e.pos)
                e.pos += float(g) * float(g)
                sq_new = math.sqrt(e.pos)
            sigma = (sq_new - sq) / self.alpha
            e.z += float(g) - sigma * e.w
            l2 = self.lambda2 + (self.beta + sq_new) / self.alpha
            w_old = e.w
            az = abs(e.z) - self.lambda1
            w = -math.copysign(az, e.z) / l2 if az > 0 else 0.0
            e.w = w
            self.norm1 += abs(w) - abs(w_old)
            self.norm2 += w * w - w_old * w_old
            if w == 0 and w_old != 0:
                self.nnz -= 1
            elif w != 0 and w_old == 0:
                self.nnz += 1

    def objv(self) -> float:
        return self.norm1 * self.lambda1 + 0.5 * self.lambda2 * math.sqrt(max(self.norm2, 0.0))

    # ------------------------------------------------------------------ worker
    def worker_gradient(self, offsets: np.ndarray, keys: np.ndarray, y: np.ndarray, vals: Optional[np.ndarray] = None):
        """Returns (unique keys, pos, neg, grad, loss, xw) for one minibatch against the current model."""
        ukeys, inv = np.unique(keys, return_inverse=True)
        w = np.array([self.get(int(k)) for k in ukeys], dtype=np.float64)
        rows = len(y)
        row_of = np.repeat(np.arange(rows), np.diff(offsets))
        v = np.ones(len(keys)) if vals is None else vals.astype(np.float64)
        xw = np.bincount(row_of, weights=w[inv] * v, minlength=rows)
        m = y * xw
        loss = float(np.sum(np.logaddexp(0.0, -m)))
        coef = -y / (1.0 + np.exp(m))
        grad = np.bincount(inv, weights=coef[row_of] * v, minlength=len(ukeys))
        pos = np.bincount(inv, weights=(y[row_of] > 0).astype(np.float64), minlength=len(ukeys))
        neg = np.bincount(inv, weights=(y[row_of] <= 0).astype(np.float64), minlength=len(ukeys))
        return ukeys, pos, neg, grad, loss, xw

    def step(self, minibatches: List[tuple]) -> float:
        """One bulk-synchronous step over W workers' minibatches [(offsets, keys, y[, vals])]; returns Σloss."""
        pushes, loss = [], 0.0
        for mb in minibatches:
            uk, pos, neg, g, l, _ = self.worker_gradient(*mb)
            pushes.append((uk, pos, neg, g))
            loss += l
        for uk, pos, neg, g in pushes:
            self.set_value(uk, pos, neg, g)
        return loss

    def nonzero(self):
        items = sorted((k, e.w) for k, e in self.model.items() if e.w != 0)
        return (np.array([k for k, _ in items], dtype=np.uint64), np.array([w for _, w in items], dtype=np.float64))
