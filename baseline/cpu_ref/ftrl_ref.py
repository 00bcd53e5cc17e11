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


class CountMinRef:
    """Count-min sketch with the reference's probe sequence (src/base/countmin.h:33-67): 32-bit
    hash h of the 64-bit key, probes (h + j·rotr17(h)) mod n, insert adds, query takes the minimum.
    Counters are uint32 (the reference's uint8 counters wrap at 256)."""

    def __init__(self, n: int, k: int):
        self.n, self.k = max(int(n), 64), max(int(k), 1)
        self.table = np.zeros(self.n, dtype=np.uint64)

    @staticmethod
    def _hash(keys: np.ndarray) -> np.ndarray:
        m, mask = np.uint64(0xc6a4a793), np.uint64(0xFFFFFFFF)
        keys = keys.astype(np.uint64)
        h = np.full(keys.shape, (0xbc9f1d34 ^ ((8 * 0xc6a4a793) & 0xFFFFFFFF)), dtype=np.uint64)
        for part in (keys & mask, keys >> np.uint64(32)):
            h = (h + part) & mask
            h = (h * m) & mask
            h ^= h >> np.uint64(16)
        return h

    def _probes(self, keys: np.ndarray):
        h = self._hash(keys)
        mask = np.uint64(0xFFFFFFFF)
        d = ((h >> np.uint64(17)) | (h << np.uint64(15))) & mask
        for _ in range(self.k):
            yield (h % np.uint64(self.n)).astype(np.int64)
            h = (h + d) & mask

    def insert(self, keys: np.ndarray, counts: np.ndarray) -> None:
        for idx in self._probes(keys):
            np.add.at(self.table, idx, counts.astype(np.uint64))

    def query(self, keys: np.ndarray) -> np.ndarray:
        out = np.full(len(keys), np.iinfo(np.uint64).max, dtype=np.uint64)
        for idx in self._probes(keys):
            out = np.minimum(out, self.table[idx])
        return out


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
    # tail-feature filter: every server s owns keys in [seps[s], seps[s+1]) and a sketch of width
    # countmin_n / num_servers; a pushed key is applied only once its estimate exceeds tail_freq
    tail_freq: int = 0
    countmin_n: int = 1 << 20
    countmin_k: int = 2
    seps: Optional[Sequence[int]] = None
    _sketch: Optional[list] = None

    def _admitted(self, keys: np.ndarray, pos: np.ndarray, neg: np.ndarray) -> np.ndarray:
        """Insert one worker's row counts server by server, then query: mask of keys that pass the filter."""
        if self.tail_freq <= 0:
            return np.ones(len(keys), dtype=bool)
        seps = list(self.seps) if self.seps is not None else [0, 1 << 64]
        S = len(seps) - 1
        if self._sketch is None:
            self._sketch = [CountMinRef(int(self.countmin_n) // S, self.countmin_k) for _ in range(S)]
        keys = np.asarray(keys, dtype=np.uint64)
        ok = np.zeros(len(keys), dtype=bool)
        for s in range(S):
            hi = seps[s + 1]
            sel = (keys >= np.uint64(seps[s])) & ((keys < np.uint64(hi)) if hi < (1 << 64) else np.ones(len(keys), bool))
            if not sel.any():
                continue
            cnt = (pos[sel] + neg[sel]).astype(np.uint64)
            self._sketch[s].insert(keys[sel], cnt)
            ok[sel] = self._sketch[s].query(keys[sel]) > np.uint64(self.tail_freq)
        return ok

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
            ok = self._admitted(uk, pos, neg)
            self.set_value(uk[ok], pos[ok], neg[ok], g[ok])
        return loss

    def nonzero(self):
        items = sorted((k, e.w) for k, e in self.model.items() if e.w != 0)
        return (np.array([k for k, _ in items], dtype=np.uint64), np.array([w for _, w in items], dtype=np.float64))
