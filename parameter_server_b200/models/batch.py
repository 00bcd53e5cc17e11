"""Plain batch solver: block proximal-gradient / gradient-descent learners over the loss and
penalty families, for jobs whose ``.conf`` has no ``darling{}`` section.

The reference ships this path half-finished — ``BatchSolver::updateModel`` is commented out and the
``learner/`` classes do not compile — but documents the intent: per feature block, aggregate the
gradient and the diagonal Hessian over the workers and let the learner update the block's weights
(src/linear_method/learner/proximal_gradient.h:20-53, gradient_descent.h:19-24,
src/linear_method/loss.h:73-104, src/linear_method/penalty.h:15-50,
src/test/aggregated_gradient_test.cc:52-104).  Here it is implemented: rows are sharded over the
ranks, every rank keeps the whole weight vector, and the block gradients are summed with an
all-reduce.  The arithmetic is torch on the device; the hot, fused path of this framework is DARLIN.
"""
from __future__ import annotations

import math
import sys
import time
from typing import List

import numpy as np
import torch

from ..parallel.peer import PeerGroup
from .darlin import DarlinConfig, Progress, block_order, print_progress

_SIGN = -(1 << 63)


# ------------------------------------------------------------------ loss / penalty families
class Loss:
    """Scalar loss on margins Xw with labels y in ±1: evaluate, per-row gradient coefficient and curvature."""

    @staticmethod
    def create(kind: str) -> "Loss":
        return {"LOGIT": LogitLoss, "SQUARE_HINGE": SquareHingeLoss}[kind]()


class LogitLoss(Loss):
    def evaluate(self, y, xw):
        return torch.nn.functional.softplus(-y * xw).sum(dtype=torch.float64)

    def coef(self, y, xw):            # d loss / d (Xw)_i
        tau = torch.sigmoid(-y * xw)
        return -y * tau, tau * (1 - tau)


class SquareHingeLoss(Loss):
    def evaluate(self, y, xw):
        return torch.clamp(1 - y * xw, min=0).square().sum(dtype=torch.float64)

    def coef(self, y, xw):
        # the reference's formula is −2·y·[y·Xw > 1] (src/linear_method/loss.h:102), which has the
        # indicator inverted; the gradient of max(0, 1 − y·Xw)² is used here
        act = (y * xw < 1).to(xw.dtype)
        return -2 * y * (1 - y * xw) * act, 2 * act


class Penalty:
    @staticmethod
    def create(kind: str, lam: float) -> "PNormPenalty":
        return PNormPenalty(1 if kind == "L1" else 2, lam)


class PNormPenalty(Penalty):
    """λ·Σ|w_i|^p."""

    def __init__(self, p: int, lam: float):
        self.p, self.lam = p, lam

    def evaluate(self, w) -> float:
        return float(self.lam * w.abs().pow(self.p).sum(dtype=torch.float64))


class ProxGradientSolver:
    """Block coordinate learner with replicated weights and row-sharded data."""

    def __init__(self, group: PeerGroup, cfg: DarlinConfig, loss: str = "LOGIT", penalty: str = "L1",
                 learner: str = "PROXIMAL_GRADIENT"):
        self.group, self.cfg, self.dev = group, cfg, group.device
        self.loss, self.penalty = Loss.create(loss), Penalty.create(penalty, cfg.lambda1)
        self.learner = learner
        self.progress: List[Progress] = []

    def preprocess(self, offsets, keys, vals, y) -> None:
        import torch.distributed as dist

        g, dev = self.group, self.dev
        uk = torch.unique(keys ^ _SIGN)
        if g.world > 1:
            sizes = [None] * g.world
            dist.all_gather_object(sizes, int(uk.numel()), group=g.group)
            pad = torch.full((max(sizes),), (1 << 63) - 1, dtype=torch.int64, device=dev)
            pad[: uk.numel()] = uk
            parts = [torch.empty_like(pad) for _ in range(g.world)]
            dist.all_gather(parts, pad, group=g.group)
            uk = torch.unique(torch.cat([p[:n] for p, n in zip(parts, sizes)]))
        self.gkeys = uk                      # ordered (sign-flipped) global keys
        col = torch.searchsorted(uk, keys ^ _SIGN)
        rows = y.numel()
        row_of = torch.repeat_interleave(torch.arange(rows, device=dev), offsets[1:] - offsets[:-1])
        order = torch.sort(col, stable=True).indices
        self.col, self.row = col[order], row_of[order]
        self.val = torch.ones_like(self.col, dtype=torch.float32) if vals is None else vals[order]
        P = uk.numel()
        self.col_ptr = torch.zeros(P + 1, dtype=torch.int64, device=dev)
        self.col_ptr[1:] = torch.bincount(self.col, minlength=P).cumsum(0)
        self.y, self.w = y, torch.zeros(P, device=dev)
        self.xw = torch.zeros(rows, device=dev)
        tot = g.all_reduce_sum([rows, keys.numel()])
        self.total_rows = int(tot[0])
        per_row = tot[1] / max(tot[0], 1)
        r = self.cfg.feature_block_ratio
        self.nblk = max(int(math.ceil(per_row * r)), 1) if (per_row > 1 + 1e-6 and r > 0) else 1
        kmin, kmax = int(uk[0].item()) - _SIGN, int(uk[-1].item()) - _SIGN + 1
        bounds = [kmin + (kmax - kmin) * i // self.nblk for i in range(self.nblk)] + [kmax]
        b = torch.tensor([min(x, (1 << 64) - 1) + _SIGN for x in bounds], dtype=torch.int64, device=dev)
        c = torch.searchsorted(uk, b)
        c[-1] = P
        self.blk = c.tolist()

    def run_block(self, b: int) -> None:
        c0, c1 = self.blk[b], self.blk[b + 1]
        if c1 <= c0:
            return
        p0, p1 = int(self.col_ptr[c0]), int(self.col_ptr[c1])
        rows, cols, v = self.row[p0:p1], self.col[p0:p1] - c0, self.val[p0:p1]
        gcoef, hcoef = self.loss.coef(self.y, self.xw)
        gu = torch.zeros((c1 - c0, 2), device=self.dev)
        gu[:, 0].index_add_(0, cols, gcoef[rows] * v)
        gu[:, 1].index_add_(0, cols, hcoef[rows] * v * v)
        if self.group.world > 1:
            import torch.distributed as dist

            dist.all_reduce(gu, group=self.group.group)
        G, U = gu[:, 0], gu[:, 1]
        w = self.w[c0:c1]
        eta, lam = self.cfg.eta, self.cfg.lambda1
        if self.learner == "GRADIENT_DESCENT":
            g = G + (2 * lam * w if self.penalty.p == 2 else 0.0)
            d = -eta * g
        elif self.penalty.p == 1:
            u = U / eta + 1e-10
            gp, gn = G + lam, G - lam
            d = torch.where(gp <= u * w, -gp / u, torch.where(gn >= u * w, -gn / u, -w)).clamp_(-5.0, 5.0)
        else:
            u = U / eta + 2 * lam + 1e-10
            d = (-(G + 2 * lam * w) / u).clamp_(-5.0, 5.0)
        self.w[c0:c1] = w + d
        self.xw.index_add_(0, rows, v * d[cols])

    def evaluate(self):
        loss = self.loss.evaluate(self.y, self.xw)
        if self.group.world > 1:
            import torch.distributed as dist

            dist.all_reduce(loss, group=self.group.group)
        return float(loss) + self.penalty.evaluate(self.w), int((self.w != 0).sum())

    def run(self, verbose: bool = False) -> List[Progress]:
        orders = block_order(self.nblk, self.cfg.max_pass, self.cfg.random_block_order, self.cfg.seed)
        for it in range(self.cfg.max_pass):
            t0 = time.time()
            for b in orders[it].tolist():
                self.run_block(b)
            objv, nnz = self.evaluate()
            rel = 1.0 if not self.progress else self.progress[-1].objv / objv - 1.0
            p = Progress(objv, rel, nnz, 0.0, self.w.numel(), 0.0, time.time() - t0)
            self.progress.append(p)
            if verbose and self.group.rank == 0:
                print_progress(it, p, file=sys.stderr)
            if 0 < rel <= self.cfg.epsilon:
                break
        return self.progress

    def model(self):
        """This rank's share of the non-zero weights (the key range split evenly), ascending keys."""
        P, W, r = self.w.numel(), self.group.world, self.group.rank
        lo, hi = P * r // W, P * (r + 1) // W
        w = self.w[lo:hi]
        nz = w != 0
        keys = (self.gkeys[lo:hi][nz] ^ _SIGN).cpu().numpy().view(np.uint64)
        return keys, w[nz].cpu().numpy()

    def save_model(self, file_prefix: str) -> str:
        from ..utils.modelio import write_model_text

        k, w = self.model()
        path = f"{file_prefix}_S{self.group.rank}"
        write_model_text(path, k, w)
        return path
