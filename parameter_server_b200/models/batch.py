"""Plain batch solver: block proximal-gradient / gradient-descent learners over the loss and
penalty families, for jobs whose ``.conf`` has no ``darling{}`` section.

The reference ships this path half-finished — ``BatchSolver::updateModel`` is commented out and the
``learner/`` classes do not compile — but documents the intent: per feature block, aggregate the
gradient and the diagonal Hessian over the workers and let the learner update the block's weights
(src/linear_method/learner/proximal_gradient.h:20-53, gradient_descent.h:19-24,
src/linear_method/loss.h:73-104, src/linear_method/penalty.h:15-50,
src/test/aggregated_gradient_test.cc:52-104).  Here it is implemented: rows are sharded over the
ranks, every rank keeps the whole weight vector, the per-block work runs in the kernels of
``csrc/batch_kernels.cu`` (block gradient and curvature for the logistic and the square hinge loss,
learner update, margin update; preprocessing with the sort / unique / remap / bucket kernels of
``ops.sparse``), and the block's (G,U) sums of the ranks are added with an NCCL all-reduce — this
solver is the simple replicated-weights counterpart of DARLIN, whose pass kernel carries the
product path over peer memory.
"""
from __future__ import annotations

import ctypes as C
import math
import sys
import time
from typing import List

import numpy as np
import torch

from ..ops import _native as N
from ..ops import sparse
from ..ops.reduce import reduce_sum
from ..parallel.peer import PeerGroup
from .darlin import DarlinConfig, Progress, block_order, print_progress

_SIGN = -(1 << 63)
LOSS_KIND = {"LOGIT": 0, "SQUARE_HINGE": 1}
LEARNER_KIND = {"PROXIMAL_GRADIENT": 0, "GRADIENT_DESCENT": 1}


class BatchShard(C.Structure):
    _fields_ = [("col_ptr", C.c_void_p), ("row_idx", C.c_void_p), ("vals", C.c_void_p), ("col_of", C.c_void_p),
                ("ym", C.c_void_p)]


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
        self.loss_name, self.penalty = loss, Penalty.create(penalty, cfg.lambda1)
        self.learner = learner
        self.progress: List[Progress] = []
        self._lib = N.lib()
        self.kernel_launches = 0

    def preprocess(self, offsets, keys, vals, y) -> None:
        import torch.distributed as dist

        g, dev = self.group, self.dev
        lkeys, _ = sparse.count_unique(keys.contiguous())          # this rank's unique keys, unsigned order
        uk = lkeys
        if g.world > 1:
            sizes = [None] * g.world
            dist.all_gather_object(sizes, int(lkeys.numel()), group=g.group)
            pad = torch.full((max(sizes),), -1, dtype=torch.int64, device=dev)
            pad[: lkeys.numel()] = lkeys
            parts = [torch.empty_like(pad) for _ in range(g.world)]
            dist.all_gather(parts, pad, group=g.group)
            uk = sparse.set_union_many([p[:n] for p, n in zip(parts, sizes)])                # union of all ranks' keys
        self.gkeys = uk ^ _SIGN              # ordered (sign-flipped) global keys
        P, rows = uk.numel(), y.numel()
        col = sparse.remap(keys.contiguous(), uk)                  # global column of every non-zero
        self.col_ptr, self.row_idx, self.val = sparse.csr_to_csc(offsets, col, vals, P)
        self.col_of = torch.repeat_interleave(torch.arange(P, dtype=torch.int32, device=dev),
                                              self.col_ptr[1:] - self.col_ptr[:-1]).contiguous()
        self.ym = torch.stack([y.to(torch.float32), torch.zeros(rows, dtype=torch.float32, device=dev)], 1).contiguous()
        self.margin = self.ym[:, 1]
        self.w = torch.zeros(P, device=dev)
        self._D = BatchShard(self.col_ptr.data_ptr(), self.row_idx.data_ptr(), 0 if self.val is None else self.val.data_ptr(),
                             self.col_of.data_ptr(), self.ym.data_ptr())
        tot = g.all_reduce_sum([rows, keys.numel()])
        self.total_rows = int(tot[0])
        per_row = tot[1] / max(tot[0], 1)
        r = self.cfg.feature_block_ratio
        self.nblk = max(int(math.ceil(per_row * r)), 1) if (per_row > 1 + 1e-6 and r > 0) else 1
        kmin, kmax = int(self.gkeys[0].item()) - _SIGN, int(self.gkeys[-1].item()) - _SIGN + 1
        bounds = [kmin + (kmax - kmin) * i // self.nblk for i in range(self.nblk)] + [kmax]
        b = torch.tensor([min(x, (1 << 64) - 1) + _SIGN for x in bounds], dtype=torch.int64, device=dev)
        c = torch.searchsorted(self.gkeys, b)
        c[-1] = P
        self.blk = c.tolist()
        self.blk_nnz = self.col_ptr[c].tolist()
        widest = max((self.blk[i + 1] - self.blk[i] for i in range(self.nblk)), default=1)
        self._gu = torch.zeros((max(widest, 1), 2), dtype=torch.float32, device=dev)
        self._d = torch.zeros((max(widest, 1),), dtype=torch.float32, device=dev)

    def run_block(self, b: int) -> None:
        c0, c1 = self.blk[b], self.blk[b + 1]
        if c1 <= c0:
            return
        lib, s = self._lib, N.stream_ptr()
        nnz_b = self.blk_nnz[b + 1] - self.blk_nnz[b]
        gu = self._gu[: c1 - c0]
        gu.zero_()
        if nnz_b:
            N.check(lib.psb_batch_block_grad(C.byref(self._D), LOSS_KIND[self.loss_name], C.c_int64(c0), C.c_int64(c1), N.ptr(gu),
                                             C.c_int64(nnz_b), s), "batch_block_grad")
        if self.group.world > 1:
            import torch.distributed as dist

            dist.all_reduce(gu, group=self.group.group)
        N.check(lib.psb_batch_block_update(N.ptr(gu), N.ptr(self.w[c0:c1]), N.ptr(self._d), C.c_int64(c1 - c0),
                                           LEARNER_KIND[self.learner], self.penalty.p, C.c_float(self.cfg.eta),
                                           C.c_float(self.cfg.lambda1), s), "batch_block_update")
        if nnz_b:
            N.check(lib.psb_batch_block_margin(C.byref(self._D), C.c_int64(c0), C.c_int64(c1), N.ptr(self._d), C.c_int64(nnz_b), s),
                    "batch_block_margin")
        self.kernel_launches += 3 if nnz_b else 1

    def evaluate(self):
        op = "sum_logistic" if self.loss_name == "LOGIT" else "sum_square_hinge"
        loss = reduce_sum(self.margin.contiguous(), op).clone()
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
