"""AUC on the device (``csrc/eval_kernels.cu`` + the sort / unique kernels of ``ops.sparse``).

``auc_histogram`` is the worker side of the reference's binned AUC (src/base/auc.h:69-98): per class, the
occupied bins ``(int64)(p * goodness)`` and their counts, ready to be merged over ranks
(``AUC.merge_data`` of the host runtime).  ``exact_auc`` is ``Evaluation::auc``
(src/base/evaluation.h:18-44): sort by score, count for every negative the positives before it.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _native as N
from . import sparse

_SIGN = -(1 << 63)


def auc_histogram(label: torch.Tensor, pred: torch.Tensor, goodness: int = 100000) -> Tuple[list, list, list, list]:
    """(tp_keys, tp_counts, fp_keys, fp_counts): occupied bins in ascending order with their counts."""
    n, dev = pred.numel(), pred.device
    label, pred = label.to(torch.float32).contiguous(), pred.to(torch.float32).contiguous()
    pos = torch.empty(n, dtype=torch.int64, device=dev)
    neg = torch.empty(n, dtype=torch.int64, device=dev)
    N.check(N.lib().psb_auc_bin_keys(N.ptr(label), N.ptr(pred), C.c_size_t(n), C.c_longlong(int(goodness)), N.ptr(pos), N.ptr(neg),
                                     N.stream_ptr()), "auc_bin_keys")
    out = []
    for keys in (pos, neg):
        uk, cnt = sparse.count_unique(keys)
        keep = uk != -1                      # the other class's placeholder
        out += [(uk[keep] ^ _SIGN).tolist(), cnt[keep].tolist()]
    return tuple(out)


def exact_auc(label: torch.Tensor, pred: torch.Tensor) -> float:
    """Area under the ROC curve from the scores sorted ascending; equal scores share their rank."""
    n, dev = pred.numel(), pred.device
    if n == 0:
        return 0.5
    label, pred = label.to(torch.float32).contiguous(), pred.to(torch.float32).contiguous()
    lib = N.lib()
    keys = torch.empty(n, dtype=torch.int64, device=dev)
    flag = torch.empty(n, dtype=torch.int32, device=dev)
    N.check(lib.psb_score_keys(N.ptr(pred), C.c_size_t(n), N.ptr(keys), N.stream_ptr()), "score_keys")
    N.check(lib.psb_label_flags(N.ptr(label), C.c_size_t(n), N.ptr(flag), N.stream_ptr()), "label_flags")
    skeys, sflag = sparse.sort_pairs(keys, flag)
    before, total = sparse.exclusive_scan(sflag)            # positives that sort before every position
    _, counts = sparse.unique_sorted(skeys)                 # runs of equal scores
    start, _ = sparse.exclusive_scan(counts)
    area = torch.zeros(1, dtype=torch.float64, device=dev)
    N.check(lib.psb_auc_area(N.ptr(start), N.ptr(counts), C.c_size_t(counts.numel()), N.ptr(before), C.c_size_t(n), N.ptr(total),
                             N.ptr(area), N.stream_ptr()), "auc_area")
    tp = float(total.item())
    fp = n - tp
    if tp == 0 or fp == 0:
        return 0.5
    # the kernel counts, for every negative, the positives that score LOWER: the complement of the AUC
    return 1.0 - float(area.item()) / (tp * fp)
