"""Model evaluation app: load ``key weight`` model files, predict on validation data, report AUC
and accuracy, optionally write the labels and predictions.

Reference: ModelEvaluation::run (src/linear_method/model_evaluation.h:15-67).  The reference is
single-node; here every rank scores its share of the validation files and the AUC histograms are
merged.
"""
from __future__ import annotations

import sys

import numpy as np

from .. import config as cfg
from ..runtime import host
from ..utils.modelio import model_arrays, read_model_text


def evaluate_model(lm, flags, group) -> dict:
    from .gpu_job import _my_files, load_csr, predict_csr

    H = host()
    files = H.search_files(cfg.data_files(lm.model_input, H)) or cfg.data_files(lm.model_input, H)
    mk, mw = model_arrays(read_model_text(*files))
    cache = (lm.local_cache.file[0] if lm.local_cache.file else "/tmp/psb200_cache/") + f"eval{group.rank}/"
    vfiles = _my_files(lm.validation_data, group, 0)
    auc = H.AUC()
    y_all, p_all = np.zeros(0, np.float32), np.zeros(0, np.float32)
    if vfiles:
        off, keys, vals, y, _ = load_csr(lm.validation_data, vfiles, flags, cache, group.device)
        xw = predict_csr(off, keys, vals, mk, mw)
        y_all, p_all = y.cpu().numpy(), xw.cpu().numpy()
        auc.add(y_all, p_all)
    if group.world > 1:
        import torch.distributed as dist

        parts = [None] * group.world
        dist.all_gather_object(parts, auc.data(), group=group.group)
        auc = H.AUC()
        for p in parts:
            auc.merge_data(*p)
    out = {"auc": auc.evaluate(), "accuracy": auc.accuracy(0.0), "model_nnz": int(len(mk)), "examples": int(len(y_all))}
    if lm.model_output.file:
        # labels and predictions of this rank, like the reference's "L" / "P" outputs
        y_all.tofile(f"{lm.model_output.file[0]}_L_{group.rank}")
        p_all.tofile(f"{lm.model_output.file[0]}_P_{group.rank}")
    if group.rank == 0:
        print(f"model with {out['model_nnz']} weights: auc {out['auc']:.6f} accuracy {out['accuracy']:.6f}", file=sys.stderr)
    return out
