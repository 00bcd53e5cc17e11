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
        from ..ops.evalops import auc_histogram

        y_all, p_all = y.cpu().numpy(), xw.cpu().numpy()
        auc.merge_data(*auc_histogram(y, xw))                    # binned on the device (the host class's default bin width)
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


class ModelEvaluationNode:
    """The evaluation app on CPU nodes (src/linear_method/model_evaluation.h:15-67).  Like the reference's it is a
    single-node program: the scheduler loads the model, streams the validation files in minibatches, predicts, writes
    the labels and predictions when ``model_output`` is set, and prints the AUC; the other nodes have nothing to do."""

    def __init__(self, ctx, app_conf, flags):
        self.ctx, self.app_conf, self.flags = ctx, app_conf, flags
        self.cust = host().Customer(ctx.po, app_conf.app_name, None, False)
        self.result: dict = {}

    def run(self, verbose: bool = True):
        from ..utils.modelio import lookup_model

        H, lm = host(), self.app_conf.linear_method
        files = H.search_files(cfg.data_files(lm.model_input, H)) or cfg.data_files(lm.model_input, H)
        mk, mw = model_arrays(read_model_text(*files))
        vd = lm.validation_data
        vfiles = H.search_files(cfg.data_files(vd, H))
        if not vfiles:
            raise FileNotFoundError(f"no validation file matches {list(vd.file)}")
        reader = H.StreamReader()
        reader.init(vfiles, getattr(H.TextFormat, vd.text if vd.has("text") else "LIBSVM"), True, bool(self.flags.shuffle_fea_id))
        auc = H.AUC()
        auc.set_goodness(int(lm.solver.auc_goodness))
        labels, preds = [], []
        while True:
            out = reader.read(100000)
            if out is None:
                break
            slots, info = out
            rows = info["num_ex"]
            y = np.where(slots[0]["value"] > 0, 1.0, -1.0).astype(np.float32)
            xw = np.zeros(rows)
            for sid, sl in slots.items():          # every feature slot contributes
                if sid == 0 or len(sl["index"]) == 0:
                    continue
                w = lookup_model(mk, mw, sl["index"])
                if len(sl["value"]):
                    w = w * sl["value"]
                row_of = np.repeat(np.arange(rows), np.diff(sl["offset"].astype(np.int64)))
                xw += np.bincount(row_of, weights=w, minlength=rows)
            auc.add(y, xw.astype(np.float32))
            labels.append(y)
            preds.append(xw.astype(np.float32))
        y_all = np.concatenate(labels) if labels else np.zeros(0, np.float32)
        p_all = np.concatenate(preds) if preds else np.zeros(0, np.float32)
        self.result = {"auc": auc.evaluate(), "exact_auc": H.exact_auc(y_all, p_all) if len(y_all) else 0.0,
                       "accuracy": auc.accuracy(0.0), "model_nnz": int(len(mk)), "examples": int(len(y_all))}
        if lm.model_output.file:
            y_all.tofile(f"{lm.model_output.file[0]}_L")
            p_all.tofile(f"{lm.model_output.file[0]}_P")
        if verbose:
            print(f"model with {self.result['model_nnz']} weights, {self.result['examples']} examples: "
                  f"auc {self.result['auc']:.6f} accuracy {self.result['accuracy']:.6f}", file=sys.stderr)
        return [self.result]

    def stop(self) -> None:
        self.cust.stop()
