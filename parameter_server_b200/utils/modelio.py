"""Text model files: one ``key<TAB>weight`` line per non-zero weight.

Writer format follows BatchSolver::saveModel (src/linear_method/batch_solver.cc:407-422)
and FTRLModel::writeToFile (src/linear_method/ftrl_model.h:24-29): unsigned decimal key,
a tab, the weight in C++ ostream default formatting (``%g``, 6 significant digits); zeros
and NaNs are skipped.  The reader accepts any whitespace between key and value, as
ModelEvaluation does (src/linear_method/model_evaluation.h:20-27).
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Tuple

import numpy as np


def write_model_text(path: str, keys: Iterable[int], weights: Iterable[float]) -> int:
    n = 0
    with open(path, "w") as f:
        for k, w in zip(keys, weights):
            w = float(w)
            if w != 0.0 and not math.isnan(w):
                f.write(f"{int(k)}\t{w:g}\n")
                n += 1
    return n


def read_model_text(*paths: str) -> Dict[int, float]:
    model: Dict[int, float] = {}
    for p in paths:
        with open(p) as f:
            toks = f.read().split()
        for i in range(0, len(toks) - 1, 2):
            model[int(toks[i])] = float(toks[i + 1])
    return model


def model_arrays(model: Dict[int, float]) -> Tuple[np.ndarray, np.ndarray]:
    keys = np.fromiter(model.keys(), dtype=np.uint64, count=len(model))
    vals = np.fromiter(model.values(), dtype=np.float64, count=len(model))
    order = np.argsort(keys, kind="stable")
    return keys[order], vals[order]


def model_files(name: str) -> List[str]:
    """The files of a model given as one file or as the ``model_output`` prefix of an earlier job (``<name>_S0`` ...)."""
    import glob
    import os

    if os.path.isfile(name):
        return [name]
    return sorted(glob.glob(glob.escape(name) + "_*"))


def lookup_model(mkeys: np.ndarray, mvals: np.ndarray, keys: np.ndarray) -> np.ndarray:
    """Weights of ``keys`` (uint64) in a model given as ascending ``mkeys`` (uint64) and ``mvals``; 0 where absent."""
    keys = np.asarray(keys, dtype=np.uint64)
    out = np.zeros(len(keys), dtype=np.float64)
    if len(mkeys) and len(keys):
        pos = np.clip(np.searchsorted(mkeys, keys), 0, len(mkeys) - 1)
        hit = mkeys[pos] == keys
        out[hit] = mvals[pos[hit]]
    return out
