"""Deterministic device sum reductions (objective values and statistics)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N

OPS = {"sum_log1p_inv": 0, "sum_abs": 1, "count_nonzero": 2, "sum_logistic": 3, "sum_square_hinge": 4}
_scratch = {}


def _scratch_for(dev: torch.device) -> torch.Tensor:
    key = (dev.type, dev.index)
    if key not in _scratch:
        lib = N.lib()
        lib.psb_reduce_scratch_bytes.restype = C.c_size_t
        _scratch[key] = torch.zeros(lib.psb_reduce_scratch_bytes(), dtype=torch.uint8, device=dev)
    return _scratch[key]


def reduce_sum(x: torch.Tensor, op: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """Σ term(x_i) in fp64 on the device; ``op`` is one of ``OPS``. Returns a 1-element float64 tensor."""
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
    if out is None:
        out = torch.empty((1,), dtype=torch.float64, device=x.device)
    sc = _scratch_for(x.device)
    N.check(N.lib().psb_reduce_sum(N.ptr(x), C.c_size_t(x.numel()), OPS[op], N.ptr(sc), C.c_size_t(sc.numel()),
                                   N.ptr(out), N.stream_ptr()), "reduce_sum")
    return out
