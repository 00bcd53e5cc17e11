"""ctypes binding of ``libpsb_kernels.so`` (the sm_100a kernels, C ABI).

The library is built in-tree by :mod:`parameter_server_b200.utils.build`; it is
loaded lazily so that CPU-only code paths (config parsing, the host runtime, the
fp64 oracle) import without CUDA.  On a machine with a GPU a missing library is
an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from ..utils import build as _build

MAX_RANKS = 8
EMPTY_KEY = 0xFFFFFFFFFFFFFFFF

_lib = None
_lock = threading.Lock()

STATUS_NAMES = {
    0: "ok",
    1: "bounded cross-GPU wait timed out",
    2: "per-minibatch dedup table full",
    3: "shard hash table full (probe limit)",
    4: "inbox overflow",
    5: "index out of bounds (skipped)",
}


class KeySeps(C.Structure):
    _fields_ = [("sep", C.c_uint64 * (MAX_RANKS + 1)), ("world", C.c_int)]


class FtrlHyper(C.Structure):
    _fields_ = [("alpha", C.c_float), ("beta", C.c_float), ("l1", C.c_float), ("l2", C.c_float),
                ("rule", C.c_int), ("pad", C.c_int),
                ("cm", C.c_void_p), ("cm_width", C.c_uint32), ("cm_k", C.c_int), ("tail_freq", C.c_uint32),
                ("pad2", C.c_uint32)]


_P8 = C.c_void_p * MAX_RANKS


class FtrlPeers(C.Structure):
    _fields_ = [("seps", KeySeps), ("rank", C.c_int), ("max_probe", C.c_int), ("tab_mask", C.c_uint64),
                ("tab", C.c_void_p), ("lt_keys", _P8), ("lt_w", _P8), ("lt_acc", _P8),
                ("ready", _P8), ("replied", _P8), ("grads", _P8), ("in_slot", C.c_void_p), ("in_keys", C.c_void_p),
                ("timeout_ns", C.c_uint64), ("tab_shift", C.c_uint32), ("region_log2", C.c_uint32)]


class Minibatch(C.Structure):
    _fields_ = [("offsets", C.c_void_p), ("keys", C.c_void_p), ("vals", C.c_void_p), ("y", C.c_void_p),
                ("nnz", C.c_int64), ("rows", C.c_int), ("off32", C.c_uint16), ("key_mode", C.c_uint16)]


class LocalScratch(C.Structure):
    _fields_ = [("lt_keys", C.c_void_p), ("lt_w", C.c_void_p), ("lt_acc", C.c_void_p), ("lt_slots", C.c_uint64),
                ("slot_of", C.c_void_p), ("coef", C.c_void_p), ("xw", C.c_void_p),
                ("send_cnt", C.c_void_p), ("recv_cnt", C.c_void_p), ("stats", C.c_void_p),
                ("status", C.c_void_p), ("trace", C.c_void_p), ("soa", C.c_uint32), ("parity", C.c_uint32)]


def lib() -> C.CDLL:
    """Load (building first if needed) the kernel library.  ``PSB_KERNELS_LIB`` names an alternative
    build of the same sources (for instance one compiled with other ``-D`` switches)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                override = os.environ.get("PSB_KERNELS_LIB")
                if override:
                    _lib = C.CDLL(override)
                else:
                    # returns at once when the library matches its sources (digest stamp beside it)
                    _lib = C.CDLL(str(_build.build_kernels()))
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: CUDA error {code}")


def stream_ptr() -> C.c_void_p:
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


# ------------------------------------------------------------------ DARLIN structs
class DarlinWorker(C.Structure):
    _fields_ = [("col_ptr", C.c_void_p), ("row_idx", C.c_void_p), ("vals", C.c_void_p), ("ym", C.c_void_p),
                ("col_of", C.c_void_p), ("w", C.c_void_p), ("delta", C.c_void_p), ("active", C.c_void_p),
                ("gslot", C.c_void_p), ("gowner", C.c_void_p), ("dw", C.c_void_p), ("cols", C.c_int64),
                ("rows", C.c_int), ("pad", C.c_int), ("gcol", C.c_void_p)]


class DarlinPeers(C.Structure):
    _fields_ = [("w", _P8), ("gu", _P8), ("arrive", _P8), ("rank", C.c_int), ("world", C.c_int),
                ("timeout_ns", C.c_uint64), ("gu_stride", C.c_int64), ("part", _P8), ("mine", C.c_void_p),
                ("colgu", _P8), ("colslot", _P8), ("coldw", _P8), ("arrive2", _P8)]


class DarlinServer(C.Structure):
    _fields_ = [("delta", C.c_void_p), ("active", C.c_void_p), ("violation", C.c_void_p), ("slots", C.c_int64),
                ("d_slot", C.c_void_p)]


class DarlinSched(C.Structure):
    _fields_ = [("order", C.c_void_p), ("blk_lc", C.c_void_p), ("blk_sl", C.c_void_p), ("nblk", C.c_int),
                ("group", C.c_int), ("seq0", C.c_uint64), ("local_bar", C.c_void_p), ("bar0", C.c_uint64),
                ("abort_flag", C.c_void_p), ("status", C.c_void_p), ("stage_base", C.c_void_p),
                ("prev", C.c_void_p), ("nprev", C.c_int), ("wide_cols", C.c_int),
                ("blk_gc", C.c_void_p), ("blk_gs0", C.c_void_p), ("gather", C.c_int), ("pad2", C.c_int),
                ("trace", C.c_void_p), ("all_cb", C.c_void_p), ("nblocks_total", C.c_int64),
                ("list_cols", C.c_int64)]


class DarlinHyper(C.Structure):
    _fields_ = [("lam", C.c_float), ("eta", C.c_float), ("delta_max", C.c_float), ("kkt_threshold", C.c_float)]
