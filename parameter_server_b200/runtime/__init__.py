"""Host runtime: loads the native module ``_psb_host`` (built in-tree under ``lib/``)."""
from __future__ import annotations

import importlib.util
import sys

from ..utils import build as _build

_mod = None


def host():
    """The pybind11 module with the control plane, data ingest and host containers."""
    global _mod
    if _mod is None:
        path = _build.build_host()      # returns at once when the module matches its sources
        spec = importlib.util.spec_from_file_location("_psb_host", str(path))
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
        sys.modules["_psb_host"] = _mod
    return _mod
