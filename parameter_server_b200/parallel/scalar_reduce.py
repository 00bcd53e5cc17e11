"""All-reduce of a few scalars over the ranks of the box inside one small kernel
(``csrc/scalar_allreduce.cu``): sums in fp64, maxima of non-negative floats.

Role: the per-pass progress merge of the batch solvers (``LinearMethod::mergeProgress``,
src/linear_method/linear_method.cc:106-120) without a collective library.  Every rank writes its values
into its copy of a symmetric buffer and raises flags on its peers; with a multicast mapping of the buffer
(NVLink SHARP) the result is one ``multimem.ld_reduce`` per value — the switch adds the ranks' copies —
otherwise one peer load per rank and value.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence, Tuple

import torch

from ..ops import _native as N
from .peer import PeerGroup

_P8 = C.c_void_p * N.MAX_RANKS
MAX_SCALARS = 32


class ScalarPeers(C.Structure):
    _fields_ = [("sums", _P8), ("maxs", _P8), ("flags", _P8), ("mc_sums", C.c_void_p), ("mc_maxs", C.c_void_p),
                ("rank", C.c_int), ("world", C.c_int), ("timeout_ns", C.c_uint64)]


def _multicast_ptr(buf) -> int:
    """Multicast address of a symmetric buffer's data, 0 when the box has no multicast support."""
    hdl = buf.handle
    try:
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
    except Exception:
        return 0
    return mc


class ScalarAllReduce:
    def __init__(self, group: PeerGroup, timeout_s: float = 5.0, use_multicast: bool = True):
        self.group, self.dev, self.seq = group, group.device, 0
        self.sums = group.alloc((2, MAX_SCALARS), torch.float64)
        self.maxs = group.alloc((2, MAX_SCALARS), torch.int32)
        self.flags = group.alloc((N.MAX_RANKS,), torch.int64)
        self.status = torch.zeros(8, dtype=torch.int32, device=self.dev)
        P = ScalarPeers()
        for r in range(group.world):
            P.sums[r], P.maxs[r], P.flags[r] = self.sums.ptrs[r], self.maxs.ptrs[r], self.flags.ptrs[r]
        mc_s = _multicast_ptr(self.sums) if (use_multicast and group.world > 1) else 0
        mc_m = _multicast_ptr(self.maxs) if (use_multicast and group.world > 1) else 0
        self.multicast = bool(mc_s and mc_m)
        P.mc_sums = mc_s if self.multicast else None
        P.mc_maxs = mc_m if self.multicast else None
        P.rank, P.world, P.timeout_ns = group.rank, group.world, int(timeout_s * 1e9)
        self._P = P
        self._out_sum = torch.zeros(MAX_SCALARS, dtype=torch.float64, device=self.dev)
        self._out_max = torch.zeros(MAX_SCALARS, dtype=torch.float32, device=self.dev)
        group.barrier()

    def __call__(self, sums: torch.Tensor, maxs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``sums``: float64 values to add over the ranks; ``maxs``: non-negative float32 values whose maximum is
        taken.  Returns device tensors (views of internal buffers, valid until the next call).  Collective."""
        ns, nm = sums.numel(), maxs.numel()
        if ns > MAX_SCALARS or nm > MAX_SCALARS:
            raise ValueError(f"at most {MAX_SCALARS} scalars per call")
        self.seq += 1
        N.check(N.lib().psb_scalar_allreduce(C.byref(self._P), N.ptr(sums.contiguous()), ns, N.ptr(maxs.contiguous()), nm,
                                             C.c_uint64(self.seq), N.ptr(self._out_sum), N.ptr(self._out_max), N.ptr(self.status),
                                             N.stream_ptr()), "scalar_allreduce")
        return self._out_sum[:ns], self._out_max[:nm]

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"rank {self.group.rank}: scalar all-reduce: {N.STATUS_NAMES.get(st[0], st[0])} (peer={st[1]})")
