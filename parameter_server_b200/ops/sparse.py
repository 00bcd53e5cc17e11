"""Device operators on key sets and sparse matrices (``csrc/sparse_kernels.cu``).

Keys are uint64 bit patterns stored in int64 tensors; every ordering here is the *unsigned* order,
as in the reference (``Key = uint64``, src/util/common.h).  The functions mirror
``Localizer::countUniqIndex`` / ``remapIndex`` (src/base/localizer.h:50-168),
``SparseMatrix::alterStorage`` (src/base/sparse_matrix.h:186-241), ``kv_partition``
(src/util/kv_partition.h), ``CountMin`` / ``FreqencyFilter`` (src/base/countmin.h,
src/parameter/frequency_filter.h) and the sorted-set helpers of ``SArray``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _native as N

_L = None


def _lib():
    global _L
    if _L is None:
        _L = N.lib()
        _L.psb_sort_tile.restype = C.c_size_t
        _L.psb_scan_tile.restype = C.c_size_t
    return _L


def _sz(n: int) -> C.c_size_t:
    return C.c_size_t(int(n))


def exclusive_scan(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exclusive prefix sum of an int32/uint32 tensor → (int64 prefix, 1-element int64 total)."""
    lib, n = _lib(), x.numel()
    out = torch.empty(n, dtype=torch.int64, device=x.device)
    tiles = torch.empty(max((n + lib.psb_scan_tile() - 1) // lib.psb_scan_tile(), 1), dtype=torch.int64, device=x.device)
    total = torch.zeros(1, dtype=torch.int64, device=x.device)
    N.check(lib.psb_exclusive_scan_u32(N.ptr(x), N.ptr(out), _sz(n), N.ptr(tiles), N.ptr(total), N.stream_ptr()), "exclusive_scan")
    return out, total


def sort_pairs(keys: torch.Tensor, vals: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Stable LSD radix sort of uint64 keys (unsigned order) with an optional int32 payload.
    Bytes that are equal in all keys are skipped (one 8-histogram pass decides)."""
    lib, n, dev = _lib(), keys.numel(), keys.device
    assert keys.dtype == torch.int64 and keys.is_contiguous()
    if n == 0:
        return keys.clone(), None if vals is None else vals.clone()
    hist = torch.zeros(8 * 256, dtype=torch.int64, device=dev)
    N.check(lib.psb_digit_histograms(N.ptr(keys), _sz(n), N.ptr(hist), N.stream_ptr()), "digit_histograms")
    need = ((hist.view(8, 256) > 0).sum(1) > 1).tolist()
    nblocks = (n + lib.psb_sort_tile() - 1) // lib.psb_sort_tile()
    block_hist = torch.empty(256 * nblocks, dtype=torch.int32, device=dev)
    block_off = torch.empty(256 * nblocks, dtype=torch.int64, device=dev)
    tile_sum = torch.empty((256 * nblocks + lib.psb_scan_tile() - 1) // lib.psb_scan_tile(), dtype=torch.int64, device=dev)
    total = torch.empty(1, dtype=torch.int64, device=dev)
    # ping-pong between two scratch buffers; the caller's tensors are only ever read
    kbuf = [torch.empty_like(keys), None]
    vbuf = [None if vals is None else torch.empty_like(vals), None]
    src_k, src_v, turn = keys, vals, 0
    for p in range(8):
        if not need[p]:
            continue
        if kbuf[turn] is None:
            kbuf[turn] = torch.empty_like(keys)
            vbuf[turn] = None if vals is None else torch.empty_like(vals)
        dst_k, dst_v = kbuf[turn], vbuf[turn]
        N.check(lib.psb_radix_pass(N.ptr(src_k), N.ptr(src_v), _sz(n), p, N.ptr(block_hist), N.ptr(block_off), N.ptr(tile_sum),
                                   N.ptr(total), N.ptr(dst_k), N.ptr(dst_v), N.stream_ptr()), "radix_pass")
        src_k, src_v, turn = dst_k, dst_v, 1 - turn
    if src_k is keys:
        return keys.clone(), None if vals is None else vals.clone()
    return src_k, src_v


def unique_sorted(sorted_keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Run-length encode a sorted key array → (unique keys, int32 counts)."""
    lib, n, dev = _lib(), sorted_keys.numel(), sorted_keys.device
    if n == 0:
        return sorted_keys.clone(), torch.zeros(0, dtype=torch.int32, device=dev)
    flag = torch.empty(n, dtype=torch.int32, device=dev)
    N.check(lib.psb_head_flags(N.ptr(sorted_keys), _sz(n), N.ptr(flag), N.stream_ptr()), "head_flags")
    pos, total = exclusive_scan(flag)
    nu = int(total.item())
    ukeys = torch.empty(nu, dtype=torch.int64, device=dev)
    ustart = torch.empty(nu, dtype=torch.int64, device=dev)
    N.check(lib.psb_write_unique(N.ptr(sorted_keys), N.ptr(flag), N.ptr(pos), _sz(n), N.ptr(ukeys), N.ptr(ustart), N.stream_ptr()), "write_unique")
    counts = torch.empty(nu, dtype=torch.int32, device=dev)
    N.check(lib.psb_counts_from_starts(N.ptr(ustart), _sz(nu), _sz(n), N.ptr(counts), N.stream_ptr()), "counts_from_starts")
    return ukeys, counts


def count_unique(keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unique keys in unsigned order with their frequencies (``Localizer::countUniqIndex``)."""
    sk, _ = sort_pairs(keys.contiguous())
    return unique_sorted(sk)


def remap(keys: torch.Tensor, dictionary: torch.Tensor) -> torch.Tensor:
    """Index of every key in the sorted ``dictionary`` as int32, -1 where absent (``Localizer::remapIndex``)."""
    out = torch.empty(keys.numel(), dtype=torch.int32, device=keys.device)
    N.check(_lib().psb_remap(N.ptr(keys), _sz(keys.numel()), N.ptr(dictionary), _sz(dictionary.numel()), N.ptr(out), N.stream_ptr()), "remap")
    return out


def bucket_order(bucket: torch.Tensor, nb: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group elements by bucket id: returns (bucket start offsets int64[nb+1], destination of every element
    int64, -1 for dropped ones with id >= nb).  Order inside a bucket is arrival order (not stable)."""
    lib, n, dev = _lib(), bucket.numel(), bucket.device
    hist = torch.zeros(nb, dtype=torch.int32, device=dev)
    N.check(lib.psb_bucket_hist(N.ptr(bucket), _sz(n), nb, N.ptr(hist), N.stream_ptr()), "bucket_hist")
    start, total = exclusive_scan(hist)
    cursor = torch.zeros(nb, dtype=torch.int32, device=dev)
    dest = torch.empty(n, dtype=torch.int64, device=dev)
    N.check(lib.psb_bucket_dest(N.ptr(bucket), _sz(n), nb, N.ptr(start), N.ptr(cursor), N.ptr(dest), N.stream_ptr()), "bucket_dest")
    return torch.cat([start, total]), dest


def csr_to_csc(offsets: torch.Tensor, col: torch.Tensor, vals: Optional[torch.Tensor], ncols: int):
    """Row-major → column-major storage (``SparseMatrix::alterStorage``): (col_ptr int64[ncols+1], row_idx int32, vals).
    Entries with a negative column id (dropped by a remap) are removed."""
    dev, rows = col.device, offsets.numel() - 1
    col_ptr, dest = bucket_order(col.to(torch.int32), ncols)
    row_of = torch.repeat_interleave(torch.arange(rows, device=dev, dtype=torch.int32), offsets[1:] - offsets[:-1])
    keep = dest >= 0
    nnz = int(col_ptr[-1].item())
    row_idx = torch.empty(nnz, dtype=torch.int32, device=dev)
    row_idx[dest[keep]] = row_of[keep]
    out_vals = None
    if vals is not None:
        out_vals = torch.empty(nnz, dtype=vals.dtype, device=dev)
        out_vals[dest[keep]] = vals[keep]
    return col_ptr, row_idx, out_vals


def partition_by_key_range(keys: torch.Tensor, vals: Optional[torch.Tensor], separators) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """k-way partition of (key, value) pairs by owner key range: (offsets int64[k+1], keys, values) with each
    owner's pairs contiguous (``kv_partition``; the routing step of a push)."""
    seps = N.KeySeps()
    k = len(separators) - 1
    for i, s in enumerate(separators):
        seps.sep[i] = int(s)
    for i in range(len(separators), N.MAX_RANKS + 1):
        seps.sep[i] = N.EMPTY_KEY
    seps.world = k
    bucket = torch.empty(keys.numel(), dtype=torch.int32, device=keys.device)
    N.check(_lib().psb_owner_of_keys(N.ptr(keys), _sz(keys.numel()), C.byref(seps), N.ptr(bucket), N.stream_ptr()), "owner_of_keys")
    start, dest = bucket_order(bucket, k)
    ok = torch.empty_like(keys)
    ok[dest] = keys
    ov = None
    if vals is not None:
        ov = torch.empty_like(vals)
        ov[dest] = vals
    return start, ok, ov


class CountMinDevice:
    """Count-min sketch on the device; ``wrap8`` reproduces the reference's wrapping uint8 counters."""

    def __init__(self, width: int, k: int, device, wrap8: bool = False):
        self.width, self.k, self.wrap = max(int(width), 64), max(int(k), 1), 0xFF if wrap8 else 0xFFFFFFFF
        self.table = torch.zeros(self.width, dtype=torch.int32, device=device)

    def insert(self, keys: torch.Tensor, counts: Optional[torch.Tensor] = None) -> None:
        N.check(_lib().psb_countmin_insert(N.ptr(keys), N.ptr(counts), _sz(keys.numel()), N.ptr(self.table), self.width, self.k, N.stream_ptr()), "countmin_insert")

    def query(self, keys: torch.Tensor) -> torch.Tensor:
        out = torch.empty(keys.numel(), dtype=torch.int32, device=keys.device)
        N.check(_lib().psb_countmin_query(N.ptr(keys), _sz(keys.numel()), N.ptr(self.table), self.width, self.k, C.c_uint32(self.wrap), N.ptr(out),
                                          N.stream_ptr()), "countmin_query")
        return out

    def filter(self, keys: torch.Tensor, freq: int) -> torch.Tensor:
        """Keys whose estimated count exceeds ``freq`` (``FreqencyFilter::queryKeys``), order preserved."""
        est = self.query(keys)
        flag = (est > freq).to(torch.int32)
        pos, total = exclusive_scan(flag)
        out = torch.empty(int(total.item()), dtype=torch.int64, device=keys.device)
        N.check(_lib().psb_compact_u64(N.ptr(keys), N.ptr(flag), N.ptr(pos), _sz(keys.numel()), N.ptr(out), N.stream_ptr()), "compact")
        return out


def set_intersection(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Keys of sorted unique ``a`` that also occur in sorted unique ``b``."""
    flag = torch.empty(a.numel(), dtype=torch.int32, device=a.device)
    N.check(_lib().psb_set_intersect_flags(N.ptr(a), _sz(a.numel()), N.ptr(b), _sz(b.numel()), N.ptr(flag), N.stream_ptr()), "intersect_flags")
    pos, total = exclusive_scan(flag)
    out = torch.empty(int(total.item()), dtype=torch.int64, device=a.device)
    N.check(_lib().psb_compact_u64(N.ptr(a), N.ptr(flag), N.ptr(pos), _sz(a.numel()), N.ptr(out), N.stream_ptr()), "compact")
    return out


def set_union(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Sorted union of two sorted unique key sets by ranking (no sort): ``SArray::setUnion``."""
    lib, na, nb, dev = _lib(), a.numel(), b.numel(), a.device
    if nb == 0:
        return a.clone()
    if na == 0:
        return b.clone()
    a, b = a.contiguous(), b.contiguous()
    dup = torch.empty(nb, dtype=torch.int32, device=dev)           # elements of b that a holds too
    N.check(lib.psb_set_intersect_flags(N.ptr(b), _sz(nb), N.ptr(a), _sz(na), N.ptr(dup), N.stream_ptr()), "intersect_flags")
    keep = torch.empty(nb, dtype=torch.int32, device=dev)
    N.check(lib.psb_invert_flags(N.ptr(dup), _sz(nb), N.ptr(keep), N.stream_ptr()), "invert_flags")
    pos, total = exclusive_scan(keep)                              # kept elements of b before every index
    out = torch.empty(na + int(total.item()), dtype=torch.int64, device=dev)
    N.check(lib.psb_merge_union(N.ptr(a), _sz(na), N.ptr(b), _sz(nb), N.ptr(dup), N.ptr(pos), N.ptr(out), N.stream_ptr()), "merge_union")
    return out


def set_union_many(parts) -> torch.Tensor:
    """Union of several sorted unique key sets (pairwise, smallest first)."""
    parts = sorted((p for p in parts if p.numel()), key=lambda t: t.numel())
    if not parts:
        return torch.zeros(0, dtype=torch.int64)
    while len(parts) > 1:
        parts = sorted([set_union(parts[0], parts[1])] + parts[2:], key=lambda t: t.numel())
    return parts[0]


def spmv(offsets: torch.Tensor, idx: torch.Tensor, vals: Optional[torch.Tensor], w: torch.Tensor) -> torch.Tensor:
    """y = X·w for CSR X with int32 local column ids (``SparseMatrix::times``, row-major)."""
    rows = offsets.numel() - 1
    y = torch.empty(rows, dtype=torch.float32, device=w.device)
    N.check(_lib().psb_spmv_csr(N.ptr(offsets), N.ptr(idx), N.ptr(vals), N.ptr(w), N.ptr(y), C.c_int64(rows), N.stream_ptr()), "spmv_csr")
    return y


def spmv_t(offsets: torch.Tensor, idx: torch.Tensor, vals: Optional[torch.Tensor], v: torch.Tensor, ncols: int) -> torch.Tensor:
    """out = Xᵀ·v for CSR X (``SparseMatrix::transTimes``)."""
    rows = offsets.numel() - 1
    out = torch.zeros(ncols, dtype=torch.float32, device=v.device)
    N.check(_lib().psb_spmv_t(N.ptr(offsets), N.ptr(idx), N.ptr(vals), N.ptr(v), N.ptr(out), C.c_int64(rows), N.stream_ptr()), "spmv_t")
    return out


def fill_gaussian(x: torch.Tensor, mean: float, std: float, seed: int) -> None:
    N.check(_lib().psb_fill_gaussian(N.ptr(x), _sz(x.numel()), C.c_float(mean), C.c_float(std), C.c_uint64(seed), N.stream_ptr()), "fill_gaussian")
