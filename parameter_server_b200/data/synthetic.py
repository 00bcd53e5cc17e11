"""Synthetic sparse data sets of the benchmark shapes (generated with torch on any device).

* :func:`ctr_minibatch` — CTR-scale stream: hashed uint64 keys over a 2^30-key space with
  Zipf(1.1) popularity, 12 feature groups with ~8 binary features each (~100 nnz/row), labels
  Bernoulli(sigmoid(X·w* − 3.2)) with a planted w* ~ N(0, 0.5) on 1 % of the keys.
* :func:`zipf_sparse_matrix` — batch L1-LR data: Zipf column ids, optional lognormal values with
  row L2 normalisation, labels from a planted sparse w*.

Keys are returned as int64 tensors holding uint64 bit patterns.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

_M1 = -4658895280553007687   # 0xbf58476d1ce4e5b9 as int64
_M2 = -7723592293110705685   # 0x94d049bb133111eb as int64


def _lsr(x: torch.Tensor, k: int) -> torch.Tensor:
    return (x >> k) & ((1 << (64 - k)) - 1)


def mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on int64 bit patterns (bijective on 64 bits)."""
    x = x ^ _lsr(x, 30)
    x = x * _M1
    x = x ^ _lsr(x, 27)
    x = x * _M2
    return x ^ _lsr(x, 31)


def zipf_ranks(n: int, s: float, vocab: int, gen: torch.Generator, device) -> torch.Tensor:
    """n draws of a rank in [0, vocab) with P(k) ∝ (k+1)^-s (bounded-Pareto inverse CDF)."""
    u = torch.rand(n, generator=gen, device=device, dtype=torch.float64)
    if abs(s - 1.0) < 1e-9:
        k = torch.exp(u * math.log(vocab + 1.0))
    else:
        a = 1.0 - s
        k = (u * ((vocab + 1.0) ** a - 1.0) + 1.0) ** (1.0 / a)
    return (k.floor().to(torch.int64) - 1).clamp_(0, vocab - 1)


def planted_weight(keys: torch.Tensor, frac: float, std: float, salt: int = 0x5EED) -> torch.Tensor:
    """Deterministic sparse w*(key): non-zero for ~frac of the keys, N(0, std²) there (float32)."""
    h = mix64(keys ^ salt)
    sel = (_lsr(h, 40) % 1000003).to(torch.float64) < frac * 1000003
    u1 = ((_lsr(h, 11) & 0xFFFFF).to(torch.float64) + 1.0) / (0x100000 + 1.0)
    u2 = (_lsr(mix64(h), 11) & 0xFFFFF).to(torch.float64) / 0x100000
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2 * math.pi * u2)
    return torch.where(sel, z * std, torch.zeros_like(z)).to(torch.float32)


def ctr_minibatch(rows: int, *, seed: int, device, key_space_log2: int = 30, zipf_s: float = 1.1, groups: int = 12,
                  feats_lo: int = 6, feats_hi: int = 10, bias: float = -3.2, wstar_frac: float = 0.01,
                  wstar_std: float = 0.5, return_ids: bool = False) -> Tuple[torch.Tensor, ...]:
    """One minibatch (offsets int64[rows+1], keys int64[nnz], y float32[rows] in ±1).  A key is the 64-bit mix
    of a feature id below 2^key_space_log2; with ``return_ids`` the ids come back too (int32[nnz], for the
    compact input encoding that hashes on the device)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    per_group = torch.randint(feats_lo, feats_hi + 1, (rows, groups), generator=gen, device=device)
    counts = per_group.sum(1)
    offsets = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    offsets[1:] = counts.cumsum(0)
    nnz = int(offsets[-1].item())
    vocab = (1 << key_space_log2) // groups
    ranks = zipf_ranks(nnz, zipf_s, vocab, gen, device)
    # group of each non-zero: expand per-row group counts
    grp = torch.repeat_interleave(torch.arange(groups, device=device).repeat(rows), per_group.reshape(-1))
    fid = ranks * groups + grp
    keys = mix64(fid)     # (a bijection: the reserved key 2^64-1 is the image of one id far above any key space here)
    wstar = planted_weight(keys, wstar_frac, wstar_std)
    row_of = torch.repeat_interleave(torch.arange(rows, device=device), counts)
    margin = torch.zeros(rows, dtype=torch.float32, device=device).index_add_(0, row_of, wstar) + bias
    y = torch.where(torch.rand(rows, generator=gen, device=device) < torch.sigmoid(margin), 1.0, -1.0)
    if return_ids:
        return offsets, keys, y.to(torch.float32), fid.to(torch.int32)
    return offsets, keys, y.to(torch.float32)


def zipf_sparse_matrix(rows: int, cols: int, nnz_per_row: int, *, seed: int, device, zipf_s: float = 1.0,
                       binary: bool = False, wstar_frac: float = 0.02, noise: float = 0.3,
                       uniform_keys: bool = False, logistic_labels: bool = False, wstar_seed: Optional[int] = None):
    """CSR (offsets, col ids int64, vals float32|None, y ±1 float32, w* float32[cols]) for batch L1-LR.

    Column ids are distinct within a row.  Values (unless ``binary``) are lognormal(0,1) with each
    row scaled to unit L2 norm.  Labels are sign(X·w* + N(0, noise)) or, with ``logistic_labels``,
    Bernoulli(sigmoid(X·w*)).
    """
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    n = rows * nnz_per_row
    if uniform_keys:
        col = torch.randint(0, cols, (n,), generator=gen, device=device)
    else:
        col = zipf_ranks(n, zipf_s, cols, gen, device)
    col = col.view(rows, nnz_per_row).sort(1).values
    keep = torch.ones_like(col, dtype=torch.bool)
    keep[:, 1:] = col[:, 1:] != col[:, :-1]
    counts = keep.sum(1)
    offsets = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    offsets[1:] = counts.cumsum(0)
    idx = col[keep]
    row_of = torch.repeat_interleave(torch.arange(rows, device=device), counts)
    if binary:
        vals = None
        v = torch.ones(idx.numel(), dtype=torch.float32, device=device)
    else:
        v = torch.exp(torch.randn(idx.numel(), generator=gen, device=device))
        nrm = torch.zeros(rows, device=device).index_add_(0, row_of, v * v).sqrt_().clamp_min_(1e-12)
        v = (v / nrm[row_of]).to(torch.float32)
        vals = v
    wgen = gen
    if wstar_seed is not None:            # the same planted model on every rank, whatever the data seed
        wgen = torch.Generator(device=device)
        wgen.manual_seed(wstar_seed)
    wstar = torch.randn(cols, generator=wgen, device=device)
    wstar = torch.where(torch.rand(cols, generator=wgen, device=device) < wstar_frac, wstar, torch.zeros_like(wstar))
    xw = torch.zeros(rows, device=device).index_add_(0, row_of, v * wstar[idx])
    if logistic_labels:
        y = torch.where(torch.rand(rows, generator=gen, device=device) < torch.sigmoid(xw), 1.0, -1.0)
    else:
        y = torch.sign(xw + noise * torch.randn(rows, generator=gen, device=device))
        y = torch.where(y == 0, torch.ones_like(y), y)
    return offsets, idx, vals, y.to(torch.float32), wstar.to(torch.float32)


def write_libsvm_parts(directory: str, offsets, idx, vals, y, num_files: int, one_based: bool = False) -> list:
    """Write a CSR matrix as ``num_files`` LIBSVM text parts (``part-000`` ...); returns the paths."""
    import os

    import numpy as np

    os.makedirs(directory, exist_ok=True)
    off = offsets.cpu().numpy()
    ix = idx.cpu().numpy().astype(np.uint64) + (1 if one_based else 0)
    v = None if vals is None else vals.cpu().numpy()
    yy = y.cpu().numpy()
    rows = len(yy)
    paths = []
    for f in range(num_files):
        r0, r1 = rows * f // num_files, rows * (f + 1) // num_files
        path = os.path.join(directory, f"part-{f:03d}")
        with open(path, "w") as out:
            for r in range(r0, r1):
                a, b = off[r], off[r + 1]
                feats = " ".join(f"{int(k)}:{(1 if v is None else float(v[i])):g}" for k, i in zip(ix[a:b], range(a, b)))
                out.write(f"{int(yy[r]):+d} {feats}\n")
        paths.append(path)
    return paths
