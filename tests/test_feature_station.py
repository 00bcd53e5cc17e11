"""Worker-side feature store: memory and disk mode give the same column ranges; prefetch threads read ahead
under a memory limit; the native block steps run on a range that was loaded on its own."""
import os
import time

import numpy as np
import pytest
import scipy.sparse as sp

from parameter_server_b200.runtime.node import host


def _matrix(rows=400, cols=300, density=0.05, seed=0, binary=False):
    rng = np.random.default_rng(seed)
    X = sp.random(rows, cols, density=density, format="csc", random_state=seed, dtype=np.float64)
    X.sort_indices()
    if binary:
        X.data[:] = 1.0
    y = np.where(rng.random(rows) < 0.5, -1.0, 1.0)
    return X, y


def _add(st, X, binary):
    st.add_group(1, X.shape[0], X.indptr.astype(np.int64), X.indices.astype(np.int32), None if binary else X.data)


@pytest.mark.parametrize("binary", [False, True])
def test_disk_ranges_equal_memory_ranges(tmp_path, binary):
    H = host()
    X, _ = _matrix(binary=binary)
    mem = H.FeatureStation("", "W0")
    disk = H.FeatureStation(str(tmp_path / "cache"), "W0", mem_limit_kb=64, threads=2)
    assert not mem.disk and disk.disk
    _add(mem, X, binary)
    _add(disk, X, binary)
    assert mem.mem_size() == disk.mem_size() == X.nnz * (4 if binary else 12) + (X.shape[1] + 1) * 8
    base = disk.file_base(1)
    for ext in ("info", "offset", "index") + (() if binary else ("value",)):
        assert os.path.exists(f"{base}.{ext}")
    assert os.path.getsize(base + ".index") == X.nnz * 4
    # the files are a binary matrix like any other
    m = H.read_bin_matrix(base, 0, 2**63)
    assert m is not None
    for task, (c0, c1) in enumerate([(0, 10), (10, 150), (150, 300), (299, 300), (5, 5)]):
        a = mem.get(task, 1, c0, c1)
        assert disk.prefetch(task, 1, c0, c1)
        assert not disk.prefetch(task, 1, c0, c1)          # a task id is used once
        b = disk.get(task, 1, c0, c1)
        ref = X[:, c0:c1]
        for got in (a, b):
            np.testing.assert_array_equal(got[0], ref.indptr)
            np.testing.assert_array_equal(got[1], ref.indices)
            if binary:
                assert got[2] is None
            else:
                np.testing.assert_array_equal(got[2], ref.data)
        disk.drop(task)
    s = disk.stats()
    assert s["prefetched"] == 5 and s["hits"] == 5 and s["misses"] == 0
    assert disk.resident_bytes() == 0
    with pytest.raises(IndexError):
        disk.get(99, 1, 0, 301)


def test_memory_limit_bounds_what_is_resident(tmp_path):
    H = host()
    X, _ = _matrix(rows=2000, cols=400, density=0.05)
    st = H.FeatureStation(str(tmp_path), "W1", mem_limit_kb=40, threads=3)
    _add(st, X, False)
    blocks = [(c, c + 20) for c in range(0, 400, 20)]                    # ≈ 24 KB each: one fits, two do not
    sizes = [st.range_bytes(1, c0, c1) for c0, c1 in blocks]
    assert max(sizes) < 40 * 1024 < min(sizes) * 2
    for t, (c0, c1) in enumerate(blocks):
        assert st.prefetch(t, 1, c0, c1)
    deadline = time.time() + 10
    while st.stats()["prefetched"] < 1 and time.time() < deadline:
        time.sleep(0.01)
    time.sleep(0.1)
    assert st.stats()["prefetched"] == 1                                # the second waits for room under the limit
    assert st.resident_bytes() == sizes[0]
    for t, (c0, c1) in enumerate(blocks):                                # the solver: use, release, next
        ip, idx, val = st.get(t, 1, c0, c1)
        np.testing.assert_array_equal(idx, X[:, c0:c1].indices)
        st.drop(t)
    s = st.stats()
    assert s["prefetched"] == len(blocks) and s["misses"] == 0
    assert s["peak_resident"] <= 40 * 1024
    assert s["limit_waits"] >= 1
    assert st.pending() == 0 and st.resident_bytes() == 0


def test_unprefetched_and_oversized_ranges(tmp_path):
    H = host()
    X, _ = _matrix(rows=1000, cols=100, density=0.1)
    st = H.FeatureStation(str(tmp_path), "W2", mem_limit_kb=1, threads=1, job_limit=2)
    _add(st, X, False)
    # never queued: the caller loads it itself
    ip, idx, val = st.get(7, 1, 0, 50)
    np.testing.assert_array_equal(val, X[:, 0:50].data)
    assert st.stats()["misses"] == 1 and st.task_used(7) and st.max_task() == 7
    st.drop(7)
    assert not st.task_used(7)
    # larger than the whole limit: admitted once nothing else is resident
    assert st.prefetch(8, 1, 0, 100)
    ip, idx, val = st.get(8, 1, 0, 100)
    assert len(idx) == X.nnz
    # the queue is bounded
    assert st.prefetch(9, 1, 0, 10) and st.prefetch(10, 1, 10, 20)
    assert not st.prefetch(11, 1, 20, 30)
    st.drop(8)
    for t, c in ((9, 0), (10, 10)):
        st.get(t, 1, c, c + 10)
        st.drop(t)
    # another range than the one that was prefetched is an error, not silent wrong data
    assert st.prefetch(12, 1, 0, 10)
    with pytest.raises(RuntimeError):
        st.get(12, 1, 0, 11)


@pytest.mark.parametrize("binary", [False, True])
def test_block_steps_on_a_loaded_range(tmp_path, binary):
    H = host()
    X, y = _matrix(binary=binary, seed=3)
    n = X.shape[1]
    rng = np.random.default_rng(1)
    st = H.FeatureStation(str(tmp_path), "W3", mem_limit_kb=1024, threads=2)
    _add(st, X, binary)
    indptr, indices = X.indptr.astype(np.int64), X.indices.astype(np.int32)
    data = None if binary else X.data
    w = rng.normal(size=n) * 0.1
    dual = np.exp(y * (X @ w))
    delta = np.full(n, 1.0)
    active = (rng.random(n) < 0.9).astype(np.uint8)
    c0, c1 = 37, 211
    st.prefetch(5, 1, c0, c1)
    G, U = st.block_gradient(5, 1, c0, c1, y, dual, delta, active, 2)
    G0, U0 = H.darlin_block_gradient(indptr, indices, data, y, dual, delta, active, c0, c1, 1)
    np.testing.assert_array_equal(G, G0)
    np.testing.assert_array_equal(U, U0)
    w_new = w[c0:c1] + rng.normal(size=c1 - c0) * 0.05
    w_new[::7] = np.nan
    a = [dual.copy(), w.copy(), delta.copy(), active.copy()]
    b = [dual.copy(), w.copy(), delta.copy(), active.copy()]
    st.block_update_dual(5, 1, c0, c1, y, *a, w_new, 5.0)
    H.darlin_update_dual(indptr, indices, data, y, *b, w_new, c0, c1, 5.0)
    for u, v in zip(a, b):
        np.testing.assert_array_equal(u, v)
    st.drop(5)
    assert st.resident_bytes() == 0
