"""Host utilities and containers (C++ via pybind11) against plain Python/NumPy restatements."""
import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from parameter_server_b200.runtime import host

H = host()


def test_crc32c_rfc3720_vectors():
    assert H.crc32c(bytes(32)) == 0x8A9136AA
    assert H.crc32c(bytes([0xFF] * 32)) == 0x62A8AB43
    assert H.crc32c(bytes(range(32))) == 0x46DD794E
    assert H.crc32c(bytes(range(31, -1, -1))) == 0x113FDB5C
    assert H.crc32c(b"123456789") == 0xE3069283
    assert H.crc32c_extend(H.crc32c(b"hello "), b"world") == H.crc32c(b"hello world")
    c = H.crc32c(b"foo")
    assert H.crc32c_unmask(H.crc32c_mask(c)) == c and H.crc32c_mask(c) != c


def test_murmur_and_djb():
    a = H.murmur3_x64_128(b"The quick brown fox jumps over the lazy dog", 0)
    assert a == (0xE34BBC7BBC071B6C, 0x7A433CA9C49A9347)       # published reference digest, seed 0
    assert H.murmur3_x64_128(b"", 0) == (0, 0)
    ids = [H.shuffle_feature_id(i) for i in range(1000)]
    assert len(set(ids)) == 1000
    h = 5381
    for ch in b"abc":
        h = (h * 33 + ch) & 0xFFFFFFFF
    assert H.djb_hash32("abc") == h


@settings(max_examples=30, deadline=None, derandomize=True)
@given(st.lists(st.tuples(st.integers(0, 2**64 - 2), st.integers(1, 5)), min_size=1, max_size=200))
def test_countmin_never_underestimates(pairs):
    cm = H.CountMin()
    cm.resize(4096, 2, True)
    truth = {}
    for k, c in pairs:
        truth[k] = truth.get(k, 0) + c
    keys = np.array([k for k, _ in pairs], dtype=np.uint64)
    cnts = np.array([c for _, c in pairs], dtype=np.uint32)
    cm.insert(keys, cnts)
    uk = np.array(list(truth), dtype=np.uint64)
    est = cm.query(uk)
    for k, e in zip(uk.tolist(), est.tolist()):
        assert e >= min(truth[k], 255)


def test_frequency_filter_and_wrap():
    f = H.FrequencyFilter()
    f.resize(1 << 16, 2)
    keys = np.arange(1000, dtype=np.uint64) * 7919
    counts = np.where(np.arange(1000) % 10 == 0, 9, 1).astype(np.uint32)
    f.insert_keys(keys, counts)
    kept = f.query_keys(keys, 4)
    assert set(keys[::10].tolist()) <= set(kept.tolist()) and len(kept) < 150
    cm = H.CountMin()
    cm.resize(64, 1, False)                      # uint8 counters wrap like the reference's
    cm.insert(np.array([5], dtype=np.uint64), np.array([300], dtype=np.uint32))
    assert cm.query(np.array([5], dtype=np.uint64))[0] == 300 % 256


def test_bitmap():
    b = H.Bitmap(130, False)
    for i in (0, 63, 64, 129):
        b.set(i)
    assert b.nnz() == 4 and b.test(64) and not b.test(65)
    b.clear(64)
    assert b.nnz() == 3
    b.fill(True)
    assert b.nnz() == 130


def test_auc_histogram_matches_exact():
    rng = np.random.RandomState(0)
    y = np.where(rng.rand(5000) < 0.3, 1, -1).astype(np.float32)
    p = (rng.randn(5000) + 0.8 * (y > 0)).astype(np.float32)
    exact = H.exact_auc(y, p)
    pos, neg = p[y > 0], p[y <= 0]
    brute = (pos[:, None] > neg[None, :]).mean() + 0.5 * (pos[:, None] == neg[None, :]).mean()
    assert exact == pytest.approx(brute, abs=1e-9)
    a, b = H.AUC(), H.AUC()
    a.add(y[:2500], p[:2500])
    b.add(y[2500:], p[2500:])
    a.merge(b)
    assert a.evaluate() == pytest.approx(exact, abs=2e-4)
    c = H.AUC()
    c.merge_data(*a.data())
    assert c.evaluate() == a.evaluate()
    assert 0.5 < a.accuracy(0.0) < 1.0


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.lists(st.integers(0, 500), max_size=80), st.lists(st.integers(0, 500), max_size=80))
def test_set_ops_and_match(a, b):
    a = np.array(sorted(set(a)), dtype=np.uint64)
    b = np.array(sorted(set(b)), dtype=np.uint64)
    assert H.set_union(a, b).tolist() == sorted(set(a.tolist()) | set(b.tolist()))
    assert H.set_intersection(a, b).tolist() == sorted(set(a.tolist()) & set(b.tolist()))
    lo, hi = H.find_range(a, 100, 300)
    assert a[lo:hi].tolist() == [x for x in a.tolist() if 100 <= x < 300]
    dst = np.zeros(len(a) * 2)
    src = np.arange(len(b) * 2, dtype=np.float64) + 1
    n = H.match(a, dst, b, src, 2, True, 3)
    assert n == len(set(a.tolist()) & set(b.tolist()))
    for j, k in enumerate(a.tolist()):
        if k in b.tolist():
            i = b.tolist().index(k)
            assert dst[2 * j:2 * j + 2].tolist() == src[2 * i:2 * i + 2].tolist()
        else:
            assert dst[2 * j:2 * j + 2].tolist() == [0, 0]


def test_kv_partition_and_sort():
    rng = np.random.RandomState(1)
    k = rng.randint(0, 1000, 500).astype(np.uint64)
    v = k.astype(np.float64) * 2
    pk, pv, off = H.kv_partition(k, v, [250, 500, 750])
    assert off[0] == 0 and off[-1] == 500 and np.all(pv == pk * 2)
    for p, (lo, hi) in enumerate([(0, 250), (250, 500), (500, 750), (750, 1001)]):
        seg = pk[off[p]:off[p + 1]]
        assert np.all((seg >= lo) & (seg < hi))
    big = rng.randint(0, 2**62, 100000).astype(np.uint64)
    assert np.array_equal(H.parallel_sort_u64(big, 4), np.sort(big))


def test_slice_key_ordered():
    keys = np.array([1, 5, 9, 10, 20, 31], dtype=np.uint64)
    vals = np.arange(12, dtype=np.float64)       # 2 per key
    parts = H.slice_key_ordered(keys.tobytes(), [vals.tobytes()], [0, 10, 20, 40], (0, 25))
    got = [np.frombuffer(p.key, dtype=np.uint64).tolist() for p in parts]
    assert got == [[1, 5, 9], [10], [20, 31]]
    assert np.frombuffer(parts[1].values[0], dtype=np.float64).tolist() == [6.0, 7.0]
    assert [p.key_range for p in parts] == [(0, 10), (10, 20), (20, 25)] and all(p.valid for p in parts)
    parts = H.slice_key_ordered(keys.tobytes(), [], [0, 10, 20, 40], (0, 10))
    assert [p.valid for p in parts] == [True, False, False]


def test_even_divide_soft_threshold_recordio_zlib(tmp_path):
    assert H.even_divide(0, 2**64 - 1, 2, 0) == (0, (2**64 - 1) // 2)
    assert H.even_divide(0, 2**64 - 1, 2, 1)[1] == 2**64 - 1
    assert H.soft_thresholding(3.0, 1.0, 2.0) == -1.0 and H.soft_thresholding(-3.0, 1.0, 2.0) == 1.0
    assert H.soft_thresholding(0.5, 1.0, 2.0) == 0.0
    recs = [b"", b"abc", bytes(range(256)) * 10]
    path = str(tmp_path / "r.rec")
    assert H.record_write(path, recs) and H.record_read(path) == recs
    nan_like = (b"\xff" * 8) * 5000           # the inactive-weight sentinel compresses well
    ok, zsize, back = H.zlib_roundtrip(nan_like)
    assert ok and back == nan_like and zsize < len(nan_like) // 50


def test_kvvector_aggregate_and_lookup():
    kv = H.KVVector(1)
    kv.merge_keys(0, np.array([2, 4, 6], dtype=np.uint64))
    kv.merge_keys(0, np.array([4, 8, 10], dtype=np.uint64))
    assert kv.keys(0).tolist() == [2, 4, 6, 8, 10]
    kv.init_values(0, 0.0)
    kv.aggregate(0, 7, 0, 9, np.array([2, 6], dtype=np.uint64), np.array([1, 10, 2, 20], dtype=np.float64), 2, 1)
    kv.aggregate(0, 7, 0, 9, np.array([4, 6], dtype=np.uint64), np.array([5, 50, 3, 30], dtype=np.float64), 2, 1)
    lo, hi, nval, vals = kv.received(7)
    assert (lo, hi, nval) == (0, 4, 2) and vals.tolist() == [1, 10, 5, 50, 5, 50, 0, 0]
    kv.set_values(0, np.array([.2, .4, .6, .8, 1.0]))
    assert kv.lookup(0, np.array([1, 4, 10], dtype=np.uint64)).tolist() == [0.0, 0.4, 1.0]


def test_numpy_countmin_restatement_matches_host():
    """The oracle's NumPy count-min (used by the FTRL / DARLIN tail-filter tests) equals the C++ one."""
    from baseline.cpu_ref.ftrl_ref import CountMinRef, FTRLRef

    rng = np.random.RandomState(0)
    keys = rng.randint(0, 2**63, size=2000, dtype=np.int64).astype(np.uint64) * np.uint64(2) + np.uint64(1)
    cnt = rng.randint(1, 6, size=2000).astype(np.uint32)
    assert np.array_equal(CountMinRef._hash(keys), np.array([H.CountMin.hash(int(k)) for k in keys], dtype=np.uint64))
    cm = H.CountMin()
    cm.resize(4096, 2, True)
    cm.insert(keys, cnt)
    ref = CountMinRef(4096, 2)
    ref.insert(keys, cnt)
    assert np.array_equal(np.asarray(cm.query(keys)).astype(np.uint64), ref.query(keys))
    assert np.all(ref.query(keys) >= cnt)                       # one-sided error
    # the filter keeps a key out of the oracle's model until its estimate passes the threshold
    f = FTRLRef(0.1, 1.0, 0.0, 0.0, tail_freq=3, countmin_n=1 << 12, countmin_k=2)
    off = np.array([0, 2, 4], dtype=np.int64)
    mb = (off, np.array([5, 9, 5, 11], dtype=np.uint64), np.array([1.0, -1.0]))
    f.step([mb])
    assert len(f.model) == 0                                    # counts 2, 1, 1: nobody above 3 yet
    f.step([mb])
    assert set(f.model) == {5}                                  # key 5 reached 4 > 3


def test_native_ftrl_model_matches_oracle():
    """FTRLModel (server-side store of the CPU online job): per-key update, pulls, running norms."""
    from baseline.cpu_ref.ftrl_ref import FTRLRef

    m = H.FTRLModel(0.05, 1.0, 0.05, 0.1)
    ref = FTRLRef(0.05, 1.0, 0.05, 0.1, "count")
    rng = np.random.RandomState(0)
    for _ in range(30):
        k = np.unique(rng.randint(0, 80, size=25)).astype(np.uint64) * np.uint64(2**57 + 3)
        g, pos, neg = rng.randn(len(k)), rng.randint(0, 5, len(k)).astype(float), rng.randint(0, 5, len(k)).astype(float)
        m.update(k, g, pos, neg)
        ref.set_value(k, pos, neg, g)
    k, w = m.nonzero()
    rk, rw = ref.nonzero()
    assert np.array_equal(k, rk) and np.allclose(w, rw, rtol=1e-12)
    n1, n2, nnz = m.stats()
    assert n1 == pytest.approx(ref.norm1) and n2 == pytest.approx(ref.norm2) and nnz == ref.nnz and m.size() == len(ref.model)
    probe = np.array([int(rk[0]), 12345], dtype=np.uint64)
    assert m.get(probe).tolist() == [pytest.approx(rw[0]), 0.0]
    with pytest.raises(ValueError):
        m.update(k, w[:-1], w, w)


@pytest.mark.parametrize("binary", [False, True])
def test_native_darlin_block_steps(binary):
    """Block gradient (threaded), server update and dual update of the CPU nodes against a NumPy restatement."""
    import scipy.sparse as sp

    rng = np.random.RandomState(1)
    rows, cols = 300, 200
    X = sp.random(rows, cols, density=0.05, random_state=rng, format="csc")
    if binary:
        X.data[:] = 1.0
    indptr, indices = X.indptr.astype(np.int64), X.indices.astype(np.int32)
    data = None if binary else X.data.astype(np.float64)
    y = np.where(rng.rand(rows) < 0.5, 1.0, -1.0)
    dual = np.exp(rng.randn(rows) * 0.3)
    delta = rng.rand(cols) + 0.5
    active = (rng.rand(cols) < 0.9).astype(np.uint8)
    c0, c1 = 20, 180
    G, U = H.darlin_block_gradient(indptr, indices, data, y, dual, delta, active, c0, c1, 4)
    tau = 1 / (1 + dual)
    t2 = tau * (1 - tau)
    for j in range(c0, c1):
        s, e = indptr[j], indptr[j + 1]
        r, v = indices[s:e], X.data[s:e]
        if not active[j]:
            assert np.isnan(G[j - c0]) and np.isnan(U[j - c0])
            continue
        assert G[j - c0] == pytest.approx(-np.sum(y[r] * tau[r] * v), rel=1e-12, abs=1e-15)
        assert U[j - c0] == pytest.approx(np.sum(np.minimum(t2[r] * np.exp(np.abs(v) * delta[j]), 0.25) * v * v), rel=1e-12, abs=1e-15)
    # server update: zero weights with a small gradient are filtered (NaN), the others move inside the trust region
    n = c1 - c0
    w = np.where(rng.rand(n) < 0.5, 0.0, rng.randn(n) * 0.1)
    dl, ac = np.ones(n), np.ones(n, dtype=np.uint8)
    g = np.nan_to_num(G, nan=0.0)
    u = np.nan_to_num(U, nan=1.0)
    w2, dl2, ac2 = w.copy(), dl.copy(), ac.copy()
    vio = H.darlin_update_weight(w2, dl2, ac2, g, u, 0.05, 1.0, 0.02, 5.0)
    filtered = (w == 0) & (g + 0.05 > 0.02) & (g - 0.05 < -0.02) & ~((g + 0.05 < 0) | (g - 0.05 > 0))
    assert np.array_equal(np.isnan(w2), filtered) and np.array_equal(ac2 == 0, filtered)
    assert vio == pytest.approx(max(0.0, np.max(np.where(w == 0, np.maximum(-(g + 0.05), g - 0.05), 0.0))))
    moved = ~filtered
    assert np.all(np.abs(w2[moved] - w[moved]) <= dl[moved] + 1e-15)
    # dual update: dual_i *= exp(y_i x_ij dw_j); NaN in w_new deactivates the column
    wn = rng.randn(n) * 0.1
    wn[3] = np.nan
    wloc, dloc, aloc, dual2 = np.zeros(cols), np.ones(cols), np.ones(cols, dtype=np.uint8), dual.copy()
    H.darlin_update_dual(indptr, indices, data, y, dual2, wloc, dloc, aloc, wn, c0, c1, 5.0)
    expect = dual.copy()
    for j in range(c0, c1):
        if np.isnan(wn[j - c0]):
            continue
        s, e = indptr[j], indptr[j + 1]
        expect[indices[s:e]] *= np.exp(y[indices[s:e]] * X.data[s:e] * wn[j - c0])
    np.testing.assert_allclose(dual2, expect, rtol=1e-12)
    assert aloc[c0 + 3] == 0 and wloc[c0 + 3] == 0 and np.allclose(np.delete(wloc[c0:c1], 3), np.delete(wn, 3))
    with pytest.raises(ValueError):
        H.darlin_block_gradient(indptr, indices, data, y, dual, delta, active, 0, cols + 5, 1)


def test_model_lookup_and_margins_for_a_warm_start(tmp_path):
    """The pieces a warm start is made of: weights of a key list from a model dump, and y * Xw from column-major data."""
    import scipy.sparse as sp
    import torch

    from parameter_server_b200.models.darlin import margins_from_weights
    from parameter_server_b200.utils.modelio import lookup_model, model_arrays, model_files, read_model_text, write_model_text

    write_model_text(str(tmp_path / "m_S0"), [3, 9, 2**63 + 5], [0.5, -1.25, 2.0])
    write_model_text(str(tmp_path / "m_S1"), [2**64 - 2], [4.0])
    paths = model_files(str(tmp_path / "m"))
    assert [p.rsplit("_", 1)[1] for p in paths] == ["S0", "S1"] and model_files(paths[0]) == [paths[0]]
    mk, mv = model_arrays(read_model_text(*paths))
    keys = np.array([1, 3, 4, 9, 2**63 + 5, 2**64 - 2, 2**64 - 1], dtype=np.uint64)
    np.testing.assert_array_equal(lookup_model(mk, mv, keys), [0, 0.5, 0, -1.25, 2.0, 4.0, 0])
    assert lookup_model(mk[:0], mv[:0], keys).sum() == 0 and len(lookup_model(mk, mv, keys[:0])) == 0

    rng = np.random.default_rng(0)
    for binary in (False, True):
        X = sp.random(50, 30, density=0.2, format="csc", random_state=1, dtype=np.float64)
        if binary:
            X.data[:] = 1
        y = np.where(rng.random(50) < 0.5, -1.0, 1.0)
        w = rng.normal(size=30)
        m = margins_from_weights(torch.from_numpy(X.indptr.astype(np.int64)), torch.from_numpy(X.indices.astype(np.int32)),
                                 None if binary else torch.from_numpy(X.data.astype(np.float32)), torch.from_numpy(y.astype(np.float32)),
                                 torch.from_numpy(w.astype(np.float32)))
        np.testing.assert_allclose(m.numpy(), y * (X @ w), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("threads", [1, 4])
def test_native_localizer(threads):
    """Unique keys with counts, global -> local ids and the change to column-major storage against NumPy / SciPy."""
    import scipy.sparse as sp

    rng = np.random.default_rng(threads)
    rows, nnz_row = 5000, 9
    keys = (rng.integers(0, 3000, rows * nnz_row).astype(np.uint64) * np.uint64(6148914691236517)) + np.uint64(2**63)
    off = np.arange(0, rows * nnz_row + 1, nnz_row, dtype=np.int64)
    vals = rng.normal(size=len(keys))
    u, c = H.count_unique(keys, threads)
    ru, rinv, rc = np.unique(keys, return_inverse=True, return_counts=True)
    np.testing.assert_array_equal(u, ru)
    np.testing.assert_array_equal(c, rc)
    for kk in (keys, keys[:1], keys[:0], np.arange(70000, dtype=np.uint64)[::-1].copy() % np.uint64(1000),
               np.array([0, 2**64 - 1, 0, 2**63, 2**64 - 1], dtype=np.uint64)):
        lu, lc, linv = H.localize(kk)                               # radix sort of (key, position) pairs
        eu, einv, ec = np.unique(kk, return_inverse=True, return_counts=True)
        np.testing.assert_array_equal(lu, eu)
        np.testing.assert_array_equal(lc, ec)
        np.testing.assert_array_equal(linv, einv)
    # a dictionary that lacks every third key: those non-zeros are dropped
    d = ru[np.arange(len(ru)) % 3 != 0]
    loc = H.remap_keys(keys, d, threads)
    pos = np.searchsorted(d, keys)
    hit = (pos < len(d)) & (d[np.minimum(pos, len(d) - 1)] == keys)
    np.testing.assert_array_equal(loc, np.where(hit, pos, -1))
    for v in (vals, None):
        ip, ri, ov = H.csr_to_csc(off, loc, v, len(d), threads)
        row_of = np.repeat(np.arange(rows), nnz_row)[hit]
        ref = sp.csr_matrix((np.ones(hit.sum()) if v is None else v[hit], (row_of, loc[hit])), shape=(rows, len(d)))
        # duplicates inside a row stay separate entries here, SciPy sums them: compare through dense products
        assert ip[-1] == hit.sum() and len(ri) == hit.sum() and (ov is None) == (v is None)
        assert np.all(np.diff(ip) >= 0)
        for j in (0, 7, len(d) - 1):
            seg = ri[ip[j]:ip[j + 1]]
            assert np.all(np.diff(seg) >= 0)                                  # rows ascend inside a column
        x = rng.normal(size=rows)
        got = np.zeros(len(d))
        np.add.at(got, np.repeat(np.arange(len(d)), np.diff(ip)), x[ri] * (1.0 if ov is None else ov))
        np.testing.assert_allclose(got, ref.T @ x, rtol=1e-9, atol=1e-9)
    with pytest.raises(ValueError):
        H.csr_to_csc(off, loc, None, 5, 1)


@pytest.mark.parametrize("binary,threads", [(False, 1), (True, 3)])
def test_native_ftrl_minibatch(binary, threads):
    rng = np.random.default_rng(5)
    rows, nk = 1500, 400
    per = rng.integers(0, 12, rows)
    off = np.concatenate([[0], np.cumsum(per)]).astype(np.int64)
    loc = rng.integers(0, nk, off[-1]).astype(np.int32)
    val = None if binary else rng.normal(size=off[-1])
    y = np.where(rng.random(rows) < 0.4, 1.0, -1.0)
    w = rng.normal(size=nk) * 3                                        # large margins: the loss must not overflow
    loss, g, pos, neg = H.ftrl_minibatch(off, loc, val, y, w, threads)
    v = np.ones(off[-1]) if binary else val
    row_of = np.repeat(np.arange(rows), per)
    m = y * np.bincount(row_of, weights=w[loc] * v, minlength=rows)
    assert loss == pytest.approx(np.sum(np.logaddexp(0.0, -m)), rel=1e-12)
    coef = -y / (1.0 + np.exp(m))
    np.testing.assert_allclose(g, np.bincount(loc, weights=coef[row_of] * v, minlength=nk), rtol=1e-12, atol=1e-12)
    np.testing.assert_array_equal(pos, np.bincount(loc, weights=(y[row_of] > 0).astype(float), minlength=nk))
    np.testing.assert_array_equal(neg, np.bincount(loc, weights=(y[row_of] <= 0).astype(float), minlength=nk))
    with pytest.raises(ValueError):
        H.ftrl_minibatch(off, loc + nk, val, y, w, 1)


def test_ftrl_model_store_grows_and_keeps_every_key():
    """The model's hash map through several doublings: sizes, look-ups of present and absent keys, key 0 and the
    largest key, and independence from how the updates were batched."""
    rng = np.random.default_rng(9)
    keys = np.unique(np.concatenate([rng.integers(0, 2**63, 60000).astype(np.uint64) * np.uint64(2),
                                     np.array([0, 2**64 - 1, 2**64 - 2], dtype=np.uint64)]))
    g = rng.normal(size=len(keys))
    pos = rng.integers(0, 3, len(keys)).astype(np.float64)
    neg = rng.integers(1, 3, len(keys)).astype(np.float64)
    a, b = H.FTRLModel(0.1, 1.0, 0.01, 0.1), H.FTRLModel(0.1, 1.0, 0.01, 0.1)
    a.update(keys, g, pos, neg)
    perm = rng.permutation(len(keys))
    for part in np.array_split(perm, 37):                      # same updates, other order and batching
        b.update(keys[part], g[part], pos[part], neg[part])
    assert a.size() == b.size() == len(keys)
    wa, wb = a.get(keys), b.get(keys)
    np.testing.assert_array_equal(wa, wb)
    assert np.count_nonzero(wa) > len(keys) // 2
    absent = keys[:1000] + np.uint64(1)                        # odd keys were never inserted (0 + 1 = 1 neither)
    absent = absent[~np.isin(absent, keys)]
    assert np.all(a.get(absent) == 0) and a.size() == len(keys)   # a look-up inserts nothing
    ka, va = a.nonzero()
    assert np.all(np.diff(ka.astype(np.float64)) >= 0) and len(ka) == np.count_nonzero(wa)
    n1, n2, nnz = a.stats()
    assert nnz == len(ka) and n1 == pytest.approx(np.abs(va).sum(), rel=1e-9) and n2 == pytest.approx((va ** 2).sum(), rel=1e-9)
