"""Device key-set / sparse-matrix operators against NumPy and torch references."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _u(t):
    return t.cpu().numpy().view(np.uint64)


@pytest.mark.parametrize("n,bits", [(1, 64), (1000, 12), (5000, 64), (300_000, 40), (1_000_003, 64)])
def test_radix_sort_is_stable_and_unsigned(n, bits):
    from parameter_server_b200.ops import sparse

    rng = np.random.RandomState(n)
    k = rng.randint(0, 2**63, size=n, dtype=np.int64).astype(np.uint64) * 2 + rng.randint(0, 2, size=n).astype(np.uint64)
    if bits < 64:
        k &= np.uint64((1 << bits) - 1)
    if n > 100:
        k[: n // 10] = k[n // 2]                       # duplicates: payload order must be preserved
        k[5] = np.uint64(2**64 - 2)                     # top bit set: unsigned order
    keys = torch.from_numpy(k.view(np.int64)).cuda()
    vals = torch.arange(n, dtype=torch.int32, device="cuda")
    sk, sv = sparse.sort_pairs(keys, vals)
    order = np.argsort(k, kind="stable")
    assert np.array_equal(_u(sk), k[order])
    assert np.array_equal(sv.cpu().numpy(), order.astype(np.int32))
    assert np.array_equal(_u(keys), k)                  # input untouched
    uk, cnt = sparse.count_unique(keys)
    ru, rc = np.unique(k, return_counts=True)
    assert np.array_equal(_u(uk), ru) and np.array_equal(cnt.cpu().numpy(), rc.astype(np.int32))


def test_scan_remap_transpose_partition():
    from parameter_server_b200.ops import sparse

    x = torch.randint(0, 5, (100_003,), dtype=torch.int32, device="cuda")
    pre, tot = sparse.exclusive_scan(x)
    ref = torch.cumsum(x.long(), 0) - x.long()
    assert torch.equal(pre, ref) and tot.item() == x.long().sum().item()
    rng = np.random.RandomState(0)
    dic = np.unique(rng.randint(0, 10_000, size=3000).astype(np.uint64) * np.uint64(2**50 + 7))
    keys = np.concatenate([rng.choice(dic, 5000), np.array([1, 2, 3], dtype=np.uint64)])
    out = sparse.remap(torch.from_numpy(keys.view(np.int64)).cuda(), torch.from_numpy(dic.view(np.int64)).cuda()).cpu().numpy()
    pos = np.searchsorted(dic, keys)
    hit = (pos < len(dic)) & (dic[np.minimum(pos, len(dic) - 1)] == keys)
    assert np.array_equal(out[hit], pos[hit].astype(np.int32)) and np.all(out[~hit] == -1)
    # CSR -> CSC
    rows, cols = 500, 300
    counts = rng.randint(0, 12, size=rows)
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    col = rng.randint(0, cols, size=off[-1]).astype(np.int32)
    col[::17] = -1                                       # dropped by an earlier remap
    val = rng.rand(off[-1]).astype(np.float32)
    cp, ri, cv = sparse.csr_to_csc(torch.from_numpy(off).cuda(), torch.from_numpy(col).cuda(), torch.from_numpy(val).cuda(), cols)
    cp, ri, cv = cp.cpu().numpy(), ri.cpu().numpy(), cv.cpu().numpy()
    row_of = np.repeat(np.arange(rows), counts)
    assert cp[-1] == (col >= 0).sum()
    for j in range(0, cols, 7):
        mine = sorted(zip(ri[cp[j]:cp[j + 1]].tolist(), cv[cp[j]:cp[j + 1]].tolist()))
        want = sorted(zip(row_of[col == j].tolist(), val[col == j].tolist()))
        assert mine == want
    # k-way partition by owner key range
    k = rng.randint(0, 2**62, size=20_000).astype(np.uint64) * 4
    v = rng.rand(20_000).astype(np.float32)
    seps = [0, 2**62, 2**63, 2**63 + 2**62, 2**64 - 1]
    st, pk, pv = sparse.partition_by_key_range(torch.from_numpy(k.view(np.int64)).cuda(), torch.from_numpy(v).cuda(), seps)
    st, pk, pv = st.cpu().numpy(), _u(pk), pv.cpu().numpy()
    assert st[0] == 0 and st[-1] == len(k)
    lookup = dict(zip(k.tolist(), v.tolist()))
    for p in range(4):
        seg = pk[st[p]:st[p + 1]]
        assert np.all((seg >= np.uint64(seps[p])) & (seg < np.uint64(seps[p + 1])))
        assert len(seg) == ((k >= np.uint64(seps[p])) & (k < np.uint64(seps[p + 1]))).sum()
    assert all(lookup[a] == pytest.approx(b) for a, b in zip(pk[:200].tolist(), pv[:200].tolist()))


def test_countmin_matches_host_and_set_ops_and_spmv():
    from parameter_server_b200.ops import sparse
    from parameter_server_b200.runtime import host

    H = host()
    rng = np.random.RandomState(3)
    keys = np.unique(rng.randint(0, 2**62, size=4000).astype(np.uint64))
    cnts = rng.randint(1, 6, size=len(keys)).astype(np.uint32)
    dk = torch.from_numpy(keys.view(np.int64)).cuda()
    cm = sparse.CountMinDevice(1 << 14, 2, "cuda")
    cm.insert(dk, torch.from_numpy(cnts.astype(np.int32)).cuda())
    hc = H.CountMin()
    hc.resize(1 << 14, 2, True)
    hc.insert(keys, cnts)
    assert np.array_equal(cm.query(dk).cpu().numpy().astype(np.uint32), hc.query(keys))     # same hash, same probes
    kept = _u(cm.filter(dk, 3))
    assert set(keys[cnts > 3].tolist()) <= set(kept.tolist()) and len(kept) < len(keys)
    a = np.unique(rng.randint(0, 5000, size=2000).astype(np.uint64))
    b = np.unique(rng.randint(0, 5000, size=2000).astype(np.uint64))
    ta, tb = torch.from_numpy(a.view(np.int64)).cuda(), torch.from_numpy(b.view(np.int64)).cuda()
    assert np.array_equal(_u(sparse.set_intersection(ta, tb)), np.intersect1d(a, b))
    assert np.array_equal(_u(sparse.set_union(ta, tb)), np.union1d(a, b))
    rows, cols = 400, 256
    counts = rng.randint(0, 20, size=rows)
    off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)).cuda()
    idx = torch.from_numpy(rng.randint(0, cols, size=int(off[-1])).astype(np.int32)).cuda()
    val = torch.rand(int(off[-1]), device="cuda")
    w, v = torch.randn(cols, device="cuda"), torch.randn(rows, device="cuda")
    dense = torch.zeros(rows, cols, device="cuda")
    row_of = torch.repeat_interleave(torch.arange(rows, device="cuda"), off[1:] - off[:-1])
    dense.index_put_((row_of, idx.long()), val, accumulate=True)
    torch.testing.assert_close(sparse.spmv(off, idx, val, w), dense @ w, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(sparse.spmv_t(off, idx, val, v, cols), dense.T @ v, rtol=1e-4, atol=1e-4)
    g = torch.empty(200_000, device="cuda")
    sparse.fill_gaussian(g, 1.0, 2.0, 7)
    assert abs(g.mean().item() - 1.0) < 0.03 and abs(g.std().item() - 2.0) < 0.03
