"""The general block store: arrays cut along a column partition, one file per block and kind, prefetch by block."""
import os
import threading
import time

import numpy as np

from parameter_server_b200.runtime import host


def _store(tmp, **kw):
    H = host()
    return H, H.Ocean(str(tmp / "pool"), "W0", **kw)


def _csc(cols=23, seed=0):
    rng = np.random.RandomState(seed)
    per_col = rng.randint(0, 6, cols)
    off = np.concatenate([[0], np.cumsum(per_col)]).astype(np.uint64)
    rows = rng.randint(0, 1000, int(off[-1])).astype(np.uint32)
    vals = rng.rand(int(off[-1]))
    return off, rows, vals


def test_blocks_come_back_as_the_slices_that_went_in(tmp_path):
    H, oc = _store(tmp_path)
    O = H.Ocean
    off, rows, vals = _csc()
    cuts = [100, 105, 105, 116, 123]                      # 23 columns with ids 100..122; the second block is empty
    assert oc.set_partition(1, cuts) and not oc.set_partition(1, cuts) and oc.num_blocks(1) == 4
    keys = np.arange(100, 123, dtype=np.uint32)
    w = np.linspace(-1, 1, 23)
    assert not oc.dump(1, O.FEATURE_KEY, rows)            # per-non-zero arrays need the offsets first
    assert oc.dump(1, O.FEATURE_OFFSET, off) and not oc.dump(1, O.FEATURE_OFFSET, off)
    assert oc.dump(1, O.FEATURE_KEY, rows) and oc.dump(1, O.FEATURE_VALUE, vals)
    assert oc.dump(1, O.PARAMETER_KEY, keys) and oc.dump(1, O.PARAMETER_VALUE, w)
    assert not oc.dump(1, O.DELTA, np.ones(5)) and not oc.dump(7, O.DELTA, np.ones(23))     # wrong length, unknown group
    assert len(os.listdir(tmp_path / "pool")) == 4 * 5
    for b in range(4):
        c0, c1 = cuts[b] - 100, cuts[b + 1] - 100
        oc.prefetch(1, b)
        o = oc.get(1, b, O.FEATURE_OFFSET, "uint64")
        assert o.tolist() == (off[c0:c1 + 1] - off[c0]).tolist()
        p0, p1 = int(off[c0]), int(off[c1])
        assert oc.get(1, b, O.FEATURE_KEY, "uint32").tolist() == rows[p0:p1].tolist()
        assert np.array_equal(oc.get(1, b, O.FEATURE_VALUE, "float64"), vals[p0:p1])
        assert oc.get(1, b, O.PARAMETER_KEY, "uint32").tolist() == keys[c0:c1].tolist()
        assert np.array_equal(oc.get(1, b, O.PARAMETER_VALUE, "float64"), w[c0:c1])
        assert oc.get(1, b, O.DELTA, "float64") is None   # never dumped
        for _ in range(6):
            oc.drop(1, b)
    st = oc.stats()
    assert st["loaded_now"] == 0 and st["prefetched"] == 4 and st["bytes_read"] == st["bytes_written"] > 0
    del oc
    assert os.listdir(tmp_path / "pool") == []            # the files go with the store


def test_prefetch_limit_reference_counts_and_load_on_demand(tmp_path):
    H, oc = _store(tmp_path, threads=2, job_limit=2)
    O = H.Ocean
    cuts = list(range(0, 81, 10))                          # 8 blocks of 10 columns
    oc.set_partition(0, cuts)
    delta = np.arange(80, dtype=np.float64)
    assert oc.dump(0, O.DELTA, delta)
    for b in range(8):
        oc.prefetch(0, b)
    deadline = time.time() + 5
    while oc.stats()["loaded_now"] < 2 and time.time() < deadline:
        time.sleep(0.01)
    time.sleep(0.05)
    assert oc.stats()["loaded_now"] == 2 and oc.pending() == 6          # the limit holds the rest back
    # a block far down the queue is loaded by its caller instead of waiting for a slot
    assert oc.get(0, 7, O.DELTA, "float64").tolist() == delta[70:80].tolist()
    assert oc.stats()["misses"] == 1 and oc.pending() == 5
    oc.drop(0, 7)
    for b in range(7):                                     # consuming in order frees slots for the loaders
        assert oc.get(0, b, O.DELTA, "float64").tolist() == delta[10 * b:10 * b + 10].tolist()
        oc.drop(0, b)
    st = oc.stats()
    assert st["loaded_now"] == 0 and st["peak_loaded"] <= 3 and st["hits"] + st["misses"] == 8
    # two prefetches of one block: it survives the first drop and leaves with the second
    oc.prefetch(0, 3)
    oc.prefetch(0, 3)
    oc.get(0, 3, O.DELTA, "float64"); oc.drop(0, 3)
    assert oc.stats()["loaded_now"] == 1
    oc.get(0, 3, O.DELTA, "float64"); oc.drop(0, 3)
    assert oc.stats()["loaded_now"] == 0


def test_less_memory_and_concurrent_users(tmp_path):
    H, oc = _store(tmp_path, threads=3, job_limit=4, less_memory=True)
    O = H.Ocean
    oc.set_partition(2, [0, 50, 100])
    w = np.random.RandomState(1).rand(100)
    oc.dump(2, O.PARAMETER_VALUE, w)
    oc.prefetch(2, 0); oc.prefetch(2, 0)
    oc.get(2, 0, O.PARAMETER_VALUE, "float64"); oc.drop(2, 0)
    assert oc.stats()["loaded_now"] == 0                  # -less_memory: gone although one prefetch is outstanding
    errs = []

    def user(i):
        try:
            for k in range(50):
                b = (i + k) % 2
                if k % 3 == 0:
                    oc.prefetch(2, b)
                got = oc.get(2, b, O.PARAMETER_VALUE, "float64")
                if not np.array_equal(got, w[50 * b:50 * b + 50]):
                    errs.append((i, k))
                oc.drop(2, b)
        except Exception as e:  # noqa: BLE001
            errs.append(repr(e))

    ts = [threading.Thread(target=user, args=(i,)) for i in range(6)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(30)
    assert not errs and oc.stats()["loaded_now"] == 0


def test_a_block_dropped_before_it_was_loaded_does_not_stay(tmp_path):
    H, oc = _store(tmp_path, threads=1, job_limit=1)
    O = H.Ocean
    oc.set_partition(0, [0, 4, 8, 12])
    oc.dump(0, O.DELTA, np.arange(12.0))
    for b in range(3):
        oc.prefetch(0, b)
        oc.drop(0, b)                      # the caller changed its mind: no get will follow
    deadline = time.time() + 5
    while (oc.pending() or oc.stats()["loaded_now"]) and time.time() < deadline:
        time.sleep(0.01)
    assert oc.pending() == 0 and oc.stats()["loaded_now"] == 0      # nothing is left holding the single job slot
    assert oc.get(0, 1, O.DELTA, "float64").tolist() == [4.0, 5.0, 6.0, 7.0]
    oc.drop(0, 1)
