"""Property tests (hypothesis) of the host runtime's pure functions: key-range slicing, the threaded merge-join
against the serial one, even range division, sorting, and the text-format parser's round trip."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from parameter_server_b200 import config as cfg
from parameter_server_b200.runtime import host
from parameter_server_b200.utils.pbtext import dumps, parse

H = host()
U64 = st.integers(min_value=0, max_value=2**64 - 2)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(st.lists(U64, max_size=200, unique=True), st.lists(U64, min_size=1, max_size=6, unique=True), st.integers(1, 3))
def test_slices_partition_a_message(keys, cuts, k):
    keys = np.array(sorted(keys), dtype=np.uint64)
    vals = np.arange(len(keys) * k, dtype=np.float64)
    sep = [0] + sorted(c for c in cuts if c > 0) + [2**64 - 1]
    parts = H.slice_key_ordered(keys.tobytes(), [vals.tobytes()], sep, (0, 2**64 - 1))
    assert len(parts) == len(sep) - 1
    got_k = [np.frombuffer(p.key, dtype=np.uint64) for p in parts]
    got_v = [np.frombuffer(p.values[0], dtype=np.float64) for p in parts]
    np.testing.assert_array_equal(np.concatenate(got_k), keys)          # nothing lost, nothing twice, order kept
    np.testing.assert_array_equal(np.concatenate(got_v), vals)
    for p, kk, vv, lo, hi in zip(parts, got_k, got_v, sep[:-1], sep[1:]):
        assert p.key_range == (lo, hi) and len(vv) == len(kk) * k
        assert all(lo <= int(x) < hi for x in kk)


@settings(max_examples=25, deadline=None, derandomize=True)
@given(st.integers(0, 2**32), st.integers(1, 7), st.integers(1, 3))
def test_threaded_aggregation_equals_serial(seed, threads, nval):
    rng = np.random.default_rng(seed)
    mine = np.unique(rng.integers(0, 60000, 9000).astype(np.uint64))      # above the size where threads are used
    out = []
    for th in (1, threads):
        kv = H.KVVector(1)
        kv.merge_keys(0, mine)
        kv.init_values(0, 0.0)
        r2 = np.random.default_rng(seed + 1)
        for _ in range(3):                                               # three senders, overlapping key sets
            k = np.unique(r2.integers(0, 70000, 5000).astype(np.uint64))
            v = r2.normal(size=len(k) * nval)
            kv.aggregate(0, 5, 0, 2**64 - 1, k, v, nval, th)
        out.append(kv.received(5))
    assert out[0][:3] == out[1][:3]
    np.testing.assert_array_equal(out[0][3], out[1][3])


@settings(max_examples=100, deadline=None, derandomize=True)
@given(U64, U64, st.integers(1, 64))
def test_even_divide_covers_the_range(a, b, n):
    lo, hi = min(a, b), max(a, b)
    pieces = [H.even_divide(lo, hi, n, i) for i in range(n)]
    assert pieces[0][0] == lo and pieces[-1][1] == hi
    for (b0, e0), (b1, e1) in zip(pieces[:-1], pieces[1:]):
        assert e0 == b1 and b0 <= e0
    sizes = [e - b for b, e in pieces]
    assert max(sizes) - min(sizes) <= 1 or hi - lo < n


@settings(max_examples=30, deadline=None, derandomize=True)
@given(st.lists(U64, max_size=3000), st.integers(1, 8))
def test_parallel_sort(keys, threads):
    a = np.array(keys, dtype=np.uint64)
    np.testing.assert_array_equal(H.parallel_sort_u64(a, threads), np.sort(a))


names = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_/.-0123456789", min_size=1, max_size=12)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(st.lists(names, max_size=4), st.floats(min_value=1e-6, max_value=1e3, allow_nan=False), st.integers(0, 50),
       st.booleans(), st.integers(0, 2**63), st.integers(0, 2**63))
def test_job_file_round_trip(files, lam, delay, rand, k0, k1):
    c = cfg.AppConfig()
    c.app_name = "p"
    c.parameter_name = ["w"]
    lm = c.mutable("linear_method")
    td = lm.mutable("training_data")
    td.format, td.text, td.file = "TEXT", "LIBSVM", list(files)
    pen = lm.mutable("penalty")
    pen.type = "L1"
    pen.set("lambda", [lam])
    s = lm.mutable("solver")
    s.max_block_delay, s.random_feature_block_order = delay, rand
    for oneline in (False, True):
        back = parse(dumps(c, oneline=oneline), cfg.AppConfig)
        assert list(back.linear_method.training_data.file) == list(files)
        assert back.linear_method.penalty.get("lambda") == [lam]
        assert back.linear_method.solver.max_block_delay == delay
        assert back.linear_method.solver.random_feature_block_order == rand
        assert dumps(back, oneline=oneline) == dumps(c, oneline=oneline)
    call = cfg.LMCall()
    call.cmd = "UPDATE_MODEL"
    r = call.mutable("key")
    r.begin, r.end = min(k0, k1), max(k0, k1)
    back = parse(dumps(call, oneline=True), cfg.LMCall)
    assert (back.key.begin, back.key.end) == (min(k0, k1), max(k0, k1)) and back.cmd == "UPDATE_MODEL"
