"""Control-plane runtime: membership, key-range slicing of pushes, logical-clock dependencies,
key cache, replies with payloads, heartbeats / failure detection, host-side fault injection."""
import threading
import time

import numpy as np
import pytest

from parameter_server_b200.runtime import host

H = host()


class Cluster:
    """1 scheduler + S servers + W workers as threads of this process over the in-process van."""

    def __init__(self, W=2, S=2, tcp=False, compress=False):
        self.hub = H.InprocHub()
        self.W, self.S = W, S
        ids = [("H", H.SCHEDULER)] + [(f"W{i}", H.WORKER) for i in range(W)] + [(f"S{i}", H.SERVER) for i in range(S)]
        self.po, self.vans = {}, {}
        sched = None
        for nid, role in ids:
            node = H.Node(role, nid, "127.0.0.1", 0)
            if tcp:
                van = H.TcpVan(node)
                van.bind()
            else:
                van = H.InprocVan(self.hub, node)
            van.set_compress(compress)
            po = H.Postoffice(van, W, S)
            if nid == "H":
                sched = van.my_node
            po.set_scheduler(sched)
            po.start()
            self.po[nid], self.vans[nid] = po, van
        for nid, _ in ids[1:]:
            self.po[nid].register_with_scheduler()
        assert self.po["H"].wait_nodes_and_init(10.0)
        for nid, _ in ids[1:]:
            assert self.po[nid].wait_nodes_ready(10.0)

    def stop(self):
        for po in self.po.values():
            po.stop()


@pytest.fixture(params=["inproc", "tcp"])
def cluster(request):
    c = Cluster(tcp=request.param == "tcp", compress=request.param == "tcp")
    yield c
    c.stop()


def test_membership_and_key_ranges(cluster):
    nodes = {n.id: n for n in cluster.po["W0"].nodes()}
    assert sorted(nodes) == ["H", "S0", "S1", "W0", "W1"]
    assert nodes["S0"].key == (0, (2**64 - 1) // 2) and nodes["S1"].key == ((2**64 - 1) // 2, 2**64 - 1)


def test_push_is_sliced_by_key_range_and_summed(cluster):
    got = {"S0": [], "S1": []}
    custs = {}

    def server_proc(nid):
        def proc(msg):
            if msg.request and msg.cmd == 1:
                got[nid].append((msg.sender, np.frombuffer(msg.key, dtype=np.uint64).tolist(),
                                 np.frombuffer(msg.values[0], dtype=np.float64).tolist(), msg.key_range))
        return proc

    for nid in cluster.po:
        custs[nid] = H.Customer(cluster.po[nid], "w", server_proc(nid) if nid.startswith("S") else None)
    half = (2**64 - 1) // 2
    for w, base in (("W0", 1.0), ("W1", 10.0)):
        keys = np.array([3, 7, half + 5, half + 9], dtype=np.uint64)
        vals = np.arange(4, dtype=np.float64) + base
        t = custs[w].submit(H.kServerGroup, cmd=1, key=keys.tobytes(), values=[vals.tobytes()], key_range=(0, 2**64 - 1))
        assert custs[w].wait_out(H.kServerGroup, t, 10.0)
    assert sorted(x[0] for x in got["S0"]) == ["W0", "W1"]
    for sender, k, v, rng in got["S0"]:
        assert k == [3, 7] and rng == (0, half) and v == ([1.0, 2.0] if sender == "W0" else [10.0, 11.0])
    for sender, k, v, rng in got["S1"]:
        assert k == [half + 5, half + 9] and rng == (half, 2**64 - 1)
    for c in custs.values():
        c.stop()


def test_wait_time_orders_tasks_and_deferred_finish(cluster):
    order, custs = [], {}
    release = threading.Event()

    def proc(msg):
        if not msg.request:
            return
        order.append(("start", msg.time))
        if msg.time == 1:
            msg.defer()                       # task 1 stays unfinished until finish_in is called
            threading.Thread(target=lambda: (release.wait(5), order.append(("fin", 1)),
                                             custs["S0"].finish_in("W0", 1))).start()

    for nid in cluster.po:
        custs[nid] = H.Customer(cluster.po[nid], "app", proc if nid == "S0" else None, False)
    t1 = custs["W0"].submit("S0", payload=b"a", time=1)
    t2 = custs["W0"].submit("S0", payload=b"b", time=2, wait_time=1)     # must not start before task 1 finished
    t3 = custs["W0"].submit("S0", payload=b"c", time=3)                   # independent: may overtake task 2
    assert (t1, t2, t3) == (1, 2, 3)
    assert custs["W0"].wait_out("S0", 3, 10.0)
    assert ("start", 2) not in order
    release.set()
    assert custs["W0"].wait_out("S0", 2, 10.0)
    assert order.index(("fin", 1)) < order.index(("start", 2))
    for c in custs.values():
        c.stop()


def test_pull_reply_with_data_and_payload_replies(cluster):
    custs, pulled = {}, {}

    def server(msg):
        if msg.request and msg.cmd == 2:
            k = np.frombuffer(msg.key, dtype=np.uint64)
            custs[msg.recver].reply(msg, key=msg.key, values=[(k.astype(np.float64) * 2).tobytes()])
        elif msg.request:
            custs[msg.recver].reply(msg, payload=b"progress from " + msg.recver.encode())

    def worker(msg):
        if not msg.request and msg.cmd == 2:
            pulled[msg.sender] = np.frombuffer(msg.values[0], dtype=np.float64).tolist()

    for nid in cluster.po:
        custs[nid] = H.Customer(cluster.po[nid], "kv", server if nid.startswith("S") else worker)
    half = (2**64 - 1) // 2
    keys = np.array([1, 2, half + 1], dtype=np.uint64)
    done = threading.Event()
    t = custs["W1"].submit(H.kServerGroup, cmd=2, key=keys.tobytes(), key_range=(0, 2**64 - 1), on_finish=done.set)
    assert done.wait(10.0)
    assert pulled == {"S0": [2.0, 4.0], "S1": [float(half + 1) * 2]}
    t = custs["H"].submit(H.kServerGroup, payload=b"EVAL", wait=True)
    rep = custs["H"].take_replies(t)
    assert rep == {"S0": b"progress from S0", "S1": b"progress from S1"}
    for c in custs.values():
        c.stop()


def test_key_cache_strips_repeated_keys():
    c = Cluster()
    try:
        seen, custs = [], {}

        def server(msg):
            if msg.request:
                seen.append((msg.has_key, len(msg.key) // 8, msg.key_signature))

        for nid in c.po:
            custs[nid] = H.Customer(c.po[nid], "kc", server if nid == "S0" else None)
        keys = np.arange(1, 5001, dtype=np.uint64)
        vals = np.ones(5000)
        sent = []
        for i in range(3):
            before = c.po["W0"].sent_bytes()
            t = custs["W0"].submit("S0", cmd=1, key=keys.tobytes(), values=[vals.tobytes()], key_range=(0, 10**6), channel=4)
            assert custs["W0"].wait_out("S0", t, 10.0)
            sent.append(c.po["W0"].sent_bytes() - before)
        assert all(s[0] and s[1] == 5000 for s in seen)        # receiver always sees the keys (restored from its cache)
        assert len({s[2] for s in seen}) == 1
        assert sent[1] < 0.6 * sent[0] and sent[2] == sent[1]  # but they crossed the wire only once
        t = custs["W0"].submit("S0", cmd=1, key=keys[:100].tobytes(), values=[vals[:100].tobytes()], key_range=(0, 10**6), channel=4)
        custs["W0"].wait_out("S0", t, 10.0)
        assert seen[-1][1] == 100                               # a different key set replaces the cache entry
        for cu in custs.values():
            cu.stop()
    finally:
        c.stop()


def test_heartbeat_failure_detector_and_message_drop():
    c = Cluster()
    try:
        for nid in ("W0", "S0", "S1"):                         # W1 never reports: it plays the failed node
            c.po[nid].start_heartbeat(0.05, lambda nid=nid: f"hostname: \"{nid}\" busy_time_milli: 5")
        time.sleep(0.5)
        hb = c.po["H"].heartbeats()
        assert b"busy_time_milli" in hb["W0"][1] and hb["W0"][0] < 0.3
        assert c.po["H"].dead_nodes(0.3) == ["W1"]
        # host-side fault injection: drop every request W0 -> S1; the sender observes a bounded timeout, not a hang
        custs = {nid: H.Customer(c.po[nid], "f") for nid in c.po}
        c.vans["W0"].set_filter(lambda s, r, typ, req, t, cust: 1 if (r == "S1" and req) else 0)
        t = custs["W0"].submit(H.kServerGroup, payload=b"x")
        assert custs["W0"].wait_out("S0", t, 5.0)
        assert not custs["W0"].wait_out("S1", t, 0.3)
        assert c.vans["W0"].dropped() == 1
        c.vans["W0"].set_filter(None)
        t2 = custs["W0"].submit(H.kServerGroup, payload=b"y")
        assert custs["W0"].wait_out(H.kServerGroup, t2, 5.0)
        for cu in custs.values():
            cu.stop()
    finally:
        c.stop()


def test_wire_roundtrip_with_compression():
    parts = H.slice_key_ordered(np.arange(100, dtype=np.uint64).tobytes(), [np.ones(100).tobytes()], [0, 1000], None)
    n_plain, m1 = H.encode_decode(parts[0], False)
    n_zip, m2 = H.encode_decode(parts[0], True)
    assert m1.key == m2.key == parts[0].key and m1.values == m2.values and n_zip < n_plain


@pytest.mark.parametrize("tcp", [False, True])
def test_stand_by_node_that_registers_after_the_table_went_out(tcp):
    """A stand-by node (role UNUSED) started late still gets the node table and the end of the job
    (node roles of src/system/postoffice.cc:185-243; stand-by nodes are never waited for)."""
    c = Cluster(W=1, S=1, tcp=tcp)
    try:
        node = H.Node(H.UNUSED, "U0", "127.0.0.1", 0)
        if tcp:
            van = H.TcpVan(node)
            van.bind()
        else:
            van = H.InprocVan(c.hub, node)
        po = H.Postoffice(van, 1, 1)
        po.set_scheduler(c.vans["H"].my_node)
        po.start()
        c.po["U0"] = po
        po.register_with_scheduler()                 # the scheduler broadcast its table long ago
        assert po.wait_nodes_ready(10.0)
        assert sorted(n.id for n in po.nodes()) == ["H", "S0", "U0", "W0"]
        assert "U0" in [n.id for n in c.po["H"].nodes()]
        c.po["H"].stop_all()
        assert po.wait_terminate(10.0)
    finally:
        c.stop()
