"""Failure detection between the ranks of a job, on the host: gloo ranks on CPU, no GPU involved.

Three ranks step in a loop and heartbeat into the process group's store.  Rank 2 goes away between steps —
once after announcing it, once silently — and the others must notice before their next "launch"."""
import multiprocessing as mp
import os
import socket
import time

import pytest


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, announce, q):
    import torch.distributed as dist

    from parameter_server_b200.parallel.monitor import RankLost, RankMonitor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mon = RankMonitor(rank, world, deadline_s=1.0)
    dist.barrier()
    t0 = time.time()
    try:
        for step in range(200):
            mon.beat(step)
            if rank == 2 and step == 3:
                if announce:
                    mon.leave()
                q.put((rank, "left", step, time.time() - t0))
                os._exit(0)                      # between steps, nothing in flight; no clean shutdown on purpose
            mon.check()                          # before the next launch
            time.sleep(0.05)                     # the "step"
        q.put((rank, "finished", 200, time.time() - t0))
    except RankLost as e:
        q.put((rank, "lost", e.ranks, time.time() - t0, str(e)))
    if rank == 0:
        time.sleep(3.0)                          # the store lives in rank 0: let the others read it before it goes
    os._exit(0)


@pytest.mark.parametrize("announce", [True, False])
def test_ranks_notice_a_departed_rank(announce):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()          # synchronous put: nothing is lost when a rank exits right after reporting
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 3, port, announce, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = {}
    deadline = time.time() + 240        # three fresh interpreters import torch first
    while len(got) < 3 and time.time() < deadline:
        if q.empty():
            time.sleep(0.05)
            continue
        r = q.get()
        got[r[0]] = r
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.terminate()
    assert set(got) == {0, 1, 2}, got
    assert got[2][1] == "left"
    for r in (0, 1):
        assert got[r][1] == "lost" and got[r][2] == [2], got[r]
        # announced: seen at the next check; silent: after the one-second deadline
        assert ("left the job" if announce else "no heartbeat") in got[r][4], got[r]
        assert got[r][3] < 20.0, got[r]
