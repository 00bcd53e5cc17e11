"""The scheduler node for GPU jobs, on CPU: gloo ranks, a stand-in solver with the interface of the GPU solver.

Checks the control flow only (tasks per pass with the block order, progress replies, the stopping rule, SAVE_MODEL,
heartbeat table, a failing task reaching the scheduler); the GPU job test runs the same code on the real solver."""
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


def _rank_main(rank, world, port, mode, tmp, q):
    import numpy as np
    import torch
    import torch.distributed as dist

    from parameter_server_b200 import config as cfg
    from parameter_server_b200.apps.gpu_control import run_scheduled
    from parameter_server_b200.models.darlin import DarlinConfig, Progress, block_order

    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # like the kernels' bounded waits: a collective whose peer is gone gives up instead of waiting for ever
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))

    class Group:
        def __init__(self):
            self.rank, self.world, self.group, self.device = rank, world, dist.group.WORLD, torch.device("cpu")

        def barrier(self):
            dist.barrier()

    class StandIn:
        """Objective halves every pass until it stalls; every pass is a collective, like the real one."""

        def __init__(self):
            self.cfg = DarlinConfig(lambda1=1.0, max_pass=12, epsilon=1e-3, random_block_order=True, seed=5,
                                    prior_fea_group=(2,), num_iter_for_prior_fea_group=2)
            self.nblk, self.block_group = 6, [1, 1, 2, 2, 3, 3]
            self.progress, self.seen = [], []

        def run_pass(self, order, reset=False, prior=None):
            it = len(self.progress)
            if mode == "heartbeat":
                time.sleep(0.1)                                      # long enough for a few reports per job
            self.seen.append((list(map(int, order)), bool(reset), None if prior is None else list(map(int, prior))))
            if mode == "vanish" and it == 2 and rank == 1:
                os._exit(0)                                          # between passes, nothing in flight, no goodbye
            part = torch.tensor([100.0 / world * max(0.5 ** it, 0.5 ** 4)], dtype=torch.float64)
            dist.all_reduce(part)                                    # runs on the node's executor thread
            objv = float(part.item())
            if mode == "fail" and it == 2 and rank == 1:
                raise ValueError("device says no")                   # after the collective: the other rank is not left in it
            rel = 1.0 if not self.progress else self.progress[-1].objv / objv - 1.0
            p = Progress(objv, rel, 10 + it, 0.5, 60, 0.0, 0.01)
            self.progress.append(p)
            return p

        def save_model(self, prefix):
            path = f"{prefix}_S{rank}"
            open(path, "w").write("1\t0.5\n")
            return path

    sol = StandIn()
    flags = cfg.Flags(report_interval=0.2 if mode in ("heartbeat", "vanish") else 0)
    try:
        out = run_scheduled(Group(), flags, "job", sol, os.path.join(tmp, "model"), verbose=False)
        orders = [o.tolist() for o in block_order(6, 12, True, 5)]
        q.put((rank, "ok", dict(passes=len(sol.progress), seen=sol.seen, orders=orders, model=out["model"],
                                sched=out.get("scheduler"), saved=out.get("saved"), dash=out.get("dashboard"))))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", f"{type(e).__name__}: {e}"))
    dist.barrier() if mode not in ("fail", "vanish") else time.sleep(1.0)
    os._exit(0)


def _run(mode, tmp, world=2, expect=None):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, mode, str(tmp), q)) for r in range(world)]
    for p in procs:
        p.start()
    expect = world if expect is None else expect
    got = {}
    deadline = time.time() + 240
    while len(got) < expect and time.time() < deadline:
        if q.empty():
            time.sleep(0.1)
            continue
        r, status, body = q.get()
        got[r] = (status, body)
    for p in procs:
        p.join(20)
        if p.is_alive():
            p.kill()
    assert len(got) == expect, f"only {sorted(got)} reported"
    return got


def test_scheduler_drives_the_passes_and_stops_by_the_rule(tmp_path):
    got = _run("plain", tmp_path)
    assert all(s == "ok" for s, _ in got.values()), got
    a, b = got[0][1], got[1][1]
    # objective 100, 50, 25, 12.5, 6.25, then constant: relative change 0 is not "0 < rel <= eps", so the job runs
    # all 12 passes; the order of every pass and the first pass's prior sweeps arrive as the scheduler made them
    assert a["passes"] == b["passes"] == 12 and a["seen"] == b["seen"]
    assert [s[0] for s in a["seen"]] == a["orders"]
    assert a["seen"][0][2] is not None and sorted(set(a["seen"][0][2])) == [2, 3] and len(a["seen"][0][2]) == 4
    assert all(s[2] is None for s in a["seen"][1:])
    assert len(a["sched"]) == 12 and a["sched"][0]["objv"] == pytest.approx(100.0) and a["sched"][1]["relative_objv"] == pytest.approx(1.0)
    assert a["saved"] == [str(tmp_path / "model_S0"), str(tmp_path / "model_S1")]
    assert a["model"].endswith("_S0") and b["model"].endswith("_S1") and os.path.exists(b["model"])
    assert b["sched"] is None


def test_heartbeats_reach_the_scheduler(tmp_path):
    got = _run("heartbeat", tmp_path)
    assert all(s == "ok" for s, _ in got.values()), got
    dash = got[0][1]["dash"]
    assert dash.splitlines()[0].startswith("Node") and "W0@" in dash and "W1@" in dash and "no report yet" not in dash


def test_a_failing_task_ends_the_job_with_its_error(tmp_path):
    got = _run("fail", tmp_path)
    assert got[0][0] == "error" and "W1" in got[0][1] and "device says no" in got[0][1]
    assert got[1][0] == "error" and "device says no" in got[1][1]


def test_a_rank_that_vanishes_does_not_hang_the_job(tmp_path):
    """Rank 1 exits between passes.  Rank 0's pass gives up in its bounded collective and says so, or the scheduler
    misses W1's heartbeats first; either way the job ends with an error that names the cause instead of waiting."""
    t0 = time.time()
    got = _run("vanish", tmp_path, expect=1)
    assert got[0][0] == "error", got
    msg = got[0][1]
    assert "no heartbeat from W1" in msg or "W0:" in msg or "task failed" in msg, msg
    assert time.time() - t0 < 120

# ---------------------------------------------------------------------------------------------------------------
def _online_main(rank, world, port, mode, tmp, q):
    import torch
    import torch.distributed as dist

    from parameter_server_b200 import config as cfg
    from parameter_server_b200.apps.gpu_control import run_scheduled_online

    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))

    class Group:
        def __init__(self):
            self.rank, self.world, self.group, self.device = rank, world, dist.group.WORLD, torch.device("cpu")

        def barrier(self):
            dist.barrier()

    conf = cfg.parse_app_config('''app_name: "ctr" parameter_name: "ctr_w"
        linear_method { loss { type: LOGIT } penalty { type: L1 lambda: 0.1 }
          solver { minibatch_size: 100 eval_interval: 0.05 } ftrl { } }''')
    state = {"examples": 0, "loss": 0.0}

    def run_training(report):
        losses = []
        for step in range(12):
            if mode == "vanish" and step == 5 and rank == 1:
                os._exit(0)
            t = torch.tensor([1.0])
            dist.all_reduce(t)                            # every step is a collective, like the real one
            if mode == "fail" and step == 5:                # rank 1 fails; rank 0 sees it as a wait that ran out
                raise ValueError("table full") if rank == 1 else TimeoutError("peer 1 silent")
            loss = 0.6 - 0.02 * step
            losses.append(loss)
            state["examples"] += 100
            state["loss"] += loss * 100
            report(loss * 100, 100, 0.5 + rank, 10 * (rank + 1))
            time.sleep(0.03)
        return losses

    try:
        out = run_scheduled_online(Group(), cfg.Flags(), conf, run_training,
                                   lambda: (state["loss"] + 0.5 + rank, 10 * (rank + 1), state["examples"]),
                                   lambda: os.path.join(tmp, f"ftrl_S{rank}"), verbose=False)
        q.put((rank, "ok", dict(result=out["result"], model=out["model"], sched=out.get("scheduler"))))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", f"{type(e).__name__}: {e}"))
    dist.barrier() if mode not in ("fail", "vanish") else time.sleep(1.0)
    os._exit(0)


def _run_online(mode, tmp, world=2, expect=None):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_online_main, args=(r, world, port, mode, str(tmp), q)) for r in range(world)]
    for p in procs:
        p.start()
    expect = world if expect is None else expect
    got = {}
    deadline = time.time() + 240
    while len(got) < expect and time.time() < deadline:
        if q.empty():
            time.sleep(0.1)
            continue
        r, status, body = q.get()
        got[r] = (status, body)
    for p in procs:
        p.join(20)
        if p.is_alive():
            p.kill()
    assert len(got) == expect, f"only {sorted(got)} reported"
    return got


def test_online_job_under_the_scheduler(tmp_path):
    import re

    got = _run_online("plain", tmp_path)
    assert all(s == "ok" for s, _ in got.values()), got
    a, b = got[0][1], got[1][1]
    assert len(a["result"]) == len(b["result"]) == 12 and a["model"].endswith("ftrl_S0") and b["model"].endswith("ftrl_S1")
    rec = a["sched"][0]
    assert b["sched"] is None and rec["examples"] == 2400 and rec["nnz_w"] == 30
    want = 2 * sum((0.6 - 0.02 * s) * 100 for s in range(12)) + 0.5 + 1.5
    assert rec["objv"] == pytest.approx(want, rel=1e-9)
    assert len(rec["reports"]) == 24 and {r["worker"] for r in rec["reports"]} == {"W0", "W1"}
    pat = re.compile(r"^\s*(\d+) examples, loss (\S+), penalty (\S+), \|w\|_0\s+(\d+)$")
    got_lines = [pat.match(l) for l in rec["lines"]]
    assert got_lines and all(got_lines)
    last = got_lines[-1]
    assert float(last.group(3)) == pytest.approx(2.0) and int(last.group(4)) == 30 and 0.3 < float(last.group(2)) < 0.7


def test_online_job_failure_reaches_the_scheduler(tmp_path):
    got = _run_online("fail", tmp_path)
    assert got[0][0] == "error" and ("table full" in got[0][1] or "peer 1 silent" in got[0][1])   # the scheduler's rank
    assert got[1][0] == "error" and "table full" in got[1][1]


def test_online_job_does_not_hang_when_a_rank_vanishes(tmp_path):
    got = _run_online("vanish", tmp_path, expect=1)
    assert got[0][0] == "error" and ("W0:" in got[0][1] or "no heartbeat" in got[0][1] or "task failed" in got[0][1]), got
