"""Addresses of CPU nodes: a job whose scheduler is not on the loopback makes every node advertise the address of a
real interface (-interface, or the first one that is up), so that nodes on other machines can reach it."""
import os
import socket
import subprocess
import sys

import pytest

from parameter_server_b200.data.synthetic import write_libsvm_parts
from parameter_server_b200.runtime import host
from parameter_server_b200.runtime.node import advertised_address
from parameter_server_b200.utils.modelio import read_model_text
from test_cpu_job import CONF, planted
from test_rank_monitor import _free_port


def test_interface_table():
    H = host()
    table = H.interfaces()
    assert table and table[-1][1].startswith("127.")                  # loopback last
    assert H.local_ip(table[0][0]) == table[0][1] and H.local_ip("no_such_if0") == ""
    assert advertised_address("127.0.0.1") == "127.0.0.1"             # single-machine job stays on the loopback
    assert advertised_address("10.1.2.3") == H.local_ip("")
    assert advertised_address("127.0.0.1", table[0][0]) == table[0][1]
    with pytest.raises(ValueError):
        advertised_address("10.1.2.3", "no_such_if0")


def test_job_over_a_real_interface(tmp_path):
    ip = host().local_ip("")
    if not ip or ip.startswith("127."):
        pytest.skip("no interface besides the loopback")
    off, idx, vals, y = planted(600, 512, 8, 2, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=0.5, passes=2, tail=0))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sched = f"role:SCHEDULER,hostname:'{ip}',port:{_free_port()},id:'H'"
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "2", "-num_workers", "2",
                        "-app", str(conf), "-scheduler", sched, "-print_van", "-parallel_match", "-num_threads", "3"],
                       cwd=tmp_path, env=dict(os.environ, PYTHONPATH=root), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    model = {}
    for s_ in ("S0", "S1"):
        model.update(read_model_text(str(tmp_path / f"model_{s_}")))
    assert len(model) > 10
    log = open(tmp_path / "van_W0").read()                              # -print_van: the worker's message log
    assert "S0" in log and "S1" in log


FAKE_MPIRUN = r'''#!/bin/sh
# stand-in for mpirun: -np N --hostfile F cmd... -> N local processes with PMI_RANK set
[ "$1" = "-np" ] || exit 2
n=$2; shift 2
[ "$1" = "--hostfile" ] || exit 2
echo "$2" > "$FAKE_MPI_LOG"; shift 2
echo "$@" >> "$FAKE_MPI_LOG"
pids=""
i=0
while [ $i -lt $n ]; do
  PMI_RANK=$i "$@" &
  pids="$pids $!"
  i=$((i+1))
done
rc=0
for p in $pids; do wait $p || rc=1; done
exit $rc
'''


def test_mpirun_launch(tmp_path):
    """-mpi_hostfile: one mpirun line starts all ranks; every rank reads its rank from the MPI environment and the
    scheduler's address is this machine's."""
    ip = host().local_ip("")
    bindir = tmp_path / "bin"
    bindir.mkdir()
    exe = bindir / "mpirun"
    exe.write_text(FAKE_MPIRUN)
    exe.chmod(0o755)
    (tmp_path / "hosts").write_text("localhost slots=8\n")
    off, idx, vals, y = planted(600, 512, 8, 2, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=0.5, passes=2, tail=0))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, PATH=str(bindir) + os.pathsep + os.environ["PATH"], FAKE_MPI_LOG=str(tmp_path / "mpi.log"))
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-mpi_hostfile", str(tmp_path / "hosts"),
                        "-num_servers", "1", "-num_workers", "2", "-app", str(conf)],
                       cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    hostfile, line = open(tmp_path / "mpi.log").read().splitlines()[:2]
    assert hostfile == str(tmp_path / "hosts")
    assert "parameter_server_b200.ps" in line and "-my_rank" not in line and f"hostname:'{ip}'" in line and "mpi_hostfile" not in line
    assert len(read_model_text(str(tmp_path / "model_S0"))) > 10


def test_mpi_conf_of_the_reference_launch_scripts(tmp_path):
    """-mpi_conf: the shell-assignment file that the reference's mpi_root.sh / mpi_node.sh read gives the node flags, the
    job file (relative to the conf), the scheduler's port and the host file."""
    from parameter_server_b200.launch import read_mpi_conf

    ip = host().local_ip("")
    bindir = tmp_path / "bin"
    bindir.mkdir()
    exe = bindir / "mpirun"
    exe.write_text(FAKE_MPIRUN)
    exe.chmod(0o755)
    (tmp_path / "hosts").write_text("localhost slots=8\n")
    off, idx, vals, y = planted(500, 512, 8, 4, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    (tmp_path / "job.conf").write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5,
                                                   ratio=0.5, passes=2, tail=0))
    port = socket.socket()
    port.bind(("127.0.0.1", 0))
    pnum = port.getsockname()[1]
    port.close()
    (tmp_path / "mpi.conf").write_text(f"""#!/bin/bash
num_workers=2
num_servers=1
num_threads=3     # per node
scheduler_network_interface=""
scheduler_network_port={pnum}
app_conf=job.conf
report_interval=0
verbose=""
print_van="-print_van"
parallel_match="-noparallel_match"
load_limit=0
hostfile=hosts
""")
    args, hostfile = read_mpi_conf(str(tmp_path / "mpi.conf"))
    assert hostfile == str(tmp_path / "hosts") and args[:6] == ["-num_workers", "2", "-num_servers", "1", "-num_threads", "3"]
    assert "-print_van" in args and "-noparallel_match" in args and "-verbose" not in args
    assert args[args.index("-app") + 1] == str(tmp_path / "job.conf") and f"port:{pnum}" in args[args.index("-scheduler") + 1]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, PATH=str(bindir) + os.pathsep + os.environ["PATH"], FAKE_MPI_LOG=str(tmp_path / "mpi.log"))
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-mpi_conf", str(tmp_path / "mpi.conf")],
                       cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    hostfile, line = open(tmp_path / "mpi.log").read().splitlines()[:2]
    assert hostfile == str(tmp_path / "hosts") and f"hostname:'{ip}',port:{pnum}" in line and "-mpi_conf" not in line
    assert len(read_model_text(str(tmp_path / "model_S0"))) > 10 and os.path.exists(tmp_path / "van_W0")


def test_stand_by_node_joins_and_leaves_with_the_job(tmp_path):
    """-num_unused 1: a stand-by node U0 registers, idles through the job and ends with it."""
    off, idx, vals, y = planted(400, 256, 8, 6, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 1)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=0.5, passes=2, tail=0))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "1", "-num_workers", "1", "-num_unused", "1",
                        "-app", str(conf), "-print_van"], cwd=tmp_path, env=dict(os.environ, PYTHONPATH=root), capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert (tmp_path / "model_S0").exists()
    log = open(tmp_path / "van_U0").read()                    # it talked to the scheduler: registration, node table, termination
    assert "U0=>H" in log and "H=>U0" in log


def _start_five(tmp_path, conf, sched, env):
    """1 scheduler + 2 workers + 2 servers as child processes with heartbeats on; the scheduler's stderr goes to H.err."""
    procs = []
    for r in range(5):
        err = open(tmp_path / "H.err", "w") if r == 0 else subprocess.DEVNULL
        procs.append(subprocess.Popen([sys.executable, "-m", "parameter_server_b200.ps", "-num_servers", "2", "-num_workers", "2",
                                       "-app", str(conf), "-scheduler", sched, "-my_rank", str(r), "-report_interval", "1"],
                                      cwd=tmp_path, env=env, stdout=subprocess.DEVNULL, stderr=err))
    return procs


def _wait_for_line(path, needle, procs, timeout_s=120.0):
    """Until the scheduler has printed a line with ``needle`` (the job is demonstrably running) or a process ended."""
    import time

    deadline = time.time() + timeout_s
    while time.time() < deadline:
        if needle in path.read_text():
            return
        if any(p.poll() is not None for p in procs):
            return
        time.sleep(0.2)
    raise AssertionError(f"no line with {needle!r} within {timeout_s:g} s:\n" + path.read_text()[-2000:])


def test_a_worker_process_that_dies_ends_the_job(tmp_path):
    """Failure detection on the host: five processes (1 + 2 + 2) over TCP with heartbeats on; one worker is ended by the
    test in the middle of the job.  The scheduler misses its reports, gives up with an error that names the node, and
    tells the others to terminate: nothing waits for ever."""
    import time

    off, idx, vals, y = planted(4000, 4096, 12, 9, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.01, ratio=8.0, passes=100000, tail=0)
                    .replace("epsilon: 1e-6", "epsilon: 1e-30"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sched = f"role:SCHEDULER,hostname:'127.0.0.1',port:{_free_port()},id:'H'"
    env = dict(os.environ, PYTHONPATH=root)
    procs = _start_five(tmp_path, conf, sched, env)                       # ranks: H, W0, W1, S0, S1
    try:
        _wait_for_line(tmp_path / "H.err", " 1 | ", procs)                # the passes are under way
        procs[2].kill()                                                   # W1: this child, by its own handle
        t0 = time.time()
        try:
            procs[0].wait(timeout=60)
        except subprocess.TimeoutExpired:
            pytest.fail("the scheduler kept waiting for the dead worker")
        err = (tmp_path / "H.err").read_text()
        assert procs[0].returncode != 0 and "no heartbeat from W1" in err, err[-2000:]
        assert time.time() - t0 < 30
        for i in (1, 3, 4):                                               # the survivors were told to terminate
            procs[i].wait(timeout=30)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


def test_a_worker_process_that_dies_ends_the_online_job(tmp_path):
    """The same for the online (FTRL) job: the scheduler's one long wait for UPDATE_MODEL notices the missing reports."""
    import shutil
    import time

    from test_cpu_ftrl_job import CONF as FTRL_CONF

    off, idx, vals, y = planted(10000, 4096, 10, 3, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 1)
    for i in range(1, 200):                                               # a long stream out of one small file
        shutil.copy(tmp_path / "train" / "part-000", tmp_path / "train" / f"part-{i:03d}")
    conf = tmp_path / "job.conf"
    conf.write_text(FTRL_CONF.format(train=tmp_path / "train", out=tmp_path, mb=100, tail=0).replace("eval_interval: 0", "eval_interval: 1"))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sched = f"role:SCHEDULER,hostname:'127.0.0.1',port:{_free_port()},id:'H'"
    env = dict(os.environ, PYTHONPATH=root)
    procs = _start_five(tmp_path, conf, sched, env)
    try:
        _wait_for_line(tmp_path / "H.err", " examples, loss ", procs)     # the workers are streaming
        if any(p.poll() is not None for p in procs):
            pytest.skip("the stream was over before the failure could be injected")
        procs[2].kill()                                                   # W1
        try:
            procs[0].wait(timeout=60)
        except subprocess.TimeoutExpired:
            pytest.fail("the scheduler kept waiting for the dead worker")
        err = (tmp_path / "H.err").read_text()
        assert procs[0].returncode != 0 and "no heartbeat from W1" in err, err[-2000:]
        for i in (1, 3, 4):
            procs[i].wait(timeout=60)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
