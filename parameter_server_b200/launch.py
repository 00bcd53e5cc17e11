"""Local launcher: starts 1 scheduler + S servers + W workers as processes on this machine,
like the reference's ``script/local.sh`` (rank 0 = scheduler ``H`` on 127.0.0.1), or — with
``-gpus N`` — one rank per GPU through ``torch.distributed.run``.

  python -m parameter_server_b200.launch -num_servers 2 -num_workers 2 -app config/rcv1_l1lr.conf
  python -m parameter_server_b200.launch -gpus 8 -app config/ctr_ftrl.conf
  python -m parameter_server_b200.launch -mpi_hostfile hosts -num_servers 2 -num_workers 2 -app job.conf   # mpirun over machines
"""
from __future__ import annotations

import socket
import subprocess
import sys

from . import config as cfg


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def mpi_command(args, flags, hostfile: str) -> list:
    """``mpirun`` line for a job over the machines of ``hostfile`` (script/mpi_root.sh:1-31, script/mpi_node.sh:1-56):
    1 + S + W ranks, every rank runs the node command and takes its rank from the MPI environment; rank 0, the
    scheduler, starts on this machine, whose address (``-interface``, or the first interface that is up) goes into
    ``-scheduler`` unless the caller gave one."""
    from .runtime import host

    n = 1 + flags.num_workers + flags.num_servers + max(int(flags.num_unused), 0)
    cmd = ["mpirun", "-np", str(n), "--hostfile", hostfile, sys.executable, "-m", "parameter_server_b200.ps", *args]
    if not any(a.lstrip("-").split("=")[0] == "scheduler" for a in args):
        ip = host().local_ip(flags.interface or "")
        if not ip:
            raise RuntimeError("no network interface with an IPv4 address for the scheduler")
        cmd += ["-scheduler", f"role:SCHEDULER,hostname:'{ip}',port:{free_port()},id:'H'"]
    return cmd


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    hostfile = ""
    for i, a in enumerate(args):                      # -mpi_hostfile FILE belongs to the launcher, not to the nodes
        if a.lstrip("-") == "mpi_hostfile" and i + 1 < len(args):
            hostfile = args[i + 1]
            del args[i:i + 2]
            break
    flags, _ = cfg.Flags.parse(args)
    if flags.gpus > 0:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={flags.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", "parameter_server_b200.ps", *args]
        return subprocess.call(cmd)
    if hostfile:
        return subprocess.call(mpi_command(args, flags, hostfile))
    # the scheduler's address: the caller's -scheduler, else the loopback with a free port
    given = any(a.lstrip("-").split("=")[0] == "scheduler" for a in args)
    extra = [] if given else ["-scheduler", f"role:SCHEDULER,hostname:'127.0.0.1',port:{free_port()},id:'H'"]
    n = 1 + flags.num_workers + flags.num_servers + max(int(flags.num_unused), 0)
    procs = []
    for r in range(n):
        cmd = [sys.executable, "-m", "parameter_server_b200.ps", *args, "-my_rank", str(r), *extra]
        procs.append(subprocess.Popen(cmd))
    # wait for all of them; when one fails the job cannot finish, so the others (exactly these children) are stopped
    import time

    rc = 0
    alive = list(procs)
    while alive:
        for p in list(alive):
            code = p.poll()
            if code is None:
                continue
            alive.remove(p)
            if code != 0 and rc == 0:
                rc = code
                for q in alive:
                    q.terminate()
        time.sleep(0.05)
    return rc


if __name__ == "__main__":
    sys.exit(main())
