"""Local launcher: starts 1 scheduler + S servers + W workers as processes on this machine,
like the reference's ``script/local.sh`` (rank 0 = scheduler ``H`` on 127.0.0.1), or — with
``-gpus N`` — one rank per GPU through ``torch.distributed.run``.

  python -m parameter_server_b200.launch -num_servers 2 -num_workers 2 -app config/rcv1_l1lr.conf
  python -m parameter_server_b200.launch -gpus 8 -app config/ctr_ftrl.conf
  python -m parameter_server_b200.launch -mpi_hostfile hosts -num_servers 2 -num_workers 2 -app job.conf   # mpirun over machines
  python -m parameter_server_b200.launch -mpi_conf config/mpi.conf                                         # the reference's mpi.conf
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
    cmd = ["mpirun", "-np", str(n), *(["--hostfile", hostfile] if hostfile != "-" else []),
           sys.executable, "-m", "parameter_server_b200.ps", *args]
    if not any(a.lstrip("-").split("=")[0] == "scheduler" for a in args):
        ip = host().local_ip(flags.interface or "")
        if not ip:
            raise RuntimeError("no network interface with an IPv4 address for the scheduler")
        cmd += ["-scheduler", f"role:SCHEDULER,hostname:'{ip}',port:{free_port()},id:'H'"]
    return cmd


def read_mpi_conf(path: str) -> tuple:
    """The reference's ``mpi.conf`` (config/mpi.conf, read by script/mpi_root.sh and script/mpi_node.sh): shell
    assignments ``name=value``.  Returns (node arguments, hostfile or "").  ``num_workers / num_servers / num_threads /
    report_interval / load_limit / line_limit / prefetch_mem_limit_kb`` become ``-name value``; ``app_conf`` becomes
    ``-app`` (relative to the conf file, like the scripts); values that are flags themselves (``verbose="-verbose"``,
    ``parallel_match="-noparallel_match"`` ...) are passed on as they are; ``scheduler_network_interface`` becomes
    ``-interface`` and, with ``scheduler_network_port``, fixes the scheduler's address."""
    import os
    import shlex

    here = os.path.dirname(os.path.abspath(path))
    vals = {}
    with open(path) as f:
        for line in f:
            line = line.split("#", 1)[0].strip()
            if "=" not in line:
                continue
            name, v = line.split("=", 1)
            toks = shlex.split(v)
            vals[name.strip()] = toks[0] if toks else ""
    out = []
    for name in ("num_workers", "num_servers", "num_threads", "report_interval", "load_limit", "line_limit", "prefetch_mem_limit_kb"):
        if vals.get(name):
            out += [f"-{name}", vals[name]]
    if vals.get("app_conf"):
        out += ["-app", os.path.normpath(os.path.join(here, vals["app_conf"]))]
    for name in ("verbose", "log_to_file", "log_instant", "print_van", "shuffle_fea_id", "parallel_match", "mmap_training_data",
                 "prefetch_detail"):
        if vals.get(name, "").startswith("-"):
            out.append(vals[name])
    iface, port = vals.get("scheduler_network_interface", ""), vals.get("scheduler_network_port", "")
    if iface:
        out += ["-interface", iface]
    if port:
        from .runtime import host

        ip = host().local_ip(iface)
        if not ip:
            raise RuntimeError(f"mpi.conf: no IPv4 address on interface '{iface}'")
        out += ["-scheduler", f"role:SCHEDULER,hostname:'{ip}',port:{int(port)},id:'H'"]
    hostfile = vals.get("hostfile", "")
    return out, (os.path.normpath(os.path.join(here, hostfile)) if hostfile else "")


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    hostfile = ""
    for i, a in enumerate(args):                      # -mpi_conf FILE: the reference's mpi.conf; later arguments win
        if a.lstrip("-") == "mpi_conf" and i + 1 < len(args):
            conf_args, hostfile = read_mpi_conf(args[i + 1])
            args = conf_args + args[:i] + args[i + 2:]
            if not hostfile:
                hostfile = "-"                         # an MPI job on this machine only: mpirun without a host file
            break
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
