"""Local launcher: starts 1 scheduler + S servers + W workers as processes on this machine,
like the reference's ``script/local.sh`` (rank 0 = scheduler ``H`` on 127.0.0.1), or — with
``-gpus N`` — one rank per GPU through ``torch.distributed.run``.

  python -m parameter_server_b200.launch -num_servers 2 -num_workers 2 -app config/rcv1_l1lr.conf
  python -m parameter_server_b200.launch -gpus 8 -app config/ctr_ftrl.conf
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


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    flags, _ = cfg.Flags.parse(args)
    if flags.gpus > 0:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={flags.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", "parameter_server_b200.ps", *args]
        return subprocess.call(cmd)
    port = free_port()
    sched = f"role:SCHEDULER,hostname:'127.0.0.1',port:{port},id:'H'"
    n = 1 + flags.num_workers + flags.num_servers
    procs = []
    for r in range(n):
        cmd = [sys.executable, "-m", "parameter_server_b200.ps", *args, "-my_rank", str(r), "-scheduler", sched]
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
