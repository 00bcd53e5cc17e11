"""Command line entry of one node, with the flag surface of the reference's ``ps_cdn`` binary:

  python -m parameter_server_b200.ps -num_servers 2 -num_workers 2 -my_rank 0 \
      -scheduler "role:SCHEDULER,hostname:'127.0.0.1',port:2060,id:'H'" -app config/rcv1_l1lr.conf

CPU nodes talk over TCP (src/ps.cc:5-16, src/system/postoffice.cc:34-84); under ``mpirun -np 1+S+W`` the rank
is taken from the launcher's environment like the reference's MPI scripts do.  With ``-gpus N`` (or under
``torch.distributed.run``) the job runs on the GPU engines instead: every rank is worker + server on
one B200 and the same ``.conf`` selects DARLIN or FTRL.
"""
from __future__ import annotations

import os
import sys

from . import config as cfg


def node_name(rank: int, num_workers: int, num_servers: int) -> str:
    """Node id of a CPU rank: 0 = scheduler H, then W0.., S0.., U0.. (src/system/van.cc:250-260)."""
    if rank == 0:
        return "H"
    if rank <= num_workers:
        return f"W{rank - 1}"
    if rank <= num_workers + num_servers:
        return f"S{rank - num_workers - 1}"
    return f"U{rank - num_workers - num_servers - 1}"


def redirect_logs(name: str, to_file: bool, instant: bool) -> str:
    """``-log_to_file``: everything this process writes to stderr (progress tables, runtime messages, native code
    included) goes to ``./log_<node>_<date>-<time>.<pid>`` like glog's files (src/system/postoffice.cc:40-43).
    ``-log_instant``: log output is not buffered (src/ps.cc:3,11).  Returns the file name, or ""."""
    import time

    path = ""
    if to_file:
        path = f"./log_{name}_{time.strftime('%Y%m%d-%H%M%S')}.{os.getpid()}"
        fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o644)
        sys.stderr.flush()
        os.dup2(fd, 2)
        os.close(fd)
    if instant or to_file:
        sys.stderr.reconfigure(line_buffering=True)
        if instant:
            sys.stdout.reconfigure(line_buffering=True)
    return path


def main(argv=None) -> int:
    flags, rest = cfg.Flags.parse(list(sys.argv[1:] if argv is None else argv))
    if flags.gpus > 0 or "LOCAL_RANK" in os.environ:
        redirect_logs(f"G{os.environ.get('RANK', '0')}", bool(flags.log_to_file), bool(flags.log_instant))
        from .apps.gpu_job import run_gpu_job

        try:
            run_gpu_job(flags)
        finally:
            try:
                import torch.distributed as dist

                if dist.is_initialized():
                    dist.destroy_process_group()
            except Exception:
                pass
        return 0
    if flags.my_rank < 0:
        # under mpirun / srun the rank comes from the launcher's environment (script/mpi_node.sh:8-17)
        for var in ("PMI_RANK", "OMPI_COMM_WORLD_RANK", "SLURM_PROCID"):
            if os.environ.get(var, "").isdigit():
                flags.my_rank = int(os.environ[var])
                break
    if flags.my_rank < 0:
        print("-my_rank is required (or PMI_RANK / OMPI_COMM_WORLD_RANK / SLURM_PROCID in the environment)", file=sys.stderr)
        return 2
    from .apps.job import run_node

    redirect_logs(node_name(flags.my_rank, int(flags.num_workers), int(flags.num_servers)), bool(flags.log_to_file),
                  bool(flags.log_instant))
    if bool(flags.verbose):
        from .runtime import host

        host().set_verbose(True)          # executors narrate every message they process
    run_node(flags.my_rank, flags, verbose=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
