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


def main(argv=None) -> int:
    flags, rest = cfg.Flags.parse(list(sys.argv[1:] if argv is None else argv))
    if flags.gpus > 0 or "LOCAL_RANK" in os.environ:
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

    run_node(flags.my_rank, flags, verbose=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
