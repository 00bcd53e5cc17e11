"""Fused push/pull over peer memory on 2+ GPUs == NCCL baseline == fp64 oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(nproc, impl, port, rule="count", tail=0):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_ftrl_worker.py"), impl,
           rule, str(tail)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("impl,rule,tail", [("fused", "count", 0), ("nccl", "count", 0), ("fused", "sumsq", 0),
                                            ("fused", "count", 3), ("nccl", "count", 3)])
def test_two_gpus_match_oracle(impl, rule, tail):
    r = _launch(2, impl, 29541 + (impl == "nccl") + 2 * (rule == "sumsq") + 4 * (tail > 0), rule, tail)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "match=True" in r.stdout


def test_all_gpus_match_oracle():
    import torch

    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip("needs >= 4 GPUs")
    r = _launch(n, "fused", 29549, "sumsq")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "match=True" in r.stdout
