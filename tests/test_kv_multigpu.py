"""DeviceKVVector push/pull over peer memory on 2+ GPUs: sums over workers land at the owners."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("impl,k,port", [("fused", 1, 29561), ("fused", 8, 29562), ("nccl", 3, 29563)])
def test_push_sums_across_workers(impl, k, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_kv_worker.py"), impl, str(k)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "match=True" in r.stdout
