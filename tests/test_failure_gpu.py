"""Failure detection on the device side without faulting a GPU: a cross-GPU wait that nothing will ever
satisfy runs out after its (short) limit, the kernel records where it gave up and returns, the host
raises from the status word, and the context and the engine stay usable."""
import time

import pytest
import torch

from parameter_server_b200.data.synthetic import ctr_minibatch

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_context_survives():
    from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper
    from parameter_server_b200.parallel.peer import PeerGroup

    eng = FTRLEngine(PeerGroup.single(torch.device("cuda", 0)), FTRLHyper(), table_capacity=1 << 14, max_rows=512,
                     max_nnz=1 << 16, local_capacity=1 << 14, timeout_s=0.25)
    off, keys, y = ctr_minibatch(200, seed=1, device="cuda", key_space_log2=12)
    mb = DeviceMinibatch(off, keys, y)
    eng.step(mb)
    eng.check_status()
    # pretend a whole step of some owner was lost: the next pull waits for "applied >= epoch-1" that never comes
    eng.epoch += 1
    t0 = time.time()
    eng.step(mb)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.2 < waited < 5.0
    with pytest.raises(RuntimeError, match="wait timed out"):
        eng.check_status()
    st = eng.status.tolist()
    assert st[0] == 1 and st[2] == 1           # code = wait timeout, phase 1 = pull waiting for the owners
    # the context is alive: plain work and a fresh engine still run
    assert torch.arange(10, device="cuda").sum().item() == 45
    eng2 = FTRLEngine(PeerGroup.single(torch.device("cuda", 0)), FTRLHyper(), table_capacity=1 << 14, max_rows=512,
                      max_nnz=1 << 16, local_capacity=1 << 14)
    eng2.step(mb)
    eng2.check_status()
    assert eng2.read_stats()["rows"] == 200
