"""Failure detection on the device side without faulting a GPU: a cross-GPU wait that nothing will ever
satisfy runs out after its (short) limit, the kernel records where it gave up and returns, the host
raises from the status word, and the context and the engine stay usable.

The peer that never answers is a stand-in: a group of two ranks whose second rank exists only as
buffers on this GPU (valid memory, but no process ever runs its kernels or sets its flags)."""
import time

import pytest
import torch

from parameter_server_b200.data.synthetic import ctr_minibatch

pytestmark = pytest.mark.gpu


def _silent_peer_group():
    from parameter_server_b200.parallel.peer import PeerGroup, SymmetricBuffer

    class SilentPeerGroup(PeerGroup):
        """Rank 0 of a world of 2; rank 1's copy of every buffer is a second tensor on this GPU."""

        def alloc(self, shape, dtype, fill=0):
            mine = torch.empty(shape, dtype=dtype, device=self.device).fill_(fill)
            ghost = torch.empty(shape, dtype=dtype, device=self.device).fill_(fill)
            buf = SymmetricBuffer(mine, [mine.data_ptr(), ghost.data_ptr()], ghost)
            self._buffers.append(buf)
            return buf

        def barrier(self):
            torch.cuda.synchronize(self.device)

    return SilentPeerGroup(0, 2, torch.device("cuda", 0))


def test_bounded_wait_expires_and_context_survives():
    from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper
    from parameter_server_b200.parallel.peer import PeerGroup

    eng = FTRLEngine(_silent_peer_group(), FTRLHyper(), table_capacity=1 << 14, max_rows=512, max_nnz=1 << 16,
                     local_capacity=1 << 14, timeout_s=0.25)
    off, keys, y = ctr_minibatch(200, seed=1, device="cuda", key_space_log2=12)
    mb = DeviceMinibatch(off, keys, y)
    t0 = time.time()
    eng.step(mb)            # the owner side of the pull waits for rank 1's table, which never comes
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 0.2 < waited < 10.0
    with pytest.raises(RuntimeError, match="wait timed out"):
        eng.check_status()
    st = eng.status.tolist()
    assert st[0] == 1 and st[1] == 1 and st[2] in (1, 2, 3)    # wait timeout, peer 1, a phase of the pull or the push
    # the context is alive: plain work and a fresh engine still run
    assert torch.arange(10, device="cuda").sum().item() == 45
    eng2 = FTRLEngine(PeerGroup.single(torch.device("cuda", 0)), FTRLHyper(), table_capacity=1 << 14, max_rows=512,
                      max_nnz=1 << 16, local_capacity=1 << 14)
    eng2.step(mb)
    eng2.check_status()
    assert eng2.read_stats()["rows"] == 200
