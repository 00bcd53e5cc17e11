"""DeviceKVVector on one GPU (fused and NCCL-baseline code paths) against a dictionary model."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("impl", ["fused", "nccl"])
@pytest.mark.parametrize("k", [1, 3, 8])
def test_push_pull_roundtrip(impl, k):
    from parameter_server_b200.parallel.kv_vector import DeviceKVVector
    from parameter_server_b200.parallel.peer import PeerGroup

    rng = np.random.RandomState(k)
    server = np.unique(rng.randint(0, 2**62, size=5000).astype(np.uint64) * 3)
    kv = DeviceKVVector(PeerGroup.single(torch.device("cuda", 0)), k=k, impl=impl)
    mine = kv.merge_keys(torch.from_numpy(server.view(np.int64)).cuda())
    assert np.array_equal(mine.cpu().numpy().view(np.uint64), server)
    kv.set_keys(mine)
    q = np.concatenate([rng.choice(server, 3000, replace=False), np.array([1, 2], dtype=np.uint64)])   # two unknown keys
    owner, slot = kv.resolve(torch.from_numpy(q.view(np.int64)).cuda())
    assert (slot[-2:] == -1).all() and (slot[:-2] >= 0).all() and (owner == 0).all()
    assert np.array_equal(server[slot[:-2].cpu().numpy()], q[:-2])
    v1 = torch.randn(len(q), k, device="cuda")
    kv.push(owner, slot, v1)
    kv.push(owner, slot, v1)                          # pushes accumulate
    out = kv.pull(owner, slot)
    torch.testing.assert_close(out[:-2], 2 * v1[:-2])
    assert (out[-2:] == 0).all()
    assert kv.local_values.abs().sum().item() == pytest.approx((2 * v1[:-2]).abs().sum().item(), rel=1e-4)
