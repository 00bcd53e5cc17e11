"""Child process of the multi-GPU DeviceKVVector test: every rank pushes its own (key, value) rows twice,
then pulls; the pulled rows must equal the sum over all ranks' pushes (computed on rank 0 from gathered inputs)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from parameter_server_b200.parallel.kv_vector import DeviceKVVector  # noqa: E402
from parameter_server_b200.parallel.peer import PeerGroup  # noqa: E402


def main():
    impl, k = sys.argv[1], int(sys.argv[2])
    group = PeerGroup.from_env()
    rank, W, dev = group.rank, group.world, group.device
    rng = np.random.RandomState(5)
    universe = np.unique(rng.randint(0, 2**63, size=6000, dtype=np.int64).astype(np.uint64) * 2 + 1)
    mine = np.sort(np.random.RandomState(10 + rank).choice(universe, 2500, replace=False))
    keys = torch.from_numpy(mine.view(np.int64)).to(dev)
    kv = DeviceKVVector(group, k=k, impl=impl)
    kv.set_keys(kv.merge_keys(keys))
    owner, slot = kv.resolve(keys)
    assert (slot >= 0).all()
    lo, hi = kv.seps[rank], kv.seps[rank + 1]
    lk = kv.local_keys.cpu().numpy().view(np.uint64)
    assert np.all((lk >= np.uint64(lo)) & (lk < np.uint64(min(hi, 2**64 - 1)))) and np.all(np.diff(lk.astype(np.float64)) > 0)
    vals = torch.randn(len(mine), k, generator=torch.Generator().manual_seed(rank)).to(dev)
    kv.push(owner, slot, vals)
    kv.push(owner, slot, vals)
    group.barrier()                         # every rank's pushes have landed
    out = kv.pull(owner, slot).cpu().numpy()
    gathered = [None] * W
    dist.all_gather_object(gathered, (mine, vals.cpu().numpy(), out), group=group.group)
    ok = True
    if rank == 0:
        total = {}
        for m, v, _ in gathered:
            for kk, vv in zip(m.tolist(), v):
                total[kk] = total.get(kk, 0) + 2 * vv
        for m, _, o in gathered:
            want = np.stack([total[kk] for kk in m.tolist()])
            ok &= bool(np.allclose(o, want, rtol=1e-4, atol=1e-5))
        print(f"impl={impl} k={k} world={W} shard_sizes={kv.nkeys} match={ok}", flush=True)
    # scalar all-reduce inside a kernel (sums in fp64, maxima), with the box's multicast mapping when it has one
    # and with plain peer loads; several calls in a row alternate the two internal buffers
    from parameter_server_b200.parallel.scalar_reduce import ScalarAllReduce

    mine_ok, used_mc = True, []
    for use_mc in (True, False):
        red = ScalarAllReduce(group, timeout_s=5.0, use_multicast=use_mc)
        used_mc.append(red.multicast)
        for call in range(3):
            sums = torch.tensor([rank + 1.0, 0.5 * call, 1e-3 * (rank + 1), -2.0 * rank], dtype=torch.float64, device=dev)
            maxs = torch.tensor([float(rank), 3.0 - rank, 0.25 * call], dtype=torch.float32, device=dev)
            s_out, m_out = red(sums, maxs)
            want_s = [W * (W + 1) / 2.0, 0.5 * call * W, 1e-3 * W * (W + 1) / 2.0, -2.0 * W * (W - 1) / 2.0]
            want_m = [float(W - 1), 3.0, 0.25 * call]
            mine_ok &= bool(np.allclose(s_out.cpu().numpy(), want_s, rtol=1e-12, atol=1e-12))
            mine_ok &= bool(np.allclose(m_out.cpu().numpy(), want_m))
        red.check_status()
    if rank == 0:
        print(f"scalar all-reduce: multicast used {used_mc[0]}, match={mine_ok}", flush=True)
    ok = ok and mine_ok if rank == 0 else mine_ok
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group.group)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
