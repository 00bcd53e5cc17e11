"""Child process of the multi-GPU FTRL tests (one rank per GPU, launched by torch.distributed.run).

Every rank trains on its own minibatches; rank 0 replays the same bulk-synchronous schedule on the
fp64 oracle (workers applied in rank order) and compares the merged model dump and per-step loss.
Exit code 0 = match.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from baseline.cpu_ref.ftrl_ref import FTRLRef  # noqa: E402
from parameter_server_b200.data.synthetic import ctr_minibatch  # noqa: E402
from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper  # noqa: E402
from parameter_server_b200.parallel.peer import PeerGroup  # noqa: E402


def main():
    impl = sys.argv[1] if len(sys.argv) > 1 else "fused"
    rule = sys.argv[2] if len(sys.argv) > 2 else "count"
    tail = int(sys.argv[3]) if len(sys.argv) > 3 else 0
    steps = 5
    group = PeerGroup.from_env()
    rank, world, dev = group.rank, group.world, group.device
    hy = FTRLHyper(alpha=0.02, beta=1.0, lambda1=0.05, lambda2=0.1, rule=rule, tail_feature_freq=tail,
                   countmin_n=1 << 14, countmin_k=2)
    eng = FTRLEngine(group, hy, table_capacity=1 << 16, max_rows=2048, max_nnz=1 << 18, local_capacity=1 << 16,
                     timeout_s=2.0, impl=impl)

    def batch(r, i):
        return ctr_minibatch(600, seed=7 + 100 * r + i, device=dev, key_space_log2=13, bias=-0.5, wstar_frac=0.2,
                             wstar_std=1.0)

    losses = []
    for i in range(steps):
        off, keys, y = batch(rank, i)
        eng.step(DeviceMinibatch(off, keys, y))
        st = eng.read_stats()
        eng.check_status()
        losses.append(st["loss_sum"])
    # predictions with the final model on a fresh batch (collective)
    off, keys, y = batch(0, 99)
    xw = eng.predict(DeviceMinibatch(off, keys, y)).cpu().numpy()
    eng.check_status()
    k, w = eng.dump_model()
    lo, hi = eng.seps[rank], eng.seps[rank + 1]
    assert all(lo <= int(x) < hi for x in k[:: max(1, len(k) // 64)]), "key outside this shard's range"
    gathered = [None] * world
    dist.all_gather_object(gathered, (k, w, losses), group=group.group)
    ok = True
    if rank == 0:
        ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, rule, tail_freq=tail, countmin_n=hy.countmin_n,
                      countmin_k=hy.countmin_k, seps=eng.seps)
        ref_losses = []
        for i in range(steps):
            mbs = []
            for r in range(world):
                o, kk, yy = batch(r, i)
                mbs.append((o.cpu().numpy(), kk.cpu().numpy().view(np.uint64), yy.cpu().numpy().astype(np.float64)))
            per = [ref.worker_gradient(*m)[4] for m in mbs]
            ref.step(mbs)
            ref_losses.append(per)
        rk, rw = ref.nonzero()
        allk = np.concatenate([g[0] for g in gathered])
        allw = np.concatenate([g[1] for g in gathered])
        order = np.argsort(allk, kind="stable")
        allk, allw = allk[order], allw[order]
        ok &= len(rk) > 50 and np.array_equal(allk, rk) and np.allclose(allw, rw, rtol=3e-3, atol=3e-5)
        for r in range(world):
            ok &= np.allclose(gathered[r][2], [p[r] for p in ref_losses], rtol=3e-4)
        _, _, _, _, _, rxw = ref.worker_gradient(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64),
                                                 y.cpu().numpy().astype(np.float64))
        ok &= np.allclose(xw, rxw, rtol=3e-3, atol=3e-4)
        sizes = [len(g[0]) for g in gathered]
        print(f"impl={impl} rule={rule} tail={tail} world={world} shards={sizes} model_nnz={len(rk)} "
              f"entries={len(ref.model)} match={ok}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0, group=group.group)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
