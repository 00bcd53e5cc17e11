"""Child process of the multi-GPU DARLIN test: every rank owns a rows shard and a key range;
rank 0 replays the run on the fp64 oracle with the same shards and compares per-pass progress
and the merged model.  Exit code 0 = match."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from baseline.cpu_ref.darlin_ref import DarlinConfig as RefConfig  # noqa: E402
from baseline.cpu_ref.darlin_ref import DarlinRef  # noqa: E402
from parameter_server_b200.data.synthetic import zipf_sparse_matrix  # noqa: E402
from parameter_server_b200.models.darlin import DarlinConfig, DarlinSolver  # noqa: E402
from parameter_server_b200.parallel.peer import PeerGroup  # noqa: E402


def shard(off, keys, vals, y, r, W):
    n = y.numel()
    r0, r1 = n * r // W, n * (r + 1) // W
    p0, p1 = int(off[r0].item()), int(off[r1].item())
    return (off[r0:r1 + 1] - p0).contiguous(), keys[p0:p1].contiguous(), None if vals is None else vals[p0:p1].contiguous(), y[r0:r1].contiguous()


def filter_tail(shards, W, freq, k=2, ratio=2.0):
    """NumPy restatement of the tail-feature filter: W servers split the key space evenly; each adds the
    workers' (key, count) lists to its count-min sketch in rank order, then keys with estimate <= freq go."""
    import math

    from baseline.cpu_ref.ftrl_ref import CountMinRef
    from parameter_server_b200.utils.range import Range

    seps = Range.all().separators(W)
    uniq = [np.unique(sh[1], return_inverse=True, return_counts=True) for sh in shards]
    keep = [np.zeros(len(u[0]), dtype=bool) for u in uniq]
    for s in range(W):
        lo, hi = np.uint64(seps[s]), np.uint64(min(seps[s + 1], (1 << 64) - 1))
        parts = [(u[0] >= lo) & (u[0] < hi) for u in uniq]
        n_first = next((int(m.sum()) for m in parts if m.any()), 0)
        cm = CountMinRef(max(int(W * n_first * ratio / math.log(W + 1)), 64), k)
        for u, m in zip(uniq, parts):
            if m.any():
                cm.insert(u[0][m], u[2][m])
        for u, m, kp in zip(uniq, parts, keep):
            if m.any():
                kp[m] = cm.query(u[0][m]) > freq
    out = []
    for (o, kk, vv, yy), u, kp in zip(shards, uniq, keep):
        sel = kp[u[1]]
        row_of = np.repeat(np.arange(len(yy)), np.diff(o))
        no = np.concatenate([[0], np.cumsum(np.bincount(row_of[sel], minlength=len(yy)))]).astype(np.int64)
        out.append((no, kk[sel], vv[sel], yy))
    return out, sum(int((~kp).sum()) for kp in keep)


def main():
    impl = sys.argv[1] if len(sys.argv) > 1 else "fused"
    tail = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    delay = int(sys.argv[3]) if len(sys.argv) > 3 else 0        # bounded delay tau
    streamed = len(sys.argv) > 4 and sys.argv[4] == "ooc"       # also run with the blocks streamed from host memory
    listed = len(sys.argv) > 5 and sys.argv[5] == "list"        # force the bulk-transfer path of very wide groups
    group = PeerGroup.from_env()
    rank, W, dev = group.rank, group.world, group.device
    off, idx, vals, y, _ = zipf_sparse_matrix(2400, 3000, 14, seed=5, device=dev, zipf_s=0.8)
    keys = idx * 104729 + 11
    kw = dict(lambda1=0.3, max_pass=5, feature_block_ratio=1.0, seed=2, max_block_delay=delay)
    sol = DarlinSolver(group, DarlinConfig(tail_feature_freq=tail, **kw), impl=impl,
                       **(dict(list_block_cols=1, gather_small_groups=False) if listed else {}))
    sol.preprocess(*shard(off, keys, vals, y, rank, W))
    prog = sol.run()
    sol.check_status()
    k, w = sol.model()
    same_streamed = True
    if streamed:
        # every rank streams the blocks of its own rows; the batches are whole synchronisation groups on all ranks
        ooc = DarlinSolver(group, DarlinConfig(tail_feature_freq=tail, **kw), impl=impl, out_of_core=True, prefetch_depth=2,
                           blocks_per_launch=3 + rank,      # the ranks ask for different batch sizes and must agree
                           wide_block_cols=1 if rank == 0 else 0)   # and rank 0 takes the two-step path for every group
        ooc.preprocess(*shard(off, keys, vals, y, rank, W))
        prog2 = ooc.run()
        ooc.check_status()
        same_streamed = len(prog2) == len(prog) and ooc.h2d_bytes > 0 and ooc.kernel_launches > len(prog2)
        for a, b in zip(prog, prog2):
            same_streamed &= abs(b.objv / a.objv - 1) < 1e-4 and abs(a.nnz_w - b.nnz_w) <= 2
    gathered = [None] * W
    dist.all_gather_object(gathered, (k, w), group=group.group)
    ok = bool(same_streamed)
    if rank == 0:
        shards = []
        for r in range(W):
            o, kk, vv, yy = shard(off, keys, vals, y, r, W)
            shards.append((o.cpu().numpy(), kk.cpu().numpy().view(np.uint64), vv.cpu().numpy(), yy.cpu().numpy()))
        dropped = 0
        if tail > 0:
            shards, dropped = filter_tail(shards, W, tail)
            ok &= dropped > 0
        ref = DarlinRef(shards, None, RefConfig(**kw))
        rprog = ref.run()
        ok &= len(prog) == len(rprog)
        for p, q in zip(prog, rprog):
            ok &= abs(p.objv / q.objv - 1) < 2e-3 and abs(p.nnz_w - q.nnz_w) <= max(3, 0.03 * q.nnz_w)
        allk = np.concatenate([g[0] for g in gathered])
        allw = np.concatenate([g[1] for g in gathered])
        ok &= all(bool(np.all(np.diff(g[0].astype(np.float64)) > 0)) for g in gathered if len(g[0]) > 1)   # ascending per shard
        ok &= len(np.unique(allk)) == len(allk)                         # shards are disjoint
        rk, rw = ref.model()
        common = np.intersect1d(allk, rk)
        ok &= len(common) >= 0.95 * max(len(allk), len(rk))
        wd, rd = dict(zip(allk.tolist(), allw.tolist())), dict(zip(rk.tolist(), rw.tolist()))
        ok &= max(abs(wd[c] - rd[c]) for c in common.tolist()) < 5e-2
        print(f"impl={impl} tail={tail} delay={delay} streamed={streamed} listed={listed} dropped={dropped} world={W} passes={len(prog)} objv={prog[-1].objv:.4f} ref={rprog[-1].objv:.4f} "
              f"shard_sizes={[len(g[0]) for g in gathered]} match={bool(ok)}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0, group=group.group)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
