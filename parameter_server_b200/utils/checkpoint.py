"""Checkpoint / resume of solver state, one file per rank.

The reference only writes the text model at the end of a job and cannot resume training
(``ParameterInitConfig::FILE`` aborts, src/base/shared_array_inl.h:121-125; ``Call::RECOVER`` is a
no-op, src/linear_method/linear_method.cc:90-93).  Here every rank periodically saves its server
shard (weights, trust regions, active set), its worker state (margins, local weights, trust
regions, active set) and the scheduler state (pass number, KKT threshold, progress so far); a job
restarted with the same ``-checkpoint_dir`` continues after the last complete pass.  The block
order of every pass is a function of (seed, pass), so it needs no saving.
"""
from __future__ import annotations

import os
import sys
from typing import List

import torch


def _path(directory: str, what: str, rank: int, step: int) -> str:
    return os.path.join(directory, f"{what}_rank{rank}_step{step}.pt")


def _latest(directory: str, what: str, rank: int) -> int:
    best = -1
    if os.path.isdir(directory):
        pre, suf = f"{what}_rank{rank}_step", ".pt"
        for n in os.listdir(directory):
            if n.startswith(pre) and n.endswith(suf):
                try:
                    best = max(best, int(n[len(pre):-len(suf)]))
                except ValueError:
                    pass
    return best


def _agree_on_step(group, step: int) -> int:
    """All ranks resume from the newest step that every rank has."""
    if group.world == 1:
        return step
    import torch.distributed as dist

    t = torch.tensor([step], dtype=torch.int64, device=group.device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group.group)
    return int(t.item())


# ------------------------------------------------------------------ DARLIN
def save_darlin(sol, directory: str, pass_idx: int, reset_flag: bool) -> str:
    os.makedirs(directory, exist_ok=True)
    state = {
        "pass": pass_idx, "reset": reset_flag, "kkt_threshold": sol.kkt_threshold,
        "progress": [p.__dict__ for p in sol.progress],
        "srv_w": sol.srv_w.local.cpu(), "srv_delta": sol.srv_delta.cpu(), "srv_active": sol.srv_active.cpu(),
        "margin": sol.margin.cpu(), "w": sol.w.cpu(), "delta": sol.delta.cpu(), "active": sol.active.cpu(),
        "skeys": sol.skeys.cpu(), "lkeys": sol.lkeys.cpu(),
    }
    path = _path(directory, "darlin", sol.group.rank, pass_idx)
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)               # a file is either absent or complete
    return path


def load_darlin(sol, directory: str, pass_idx: int):
    from ..models.darlin import Progress

    st = torch.load(_path(directory, "darlin", sol.group.rank, pass_idx), map_location="cpu", weights_only=False)
    if not (torch.equal(st["skeys"], sol.skeys.cpu()) and torch.equal(st["lkeys"], sol.lkeys.cpu())):
        raise RuntimeError("checkpoint was written for different data or a different number of ranks")
    dev = sol.dev
    sol.srv_w.local.copy_(st["srv_w"].to(dev))
    sol.srv_delta.copy_(st["srv_delta"].to(dev))
    sol.srv_active.copy_(st["srv_active"].to(dev))
    sol.margin.copy_(st["margin"].to(dev))
    sol.w.copy_(st["w"].to(dev))
    sol.delta.copy_(st["delta"].to(dev))
    sol.active.copy_(st["active"].to(dev))
    sol.kkt_threshold = st["kkt_threshold"]
    sol.progress = [Progress(**p) for p in st["progress"]]
    sol.group.barrier()
    return st["pass"], st["reset"]


def run_with_checkpoints(sol, directory: str, interval: int = 1, verbose: bool = False) -> List:
    """``DarlinSolver.run`` with a checkpoint every ``interval`` passes and resume from the newest one."""
    from ..models.darlin import block_order, print_progress

    cfg = sol.cfg
    orders = block_order(sol.nblk, cfg.max_pass, cfg.random_block_order, cfg.seed)
    start, reset = 0, False
    last = _agree_on_step(sol.group, _latest(directory, "darlin", sol.group.rank))
    if last >= 0:
        done, reset = load_darlin(sol, directory, last)
        start = done + 1
        if sol.group.rank == 0:
            print(f"resumed after pass {done} from {directory}", file=sys.stderr)
    for it in range(start, cfg.max_pass):
        p = sol.run_pass(orders[it], reset)
        if verbose and sol.group.rank == 0:
            print_progress(it, p, file=sys.stderr)
        stop = False
        if 0 < p.relative_objv <= cfg.epsilon:
            stop = reset
            reset = True
        else:
            reset = False
        if (it + 1) % max(interval, 1) == 0 or stop or it + 1 == cfg.max_pass:
            save_darlin(sol, directory, it, reset)
        if stop:
            break
    return sol.progress


# ------------------------------------------------------------------ FTRL
def save_ftrl(eng, directory: str, step: int) -> str:
    os.makedirs(directory, exist_ok=True)
    path = _path(directory, "ftrl", eng.group.rank, step)
    tmp = path + ".tmp"
    sketch = eng.cm.cpu() if getattr(eng, "cm", None) is not None else None
    # plain tensors, numbers and strings only, so that the file loads with weights_only=True
    torch.save({"step": step, "cap": eng.cap, "seps": [int(x) for x in eng.seps], "hyper": dict(eng.hyper.__dict__),
                "epoch": int(eng.epoch), "table": eng.tab.local.cpu(), "stats": eng.stats.cpu(), "sketch": sketch}, tmp)
    os.replace(tmp, path)
    return path


def load_ftrl(eng, directory: str, step: int = -1) -> int:
    """Restore this rank's shard; returns the step stored in the checkpoint (-1 if none exists)."""
    if step < 0:
        step = _agree_on_step(eng.group, _latest(directory, "ftrl", eng.group.rank))
    if step < 0:
        return -1
    st = torch.load(_path(directory, "ftrl", eng.group.rank, step), map_location="cpu", weights_only=True)
    if [int(x) for x in st["seps"]] != [int(x) for x in eng.seps]:
        raise RuntimeError("checkpoint was written with a different key-range partition")
    eng._set_table(st["table"].to(eng.dev))      # whatever size the table had grown to
    eng.stats.copy_(st["stats"].to(eng.dev))
    if st.get("sketch") is not None and getattr(eng, "cm", None) is not None:
        if st["sketch"].numel() != eng.cm.numel():
            raise RuntimeError("checkpoint was written with a different count-min width")
        eng.cm.copy_(st["sketch"].to(eng.dev))
    # fresh and used engines continue in step: flag words and sequence numbers restart from zero everywhere
    eng.epoch = int(st.get("epoch", 0))
    eng.reset_protocol()
    return st["step"]
