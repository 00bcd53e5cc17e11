"""Host-side liveness of the ranks of a GPU job.

The fused kernels never wait forever (every device wait is bounded and reports through the status word),
but a rank that is gone should be noticed *before* the next launch, on the host.  Every rank writes a
heartbeat ``(step, wall time)`` into the job's key-value store between steps; before launching, a rank
looks at the others: a rank that announced its departure, or whose heartbeat is older than the deadline, is
reported and the caller stops launching (``RankLost``).  This is the scheduler-side heartbeat table of the
reference (``Postoffice`` HEARTBEATING, src/system/postoffice.cc:245-269) with the dead-node action the
reference leaves out, for ranks that are peers instead of nodes under a scheduler.

The store is any ``torch.distributed`` store (the process group's own TCP store by default), so the same code
runs under ``gloo`` on CPU ranks, which is how it is tested.
"""
from __future__ import annotations

import time
from typing import List, Optional


class RankLost(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"rank(s) {ranks} lost ({reason}); stop launching and restart from the last checkpoint")
        self.ranks = ranks


def default_store():
    """The key-value store of the default process group, under a prefix of its own."""
    import torch.distributed as dist

    base = dist.distributed_c10d._get_default_store()
    return dist.PrefixStore("psb_monitor", base)


class RankMonitor:
    def __init__(self, rank: int, world: int, store=None, deadline_s: float = 10.0):
        self.rank, self.world, self.deadline_s = rank, world, deadline_s
        self.store = store if store is not None else default_store()
        self.step = -1
        self.beat(-1)

    def beat(self, step: Optional[int] = None) -> None:
        """Call between steps (nothing of this rank in flight)."""
        self.step = self.step + 1 if step is None else step
        self.store.set(f"hb/{self.rank}", f"{self.step}:{time.time():.6f}")

    def leave(self) -> None:
        """Announce an orderly departure (between steps) so that the others stop at once."""
        self.store.set(f"left/{self.rank}", "1")

    def lost(self) -> List[int]:
        """Ranks that left or whose last heartbeat is older than the deadline."""
        now, out = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([f"left/{r}"]):
                out.append(r)
                continue
            if not self.store.check([f"hb/{r}"]):
                continue                      # not started yet: the rendezvous covers start-up
            _, t = self.store.get(f"hb/{r}").decode().split(":")
            if now - float(t) > self.deadline_s:
                out.append(r)
        return out

    def tick(self, step: Optional[int] = None, interval_s: float = 1.0) -> None:
        """Per-step call for hot loops: heartbeat and look at the others at most every ``interval_s`` seconds
        (a look costs one store round trip per rank)."""
        now = time.time()
        if now - getattr(self, "_last_tick", 0.0) < interval_s:
            self.step = self.step + 1 if step is None else step
            return
        self._last_tick = now
        self.beat(step)
        self.check()

    def check(self) -> None:
        try:
            gone = self.lost()
            left = [r for r in gone if self.store.check([f"left/{r}"])]
        except RankLost:
            raise
        except Exception as e:  # noqa: BLE001 — the store lives in rank 0's process: unreachable = rank 0 is gone
            raise RankLost([0], f"store unreachable: {type(e).__name__}") from e
        if gone:
            raise RankLost(gone, "left the job" if left == gone else f"no heartbeat for {self.deadline_s:.1f} s")
