"""Peer-memory transport: symmetric device buffers reachable from every GPU of the box.

This replaces the reference's ZeroMQ ``Van`` data plane (src/system/van.cc:59-233)
on a single NVSwitch box.  Every rank allocates the same buffers; after a
rendezvous each rank knows the device address of every peer's copy, and kernels
read and write them directly (plain ``ld/st/red.global`` over NVLink).  No data
message is ever serialised, compressed or copied through the host.

With one rank the "peers" are the local buffers themselves, so the same kernels
serve single-GPU runs.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class SymmetricBuffer:
    local: torch.Tensor          # this rank's copy
    ptrs: List[int]              # device address of every rank's copy, by rank
    handle: object = None        # keeps the symmetric-memory mapping alive


@dataclass
class PeerGroup:
    rank: int = 0
    world: int = 1
    device: torch.device = field(default_factory=lambda: torch.device("cuda", 0))
    group: object = None
    _buffers: list = field(default_factory=list)
    numa: dict = field(default_factory=dict)   # what bind_to_gpu_node found / did for this rank

    @staticmethod
    def single(device: Optional[torch.device] = None) -> "PeerGroup":
        return PeerGroup(0, 1, device or torch.device("cuda", torch.cuda.current_device()))

    @staticmethod
    def from_env(backend: str = "nccl") -> "PeerGroup":
        """Join the process group described by RANK/LOCAL_RANK/WORLD_SIZE/MASTER_* (torchrun)."""
        import torch.distributed as dist

        from ..utils.numa import bind_to_gpu_node

        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            g = PeerGroup(0, 1, dev)
            g.numa = bind_to_gpu_node(dev.index)
            return g
        rank = int(os.environ["RANK"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        dev = torch.device("cuda", local)
        torch.cuda.set_device(dev)
        numa = bind_to_gpu_node(local)      # before any pinned buffer is allocated (PSB_NUMA_BIND=1)
        if not dist.is_initialized():
            dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=dev)
        g = PeerGroup(rank, world, dev, dist.group.WORLD)
        g.numa = numa
        return g

    # ------------------------------------------------------------------ memory
    def alloc(self, shape, dtype, fill=0) -> SymmetricBuffer:
        """Allocate a buffer that every rank of the group can address."""
        if self.world == 1:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            t.fill_(fill)
            buf = SymmetricBuffer(t, [t.data_ptr()])
        else:
            import torch.distributed._symmetric_memory as symm

            t = symm.empty(shape, dtype=dtype, device=self.device)
            t.fill_(fill)
            hdl = symm.rendezvous(t, group=self.group)
            buf = SymmetricBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl)
        self._buffers.append(buf)
        return buf

    def barrier(self) -> None:
        """Host-side barrier that also drains this rank's stream."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier(group=self.group, device_ids=[self.device.index])
            torch.cuda.synchronize(self.device)

    def all_reduce_max(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch.distributed as dist

        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def all_reduce_sum(self, values) -> list:
        if self.world == 1:
            return list(values)
        import torch.distributed as dist

        t = torch.tensor(list(values), dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t.tolist()
