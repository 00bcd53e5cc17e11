"""Keep a rank's host threads and pinned buffers on the NUMA node its GPU hangs off.

A rank streams minibatches (tens of MB per step) from pinned host memory.  On a two-socket box a
process that runs — and therefore first-touches its pinned pages — on the other socket sends every
DMA read across the inter-socket link.  ``bind_to_gpu_node`` restricts the calling process to the
CPUs of the GPU's node before any buffer is allocated; with the default local allocation policy the
pinned pages then land on that node.  Everything here is best effort: without sysfs, with an unknown
node (-1) or with a cpuset that excludes the node's CPUs nothing is changed.

The reference pins worker threads only through ``-num_threads``; this is the GPU-box equivalent of
placing a worker next to its data (src/system/postoffice.cc:10-24 lists the thread flags).
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Set


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def parse_cpulist(text: str) -> Set[int]:
    """``"0-3,8,10-11"`` → {0,1,2,3,8,10,11}."""
    out: Set[int] = set()
    for part in text.split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            out.update(range(int(a), int(b) + 1))
        else:
            out.add(int(part))
    return out


def gpu_pci_address(device_index: int) -> Optional[str]:
    import torch

    try:
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def gpu_numa_node(device_index: int, sysfs: str = "/sys") -> int:
    """NUMA node of the GPU's PCI function, -1 when unknown."""
    addr = gpu_pci_address(device_index)
    if addr is None:
        return -1
    text = _read(f"{sysfs}/bus/pci/devices/{addr}/numa_node")
    try:
        return int(text) if text is not None else -1
    except ValueError:
        return -1


def node_cpus(node: int, sysfs: str = "/sys") -> Set[int]:
    text = _read(f"{sysfs}/devices/system/node/node{node}/cpulist")
    return parse_cpulist(text) if text else set()


def bind_to_gpu_node(device_index: int, sysfs: str = "/sys") -> Dict[str, object]:
    """Restrict this process to the CPUs of the GPU's NUMA node.  Returns what was found and done."""
    info: Dict[str, object] = {"node": -1, "bound": False, "cpus": 0}
    if os.environ.get("PSB_NUMA_BIND", "0") != "1" or not hasattr(os, "sched_setaffinity"):
        return info
    node = gpu_numa_node(device_index, sysfs)
    info["node"] = node
    if node < 0:
        return info
    try:
        allowed = os.sched_getaffinity(0)
        want = node_cpus(node, sysfs) & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            info["bound"] = True
        info["cpus"] = len(want)
    except OSError:
        pass
    return info
