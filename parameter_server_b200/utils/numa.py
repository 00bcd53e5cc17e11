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


def parse_topo_cpu_affinity(text: str) -> Dict[int, Set[int]]:
    """CPU affinity per GPU from the matrix that ``nvidia-smi topo -m`` prints (tab-separated cells, one
    header line that names a ``CPU Affinity`` column, one row per ``GPU<i>``)."""
    import re

    out: Dict[int, Set[int]] = {}
    col = None
    for line in re.sub(r"\x1b\[[0-9;]*m", "", text).splitlines():
        cells = [c.strip() for c in line.split("\t")]
        if col is None:
            if "CPU Affinity" in cells:
                col = cells.index("CPU Affinity")
            continue
        name = cells[0] if cells else ""
        if name.startswith("GPU") and name[3:].isdigit() and col < len(cells):
            try:
                out[int(name[3:])] = parse_cpulist(cells[col])
            except ValueError:
                pass
    return out


def gpu_cpus_from_driver(device_index: int) -> Set[int]:
    """Fallback when sysfs hides the NUMA node (containers): ask the driver's topology report (read only)."""
    import subprocess

    try:
        r = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20)
    except (OSError, subprocess.SubprocessError):
        return set()
    if r.returncode != 0:
        return set()
    # torch's device order follows CUDA_VISIBLE_DEVICES; the report lists physical indices
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    phys = device_index
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if ids and device_index < len(ids) and ids[device_index].isdigit():
        phys = int(ids[device_index])
    return parse_topo_cpu_affinity(r.stdout).get(phys, set())


def bind_to_gpu_node(device_index: int, sysfs: str = "/sys") -> Dict[str, object]:
    """Restrict this process to the CPUs next to the GPU.  Returns what was found and done."""
    info: Dict[str, object] = {"node": -1, "bound": False, "cpus": 0, "source": None}
    if os.environ.get("PSB_NUMA_BIND", "0") != "1" or not hasattr(os, "sched_setaffinity"):
        return info
    node = gpu_numa_node(device_index, sysfs)
    info["node"] = node
    cpus: Set[int] = set()
    if node >= 0:
        cpus, info["source"] = node_cpus(node, sysfs), "sysfs"
    if not cpus:
        cpus = gpu_cpus_from_driver(device_index)
        info["source"] = "driver" if cpus else None
    if not cpus:
        return info
    try:
        allowed = os.sched_getaffinity(0)
        want = cpus & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            info["bound"] = True
        info["cpus"] = len(want)
    except OSError:
        pass
    return info
