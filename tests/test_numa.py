"""NUMA placement helper against a fake sysfs tree (no GPU needed)."""
import os

from parameter_server_b200.utils import numa


def _fake_sysfs(tmp_path, node, cpulist):
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text(f"{node}\n")
    nd = tmp_path / "devices" / "system" / "node" / f"node{max(node, 0)}"
    nd.mkdir(parents=True)
    (nd / "cpulist").write_text(cpulist + "\n")
    return str(tmp_path)


def test_parse_cpulist():
    assert numa.parse_cpulist("0-3,8,10-11") == {0, 1, 2, 3, 8, 10, 11}
    assert numa.parse_cpulist("") == set()


def test_bind_uses_the_gpu_node(tmp_path, monkeypatch):
    allowed = sorted(os.sched_getaffinity(0))
    keep = allowed[: max(1, len(allowed) // 2)]
    sysfs = _fake_sysfs(tmp_path, 1, ",".join(map(str, keep)))
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: "0000:1b:00.0")
    assert numa.gpu_numa_node(0, sysfs) == 1
    assert numa.node_cpus(1, sysfs) == set(keep)
    monkeypatch.setenv("PSB_NUMA_BIND", "0")
    assert numa.bind_to_gpu_node(0, sysfs)["bound"] is False and os.sched_getaffinity(0) == set(allowed)
    monkeypatch.setenv("PSB_NUMA_BIND", "1")
    try:
        info = numa.bind_to_gpu_node(0, sysfs)
        assert info["node"] == 1 and info["cpus"] == len(keep)
        assert os.sched_getaffinity(0) == set(keep)
        assert info["bound"] == (set(keep) != set(allowed))
    finally:
        os.sched_setaffinity(0, allowed)


def test_parse_driver_topology_report():
    text = ("\t\x1b[4mGPU0\tGPU1\tNIC0\tCPU Affinity\tNUMA Affinity\tGPU NUMA ID\x1b[0m\n"
            "GPU0\t X \tNV18\tNODE\t0-3,8-11\t0\t\tN/A\n"
            "GPU1\tNV18\t X \tSYS\t4-7\t1\t\tN/A\n"
            "NIC0\tNODE\tSYS\t X \t\t\t\t\n\nLegend:\n  X    = Self\n")
    aff = numa.parse_topo_cpu_affinity(text)
    assert aff == {0: {0, 1, 2, 3, 8, 9, 10, 11}, 1: {4, 5, 6, 7}}
    assert numa.parse_topo_cpu_affinity("no matrix here") == {}


def test_bind_falls_back_to_the_driver_report(tmp_path, monkeypatch):
    allowed = sorted(os.sched_getaffinity(0))
    keep = set(allowed[: max(1, len(allowed) // 2)])
    sysfs = _fake_sysfs(tmp_path, -1, "0")
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: "0000:1b:00.0")
    monkeypatch.setattr(numa, "gpu_cpus_from_driver", lambda i: keep)
    monkeypatch.setenv("PSB_NUMA_BIND", "1")
    try:
        info = numa.bind_to_gpu_node(0, sysfs)
        assert info["source"] == "driver" and info["cpus"] == len(keep) and os.sched_getaffinity(0) == keep
    finally:
        os.sched_setaffinity(0, allowed)


def test_unknown_node_changes_nothing(tmp_path, monkeypatch):
    before = os.sched_getaffinity(0)
    sysfs = _fake_sysfs(tmp_path, -1, "0")
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: "0000:1b:00.0")
    monkeypatch.setenv("PSB_NUMA_BIND", "1")
    info = numa.bind_to_gpu_node(0, sysfs)
    assert info["node"] == -1 and not info["bound"] and os.sched_getaffinity(0) == before
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: None)
    assert numa.gpu_numa_node(0, sysfs) == -1
