"""Process bootstrap of one node of a job: identity from the rank, van, post office, membership.

Identity rules of the reference (src/system/van.cc:243-281): rank 0 is the scheduler ``H``; ranks
1..W are workers ``W0..``; ranks W+1..W+S are servers ``S0..``; anything above is an unused
stand-by ``U*``.  The scheduler's address comes from ``-scheduler`` (a text-format ``Node``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

from . import host
from .. import config as cfg


def role_of_rank(rank: int, num_workers: int, num_servers: int):
    H = host()
    if rank == 0:
        return H.SCHEDULER, "H"
    if rank <= num_workers:
        return H.WORKER, f"W{rank - 1}"
    if rank <= num_workers + num_servers:
        return H.SERVER, f"S{rank - num_workers - 1}"
    return H.UNUSED, f"U{rank - num_workers - num_servers - 1}"


def _host_stats() -> dict:
    """Busy / total jiffies of the machine and its memory in use, from /proc (zeros where /proc is absent)."""
    out = dict(busy=0, total=0, used_gb=0, used_pct=0)
    try:
        with open("/proc/stat") as f:
            v = [int(x) for x in f.readline().split()[1:]]
        out["total"] = sum(v)
        out["busy"] = sum(v) - v[3] - (v[4] if len(v) > 4 else 0)          # all but idle and iowait
        mem = {}
        with open("/proc/meminfo") as f:
            for line in f:
                k, _, rest = line.partition(":")
                mem[k] = int(rest.split()[0])
        used = mem.get("MemTotal", 0) - mem.get("MemAvailable", mem.get("MemFree", 0))
        out["used_gb"] = used >> 20
        out["used_pct"] = int(100 * used / max(mem.get("MemTotal", 1), 1))
    except (OSError, ValueError, IndexError):
        pass
    return out


def heartbeat_report(node_id: str, state: dict) -> str:
    """Text-format ``HeartbeatReport`` of this process (src/system/heartbeat_info.cc:37-155): CPU share of the process
    and of the machine since the previous report, memory of both, time spent in compute sections (``busy_ms``, added
    by the application), network totals and rates.  ``state["where"]`` (a GPU rank: its device and the device memory
    in use) is appended to the host name, the table's last column."""
    import socket

    H = host()
    u = H.resource_usage()
    hs = _host_stats()
    now = time.time()
    dt = max(now - state.get("t", now - 1.0), 1e-3)
    d_proc = u["proc_jiffies"] - state.get("proc", u["proc_jiffies"])
    d_host = max(u["host_jiffies"] - state.get("host", u["host_jiffies"]), 1)
    d_busy = hs["busy"] - state.get("hbusy", hs["busy"])
    d_total = max(hs["total"] - state.get("htotal", hs["total"]), 1)
    r = cfg.HeartbeatReport(
        task_id=int(state.get("task", 0)), hostname=f"{node_id}@{socket.gethostname()}{state.get('where', '')}", seconds_since_epoch=int(now), total_time_milli=int(dt * 1000),
        busy_time_milli=int(state.get("busy_ms", 0)), net_in_mb=int(u["net_in"] >> 20), net_out_mb=int(u["net_out"] >> 20),
        process_cpu_usage=int(100 * d_proc / d_host * (state.get("ncpu", 1))), host_cpu_usage=int(100 * d_busy / d_total),
        process_rss_mb=int(u["rss_mb"]), process_virt_mb=int(u["virt_mb"]),
        host_in_use_gb=int(hs["used_gb"]), host_in_use_percentage=int(hs["used_pct"]),
        host_net_in_bw=int((u["net_in"] - state.get("in", u["net_in"])) / dt / 1e6),
        host_net_out_bw=int((u["net_out"] - state.get("out", u["net_out"])) / dt / 1e6))
    state.update(t=now, proc=u["proc_jiffies"], host=u["host_jiffies"], hbusy=hs["busy"], htotal=hs["total"],
                 **{"in": u["net_in"], "out": u["net_out"]})
    state["busy_ms"] = 0
    from ..utils.pbtext import dumps

    return dumps(r, oneline=True)


@dataclass
class NodeContext:
    po: object
    van: object
    node_id: str
    role: int
    num_workers: int
    num_servers: int
    hb_state: dict = None          # heartbeat bookkeeping; applications add their compute time to hb_state["busy_ms"]

    def add_busy(self, seconds: float) -> None:
        if self.hb_state is not None:
            self.hb_state["busy_ms"] = self.hb_state.get("busy_ms", 0) + 1000.0 * seconds

    @property
    def is_scheduler(self) -> bool:
        return self.role == host().SCHEDULER

    @property
    def is_worker(self) -> bool:
        return self.role == host().WORKER

    @property
    def is_server(self) -> bool:
        return self.role == host().SERVER

    def stop(self) -> None:
        self.po.stop()


def advertised_address(scheduler_host: str, interface: str = "") -> str:
    """The address other nodes use to reach this one.  A job whose scheduler is on the loopback runs on one machine
    and stays there; otherwise the address of ``-interface``, or of the first interface that is up and not the
    loopback (src/system/van.cc:262-275)."""
    H = host()
    if interface:
        ip = H.local_ip(interface)
        if not ip:
            raise ValueError(f"-interface {interface}: no such interface with an IPv4 address ({H.interfaces()})")
        return ip
    if scheduler_host in ("127.0.0.1", "localhost", ""):
        return "127.0.0.1"
    return H.local_ip("") or "127.0.0.1"


def start_node(rank: int, flags: cfg.Flags, hub=None, timeout_s: float = 60.0) -> NodeContext:
    """Create the van + post office of rank ``rank`` and join the job (blocks until the node table is known).

    ``hub`` selects the in-process van (all nodes are threads of this process); otherwise TCP.
    """
    H = host()
    W, S = flags.num_workers, flags.num_servers
    role, nid = role_of_rank(rank, W, S)
    sched = cfg.parse_node(flags.scheduler)
    sched_node = H.Node(H.SCHEDULER, sched.id or "H", sched.hostname or "127.0.0.1", sched.port)
    me = H.Node(role, nid, advertised_address(sched.hostname or "127.0.0.1", flags.interface), sched.port if role == H.SCHEDULER else 0)
    if hub is not None:
        van = H.InprocVan(hub, me)
    else:
        van = H.TcpVan(me)
        van.set_retries(max(flags.num_retries, 40))
        van.bind()
    van.set_compress(bool(flags.compress_message) and hub is None)
    if flags.print_van:
        van.set_log(f"van_{nid}")
    po = H.Postoffice(van, W, S, flags.num_replicas)
    po.set_key_cache(bool(flags.key_cache))
    po.set_scheduler(sched_node if role != H.SCHEDULER else van.my_node)
    po.start()
    ctx = NodeContext(po, van, nid, role, W, S, hb_state={})
    if role == H.SCHEDULER:
        if not po.wait_nodes_and_init(timeout_s):
            raise TimeoutError("scheduler: not every worker/server registered in time")
    else:
        po.register_with_scheduler()
        if not po.wait_nodes_ready(timeout_s):
            raise TimeoutError(f"{nid}: no node table from the scheduler")
        if flags.report_interval > 0:
            po.start_heartbeat(float(flags.report_interval), lambda: heartbeat_report(nid, ctx.hb_state))
    return ctx


def dashboard(po) -> str:
    """The scheduler's heartbeat table (src/system/postoffice.cc:292-374)."""
    from ..utils.pbtext import parse

    rows = ["Node  Task  MyCPU%  MyRSS  MyVir  Busy(ms)  Busy%  InMB  OutMB  HostCPU%  HostUseGB(%)  HostInBW  HostOutBW  age(s)  HostName"]

    def order(k):
        return (k[0], int(k[1:]) if k[1:].isdigit() else 0)

    hb = po.heartbeats()
    for nid in sorted(hb, key=order):
        age, text = hb[nid]
        try:
            if not text:                                   # registered, but no report has arrived yet
                raise ValueError("empty")
            r = parse(text.decode(), cfg.HeartbeatReport)
            busy_pct = int(100 * r.busy_time_milli / max(r.total_time_milli, 1))
            use = f"{r.host_in_use_gb}({r.host_in_use_percentage}%)"
            rows.append(f"{nid:<5} {r.task_id:>4}  {r.process_cpu_usage:>6}  {r.process_rss_mb:>5}  "
                        f"{r.process_virt_mb:>5}  {r.busy_time_milli:>8}  {busy_pct:>5}  {r.net_in_mb:>4}  {r.net_out_mb:>5}  "
                        f"{r.host_cpu_usage:>8}  {use:>12}  "
                        f"{r.host_net_in_bw:>8}  {r.host_net_out_bw:>9}  {age:6.2f}  {r.hostname}")
        except Exception:
            rows.append(f"{nid:<5} (no report yet)  {age:6.2f}")
    return "\n".join(rows)
