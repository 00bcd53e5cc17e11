"""-log_to_file / -log_instant of the node command line: every node of a launched job writes its own log file."""
import glob
import os
import subprocess
import sys

from parameter_server_b200.data.synthetic import write_libsvm_parts
from parameter_server_b200.ps import node_name
from test_cpu_job import CONF, planted


def test_node_names():
    assert [node_name(r, 2, 3) for r in range(8)] == ["H", "W0", "W1", "S0", "S1", "S2", "U0", "U1"]


def test_every_node_logs_to_its_own_file(tmp_path):
    off, idx, vals, y = planted(600, 512, 8, 2, False)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 1)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=0.5, passes=2, tail=0))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "1", "-num_workers", "1",
                        "-app", str(conf), "-log_to_file", "-log_instant", "-verbose"], cwd=tmp_path, env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    logs = {n: glob.glob(str(tmp_path / f"log_{n}_*")) for n in ("H", "W0", "S0")}
    assert all(len(v) == 1 for v in logs.values()), logs
    table = open(logs["H"][0]).read()
    assert "objective" in table and "|w|_0" in table          # the scheduler's progress table went to its file
    assert "objective" not in r.stderr                          # and not to the terminal
    assert (tmp_path / "model_S0").exists()
    narration = open(logs["W0"][0]).read()                     # -verbose: the worker's executors tell what they process
    assert "[plumb@W0] request t=" in narration and "[plumb_w@W0] reply t=" in narration
