import json

import numpy as np

from parameter_server_b200.data import tools
from parameter_server_b200.utils.trace import ChromeTrace, MetricsLog, nvtx_range


def test_text2bin_show_bin2text_roundtrip(tmp_path):
    src = tmp_path / "part-0"
    src.write_text("+1 1:0.5 7:2\n-1 2:1\n+1 3:1 4:1 9:0.25\n")
    st = tools.text2bin("LIBSVM", str(tmp_path / "part-.*"), str(tmp_path / "m"), str(tmp_path / "cache") + "/")
    assert st == {"rows": 3, "cols": 10, "nnz": 6, "files": 1}
    assert tools.show(str(tmp_path / "m"))["nnz"] == 6
    assert tools.bin2text(str(tmp_path / "m"), str(tmp_path / "back.txt")) == 3
    assert (tmp_path / "back.txt").read_text() == src.read_text()
    assert "'num_ex': 3" in tools.info("LIBSVM", str(tmp_path / "part-.*"))


def test_chrome_trace_and_metrics(tmp_path):
    tr = ChromeTrace(str(tmp_path / "t.json"), pid=3)
    with tr.span("pass", cat="solver", block=7):
        with nvtx_range("inner"):
            tr.instant("mark", k=1)
    path = tr.save()
    ev = json.load(open(path))["traceEvents"]
    assert {e["name"] for e in ev} == {"pass", "mark"} and ev[-1]["args"]["block"] == 7 and ev[-1]["dur"] >= 0
    assert ChromeTrace(None).save() is None
    ml = MetricsLog(str(tmp_path / "m.jsonl"))
    ml.log(examples_per_s=1.5e8, step=3)
    rec = json.loads(open(tmp_path / "m.jsonl").read().strip())
    assert rec["step"] == 3 and "time" in rec
