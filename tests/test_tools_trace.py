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


def test_split_into_train_and_test_parts(tmp_path):
    """The dataset script's layout: 1000-line parts, the first 13 for training, the rest for testing (here: 10 / 3)."""
    import bz2

    from parameter_server_b200.data import tools

    lines = [f"{'+1' if i % 3 else '-1'} {i % 50 + 1}:1 {i % 7 + 60}:0.5\n" for i in range(47)]
    src = tmp_path / "toy.binary.bz2"
    with bz2.open(src, "wt") as f:
        f.writelines(lines)
    (tmp_path / "out" / "train").mkdir(parents=True)
    (tmp_path / "out" / "train" / "part-999").write_text("stale\n")          # an earlier split is cleared, like rm -f
    assert tools.main(["split", str(src), str(tmp_path / "out"), "10", "3"]) == 0
    tr = sorted(p.name for p in (tmp_path / "out" / "train").iterdir())
    te = sorted(p.name for p in (tmp_path / "out" / "test").iterdir())
    assert tr == ["part-000", "part-001", "part-002"] and te == ["part-003", "part-004"]
    back = "".join((tmp_path / "out" / d / n).read_text() for d, names in (("train", tr), ("test", te)) for n in names)
    assert back == "".join(lines)
    assert len((tmp_path / "out" / "test" / "part-004").read_text().splitlines()) == 7


def test_rcv1_fetch_unpack_split(tmp_path, monkeypatch):
    """The data set script end to end, with a file:// URL in place of the download; then the failure without a network."""
    import bz2

    import pytest

    lines = [f"{'1' if i % 2 else '-1'} {i % 9 + 1}:0.5\n" for i in range(35)]
    served = tmp_path / "served.bz2"
    with bz2.open(served, "wt") as f:
        f.writelines(lines)
    work = tmp_path / "work"
    work.mkdir()
    monkeypatch.chdir(work)
    got = tools.rcv1("rcv1", served.as_uri(), lines_per_part=10, train_parts=2)
    assert got == {"train": 2, "test": 2, "lines": 35}
    assert (work / "rcv1_train.binary").read_text() == "".join(lines)
    assert sorted(p.name for p in (work / "rcv1" / "test").iterdir()) == ["part-002", "part-003"]
    # a second run finds the unpacked file and does not fetch
    assert tools.rcv1("again", "file:///nonexistent", lines_per_part=10, train_parts=2)["lines"] == 35
    other = tmp_path / "offline"
    other.mkdir()
    monkeypatch.chdir(other)
    with pytest.raises(OSError, match="by hand"):
        tools.rcv1("rcv1", "file:///nonexistent/rcv1_train.binary.bz2")
    assert list(other.iterdir()) == []
