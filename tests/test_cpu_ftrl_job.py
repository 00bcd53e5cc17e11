"""Online FTRL as CPU nodes over the message protocol (scheduler + servers + workers).

With one worker the schedule is deterministic: the per-server model dumps must equal the fp64 oracle
run over the same minibatches (with and without the tail-feature filter).  With two workers the run is
eventually consistent; it must still learn."""
import numpy as np
import pytest

from baseline.cpu_ref.ftrl_ref import FTRLRef
from parameter_server_b200 import config as cfg
from parameter_server_b200.apps.job import run_local_threads
from parameter_server_b200.data.synthetic import write_libsvm_parts
from parameter_server_b200.utils.modelio import read_model_text
from parameter_server_b200.utils.range import Range
from tests.test_cpu_job import planted

CONF = '''
app_name: "ctr"
parameter_name: "ctr_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{train}/part-.*" }}
  model_output {{ format: TEXT file: "{out}/model" }}
  loss {{ type: LOGIT }}
  penalty {{ type: L1 lambda: 0.05 lambda: 0.1 }}
  learning_rate {{ type: CONSTANT alpha: 0.05 beta: 1 }}
  solver {{ minibatch_size: {mb} tail_feature_freq: {tail} countmin_n: 8192 countmin_k: 2 eval_interval: 0 }}
  ftrl {{ }}
}}
'''


def _minibatches(off, idx, y, mb):
    """The oracle's view of what a worker streams: consecutive row blocks of one file."""
    off, idx, y = off.numpy(), idx.numpy().astype(np.uint64), y.numpy().astype(np.float64)
    for r0 in range(0, len(y), mb):
        r1 = min(r0 + mb, len(y))
        o = off[r0:r1 + 1]
        yield (o - o[0]).astype(np.int64), idx[o[0]:o[-1]], y[r0:r1]


@pytest.mark.parametrize("tail", [0, 2])
def test_one_worker_equals_the_oracle(tmp_path, tail):
    rows, cols, mb = 900, 512, 200
    off, idx, vals, y = planted(rows, cols, 10, 1, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 1)
    flags = cfg.Flags(num_workers=1, num_servers=2, seed=0)
    prog = run_local_threads(flags, CONF.format(train=tmp_path / "train", out=tmp_path, mb=mb, tail=tail))
    assert prog[0]["examples"] == rows
    ref = FTRLRef(0.05, 1.0, 0.05, 0.1, "count", tail_freq=tail, countmin_n=8192, countmin_k=2,
                  seps=Range.all().separators(2))
    loss = sum(ref.step([b]) for b in _minibatches(off, idx, y, mb))
    rk, rw = ref.nonzero()
    model = {}
    for s in ("S0", "S1"):
        model.update(read_model_text(str(tmp_path / f"model_{s}")))
    assert len(rk) > 20 and sorted(model) == rk.tolist()
    np.testing.assert_allclose([model[int(k)] for k in rk], rw, rtol=2e-5, atol=1e-9)   # text dump: 6 digits
    # every server reports lambda1·|w|_1 + lambda2/2·sqrt(|w|_2^2) of its own shard (FTRLModel::objv); the scheduler adds them up
    half = Range.all().separators(2)[1]
    pen = sum(0.05 * np.abs(rw[m]).sum() + 0.05 * np.sqrt((rw[m] ** 2).sum()) for m in (rk < np.uint64(half), rk >= np.uint64(half)))
    assert prog[0]["objv"] == pytest.approx(loss + pen, rel=1e-9)
    if tail:      # the filter held keys back: their first (sub-threshold) occurrences never reached the model
        seen = sum(e.pos + e.neg for e in ref.model.values())
        assert seen < idx.numel()


def test_two_workers_learn(tmp_path):
    rows, cols = 2000, 256
    off, idx, vals, y = planted(rows, cols, 10, 2, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    flags = cfg.Flags(num_workers=2, num_servers=2, seed=0)
    prog = run_local_threads(flags, CONF.format(train=tmp_path / "train", out=tmp_path, mb=100, tail=0))
    assert prog[0]["examples"] == rows and prog[0]["nnz_w"] > 10
    # eval_interval 0: every minibatch is reported to the scheduler (2 workers x 10 minibatches of 100 rows)
    reps = prog[0]["reports"]
    assert len(reps) == 20 and {r["worker"] for r in reps} == {"W0", "W1"} and reps[-1]["examples"] == rows
    # mean logistic loss over the stream must beat the constant predictor (log 2)
    model = {}
    for s in ("S0", "S1"):
        model.update(read_model_text(str(tmp_path / f"model_{s}")))
    keys, yy, oo = idx.numpy().astype(np.uint64), y.numpy(), off.numpy()
    row_of = np.repeat(np.arange(rows), np.diff(oo))
    xw = np.bincount(row_of, weights=np.array([model.get(int(k), 0.0) for k in keys]), minlength=rows)
    assert np.mean(np.logaddexp(0.0, -yy * xw)) < 0.66      # log 2 = 0.693 for the constant predictor


def test_progress_lines_merge_worker_and_server_reports(tmp_path):
    """eval_interval > 0: workers report loss and examples, servers their penalty and non-zeros, every interval; the
    scheduler shows one merged line per interval in the reference's format."""
    import re

    rows, cols = 60000, 4096
    off, idx, vals, y = planted(rows, cols, 8, 5, False)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    text = CONF.format(train=tmp_path / "train", out=tmp_path, mb=50, tail=0).replace("eval_interval: 0", "eval_interval: 0.05")
    prog = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), text)
    assert prog[0]["examples"] == rows
    lines = prog[0]["lines"]
    if not lines:
        pytest.skip("the job ended within one interval on this machine")
    pat = re.compile(r"^\s*(\d+) examples, loss (\S+), penalty (\S+), \|w\|_0\s+(\d+)$")
    got = [pat.match(l) for l in lines]
    assert all(got)
    seen = [int(m.group(1)) for m in got]
    assert seen == sorted(seen) and 0 < seen[-1] <= rows
    assert any(float(m.group(3)) > 0 and int(m.group(4)) > 0 for m in got) or len(lines) < 2    # the servers' reports arrived
    assert 0.0 < float(got[-1].group(2)) < 1.5


def test_processes_over_tcp(tmp_path):
    """The same job as five real processes (1 + 2 + 2) over the TCP van, started by the launcher."""
    import os
    import subprocess
    import sys

    rows, cols = 1200, 256
    off, idx, vals, y = planted(rows, cols, 10, 4, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    conf = tmp_path / "job.conf"
    conf.write_text(CONF.format(train=tmp_path / "train", out=tmp_path, mb=150, tail=2))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "2", "-num_workers", "2",
                        "-app", str(conf)], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"{rows} examples" in r.stderr + r.stdout
    model = {}
    for s_ in ("S0", "S1"):
        model.update(read_model_text(str(tmp_path / f"model_{s_}")))
    assert len(model) > 20


def test_launcher_stops_the_job_when_a_node_fails(tmp_path):
    """A scheduler that cannot read its job file exits; the launcher ends the other nodes instead of waiting forever."""
    import os
    import subprocess
    import sys
    import time

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    t0 = time.time()
    r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "1", "-num_workers", "1",
                        "-app", str(tmp_path / "missing.conf")], cwd=root, capture_output=True, text=True, timeout=120)
    assert r.returncode != 0 and time.time() - t0 < 60
