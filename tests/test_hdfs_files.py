"""Data on HDFS: ``hdfs { home ... }`` in a DataConfig makes the host runtime list directories with ``hadoop fs -ls``
and read files through ``hadoop fs -cat`` pipes (plain and gzip).  A stand-in ``hadoop`` script serves a local folder."""
import gzip
import os
import stat

import numpy as np
import pytest
import torch

from parameter_server_b200 import config as cfg
from parameter_server_b200.apps.job import run_local_threads
from parameter_server_b200.data.synthetic import write_libsvm_parts
from parameter_server_b200.runtime import host
from parameter_server_b200.utils.pbtext import parse

FAKE = r'''#!/bin/sh
# stand-in for `hadoop fs`: serves paths below $FAKE_HDFS_ROOT and logs every call
[ "$1" = "fs" ] || exit 2
shift
while [ "$1" = "-D" ]; do shift; shift; done
echo "$HADOOP_USER_NAME $*" >> "$FAKE_HDFS_ROOT/calls.log"
case "$1" in
  -ls)
    echo "Found 99 items"
    for f in "$FAKE_HDFS_ROOT$2"/*; do
      if [ -d "$f" ]; then echo "drwxr-xr-x   - user group          0 2014-01-01 00:00 ${f#$FAKE_HDFS_ROOT}"
      else echo "-rw-r--r--   3 user group       1234 2014-01-01 00:00 ${f#$FAKE_HDFS_ROOT}"; fi
    done ;;
  -cat) cat "$FAKE_HDFS_ROOT$2" ;;
  -test) [ -e "$FAKE_HDFS_ROOT$3" ] ;;
  *) exit 2 ;;
esac
'''


@pytest.fixture
def fake_hdfs(tmp_path, monkeypatch):
    home = tmp_path / "hadoop_home"
    (home / "bin").mkdir(parents=True)
    exe = home / "bin" / "hadoop"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IXUSR)
    root = tmp_path / "hdfs_root"
    (root / "data" / "train" / "subdir").mkdir(parents=True)
    monkeypatch.setenv("FAKE_HDFS_ROOT", str(root))
    old = host().hadoop_fs()
    yield home, root
    host().set_hadoop_fs(old)


def _planted(rows=600, cols=512, nnz=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    keys = torch.randint(1, cols, (rows, nnz), generator=g).sort(1).values
    keep = torch.ones_like(keys, dtype=torch.bool)
    keep[:, 1:] = keys[:, 1:] != keys[:, :-1]
    off = torch.zeros(rows + 1, dtype=torch.int64)
    off[1:] = keep.sum(1).cumsum(0)
    idx = keys[keep]
    y = torch.where(torch.rand(rows, generator=g) < 0.5, -1.0, 1.0)
    return off, idx, torch.ones(idx.numel()), y


def test_listing_and_reading_through_the_pipe(fake_hdfs):
    home, root = fake_hdfs
    H = host()
    off, idx, vals, y = _planted()
    write_libsvm_parts(str(root / "data" / "train"), off, idx, vals, y, 3)
    names = sorted(n for n in os.listdir(root / "data" / "train") if n.startswith("part-"))
    assert len(names) == 3
    # one of the parts is gzip on the remote side
    raw = (root / "data" / "train" / names[2]).read_bytes()
    (root / "data" / "train" / names[2]).unlink()
    with gzip.open(root / "data" / "train" / (names[2] + ".gz"), "wb") as f:
        f.write(raw)
    dc = parse('format: TEXT text: LIBSVM file: "/data/train/part-.*" hdfs { home: "%s" ugi: "alice,secret" namenode: "hdfs://nn:9000" }' % home,
               cfg.DataConfig)
    pats = cfg.data_files(dc, H)
    assert pats == ["hdfs:/data/train/part-.*"]
    assert H.hadoop_fs() == f"HADOOP_USER_NAME=alice {home}/bin/hadoop fs -D fs.defaultFS=hdfs://nn:9000"
    files = H.search_files(pats)
    assert files == [f"hdfs:/data/train/{n}" for n in (names[0], names[1], names[2] + ".gz")]     # the sub-directory is not a file
    r = H.SlotReader()
    r.init(files, H.TextFormat.LIBSVM, str(root / "cache") + "/", True, False, False, 0, 2048)
    info, hits = r.read(3)
    assert hits == 0 and info["num_ex"] == 600
    np.testing.assert_array_equal(r.index(1), idx.numpy().astype(np.uint64))
    np.testing.assert_array_equal(r.value(0), y.numpy())
    log = (root / "calls.log").read_text().splitlines()
    assert sum(1 for l in log if " -cat " in l) == 3 and all(l.startswith("alice ") for l in log)
    # the streaming reader takes the same paths
    sr = H.StreamReader()
    sr.init(files, H.TextFormat.LIBSVM, False, False)
    n = 0
    while True:
        mb = sr.read(250)
        if mb is None:
            break
        n += mb[1]["num_ex"]
    assert n == 600


def test_cpu_job_with_training_data_on_hdfs(fake_hdfs, tmp_path):
    home, root = fake_hdfs
    off, idx, vals, y = _planted(seed=1)
    write_libsvm_parts(str(root / "data" / "train"), off, idx, vals, y, 2)
    local = tmp_path / "local_data"
    write_libsvm_parts(str(local), off, idx, vals, y, 2)
    conf = '''
app_name: "h" parameter_name: "h_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{train}/part-.*" {hdfs} }}
  local_cache {{ format: BIN file: "{cache}/" }}
  model_output {{ format: TEXT file: "{out}/model" }}
  loss {{ type: LOGIT }} penalty {{ type: L1 lambda: 0.5 }} learning_rate {{ type: CONSTANT eta: 1 }}
  solver {{ feature_block_ratio: 1 max_pass_of_data: 3 max_block_delay: 0 epsilon: 1e-6 random_feature_block_order: true
           tail_feature_freq: 0 }}
  darling {{ delta_init_value: 1 delta_max_value: 5 kkt_filter_threshold_ratio: 10 }}
}}'''
    progs = []
    for name, train, hd in (("remote", "/data/train", 'hdfs { home: "%s" }' % home), ("local", str(local), "")):
        out = tmp_path / name
        out.mkdir()
        text = conf.format(train=train, hdfs=hd, cache=tmp_path / ("cache_" + name), out=out)
        progs.append(run_local_threads(cfg.Flags(num_workers=2, num_servers=1, seed=0), text))
    assert [p["objv"] for p in progs[0]] == [p["objv"] for p in progs[1]]
    assert (tmp_path / "remote" / "model_S0").read_text() == (tmp_path / "local" / "model_S0").read_text()
