"""The plumbing configuration: 1 scheduler + 2 servers + 2 workers as CPU nodes running DARLIN through
the message protocol (LOAD -> PREPROCESS -> UPDATE per block -> EVALUATE -> SAVE); objective per pass and
the per-server model dumps must equal the single-process fp64 oracle."""
import os

import numpy as np
import pytest
import torch

from baseline.cpu_ref.darlin_ref import DarlinConfig as RefConfig
from baseline.cpu_ref.darlin_ref import DarlinRef
from parameter_server_b200 import config as cfg
from parameter_server_b200.apps.job import run_local_threads
from parameter_server_b200.data.synthetic import write_libsvm_parts
from parameter_server_b200.utils.modelio import read_model_text

CONF = '''
app_name: "plumb"
parameter_name: "plumb_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{train}/part-.*" }}
  local_cache {{ format: BIN file: "{cache}/" }}
  model_output {{ format: TEXT file: "{out}/model" }}
  loss {{ type: LOGIT }}
  penalty {{ type: L1 lambda: {lam} }}
  learning_rate {{ type: CONSTANT eta: 1 }}
  solver {{ feature_block_ratio: {ratio} max_pass_of_data: {passes} max_block_delay: 0 epsilon: 1e-6
           tail_feature_freq: {tail} random_feature_block_order: true }}
  darling {{ delta_init_value: 1 delta_max_value: 5 kkt_filter_threshold_ratio: 10 }}
}}
'''


def planted(rows, cols, nnz, seed, spread):
    g = torch.Generator().manual_seed(seed)
    keys = torch.randint(0, cols, (rows, nnz), generator=g).sort(1).values
    keep = torch.ones_like(keys, dtype=torch.bool)
    keep[:, 1:] = keys[:, 1:] != keys[:, :-1]
    counts = keep.sum(1)
    off = torch.zeros(rows + 1, dtype=torch.int64)
    off[1:] = counts.cumsum(0)
    idx = keys[keep]
    w = torch.randn(cols, generator=g) * (torch.rand(cols, generator=g) < 0.05)
    row_of = torch.repeat_interleave(torch.arange(rows), counts)
    xw = torch.zeros(rows).index_add_(0, row_of, w[idx])
    y = torch.sign(xw + 0.1 * torch.randn(rows, generator=g))
    y[y == 0] = 1
    if spread:                                   # keys over the whole uint64 space: both servers own some
        idx = idx * ((1 << 63) // cols * 2 - 12345)
    return off, idx, torch.ones(idx.numel()), y


@pytest.mark.parametrize("spread", [False, True])
def test_darlin_over_the_protocol_matches_oracle(tmp_path, spread):
    rows, cols, nnz, passes, lam, ratio = 1200, 2048, 12, 4, 0.5, 0.5
    off, idx, vals, y = planted(rows, cols, nnz, 0, spread)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=lam, ratio=ratio,
                       passes=passes, tail=0)
    flags = cfg.Flags(num_workers=2, num_servers=2, seed=0)
    prog = run_local_threads(flags, text)
    k = idx.numpy().view(np.uint64) if spread else idx.numpy().astype(np.uint64)
    o = off.numpy()
    h = rows // 2
    shards = [(o[:h + 1], k[:o[h]], vals.numpy()[:o[h]], y.numpy()[:h]),
              (o[h:] - o[h], k[o[h]:], vals.numpy()[o[h]:], y.numpy()[h:])]
    ref = DarlinRef(shards, None, RefConfig(lambda1=lam, max_pass=passes, feature_block_ratio=ratio, epsilon=1e-6,
                                            delta_init=1, delta_max=5, kkt_ratio=10, seed=0))
    rprog = ref.run()
    assert len(prog) == len(rprog) == passes
    for p, r in zip(prog, rprog):
        assert p["objv"] == pytest.approx(r.objv, rel=1e-9)
        assert p["nnz_w"] == r.nnz_w and p["nnz_active_set"] == r.nnz_active
        assert p["violation"] == pytest.approx(r.violation, rel=1e-9)
    m0, m1 = (read_model_text(str(tmp_path / f"model_S{i}")) if os.path.exists(tmp_path / f"model_S{i}") else {} for i in (0, 1))
    rk, rw = ref.model()
    merged = {**m0, **m1}
    assert sorted(merged) == rk.tolist()
    for kk, ww in zip(rk.tolist(), rw.tolist()):
        assert merged[kk] == pytest.approx(ww, rel=1e-5)
    if spread:
        assert len(m0) > 0 and len(m1) > 0 and max(m0) < min(m1)      # key-range sharded dumps
    else:
        assert len(m1) == 0                                            # small ids all fall into S0's range


def test_tail_feature_filter_drops_rare_keys(tmp_path):
    off, idx, vals, y = planted(600, 4096, 10, 3, False)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.2, ratio=0.5, passes=2, tail=2)
    prog = run_local_threads(cfg.Flags(num_workers=2, num_servers=2), text)
    cnt = np.bincount(idx.numpy(), minlength=4096)
    model = read_model_text(str(tmp_path / "model_S0"))
    rare_total = int(((cnt > 0) & (cnt <= 2)).sum())
    rare_kept = sum(1 for k in model if cnt[k] <= 2)
    # the sketch never drops a frequent key and lets only a few rare ones through (hash collisions)
    assert len(model) > 0 and rare_total > 100 and rare_kept < 0.2 * rare_total
    assert prog[-1]["objv"] < prog[0]["objv"] * 1.001


def test_features_on_disk_give_the_same_job(tmp_path, capfd):
    """-mmap_training_data: workers keep their column blocks in files of the local cache directory and read them
    back through prefetch threads under a small memory limit; nothing about the result may change."""
    rows, cols, nnz, passes, lam, ratio = 1200, 2048, 12, 3, 0.5, 2.0
    off, idx, vals, y = planted(rows, cols, nnz, 5, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    progs, models = [], []
    for mode, tau in (("mem", 0), ("disk", 0), ("disk", 2)):
        out = tmp_path / f"{mode}{tau}"
        out.mkdir()
        text = CONF.format(train=tmp_path / "train", cache=tmp_path / f"cache_{mode}{tau}", out=out, lam=lam, ratio=ratio,
                           passes=passes, tail=0).replace("max_block_delay: 0", f"max_block_delay: {tau}")
        flags = cfg.Flags(num_workers=2, num_servers=2, seed=0, mmap_training_data=(mode == "disk"), prefetch_mem_limit_kb=16,
                          num_threads=2, verbose=(mode == "disk"))
        progs.append(run_local_threads(flags, text))
        models.append({**{k: v for i in (0, 1) if os.path.exists(out / f"model_S{i}") for k, v in read_model_text(str(out / f"model_S{i}")).items()}})
        if mode == "disk":
            left = [p for p in os.listdir(tmp_path / f"cache_{mode}{tau}") if "_features_" in p]
            assert left == [], left                                    # the workers removed their feature files
    text = capfd.readouterr().out
    assert "feature station" in text and "'prefetched': 0" not in text     # read-ahead happened on every worker
    for p, q in zip(progs[0], progs[1]):                                # same schedule, same arithmetic
        assert p["objv"] == q["objv"] and p["nnz_w"] == q["nnz_w"]
    assert models[0] == models[1] and len(models[0]) > 0
    assert progs[2][-1]["objv"] < progs[2][0]["objv"]                    # bounded delay: runs and converges


def test_warm_start_from_a_model_dump(tmp_path):
    """init_w { type: FILE }: a second job starts from the dump of the first and carries on from its objective."""
    off, idx, vals, y = planted(1200, 2048, 12, 7, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    first = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path / "a", lam=0.5, ratio=0.5, passes=4, tail=0)
    p1 = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), first)
    second = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path / "b", lam=0.5, ratio=0.5, passes=1, tail=0)
    second = second.replace("loss {", 'init_w { type: FILE file_name: "%s/model" }\n  loss {' % (tmp_path / "a"))
    # other key ranges than the first job: three servers read the two parts
    p2 = run_local_threads(cfg.Flags(num_workers=2, num_servers=3, seed=1), second)
    assert p2[0]["objv"] < p1[-1]["objv"] * (1 + 1e-4)           # the dump keeps six digits
    assert p2[0]["objv"] < p1[1]["objv"]                          # far below where a cold start is after two passes
    cold = run_local_threads(cfg.Flags(num_workers=2, num_servers=3, seed=1), second.replace("type: FILE", "type: ZERO"))
    assert cold[0]["objv"] > p2[0]["objv"] * 1.01


def test_validation_auc_after_training(tmp_path):
    """validation_data in the job file: after the last pass the workers score their validation files with the servers'
    weights and the scheduler merges the AUC histograms."""
    from parameter_server_b200.runtime import host

    off, idx, vals, y = planted(1600, 1024, 12, 11, False)
    h = 1200
    o = off.numpy()
    write_libsvm_parts(str(tmp_path / "train"), off[:h + 1], idx[:o[h]], vals[:o[h]], y[:h], 2)
    write_libsvm_parts(str(tmp_path / "valid"), off[h:] - off[h], idx[o[h]:], vals[o[h]:], y[h:], 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.2, ratio=0.5, passes=4, tail=0)
    text = text.replace("local_cache {", 'validation_data { format: TEXT text: LIBSVM file: "%s/part-.*" }\n  local_cache {' % (tmp_path / "valid"))
    prog = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), text)
    last = prog[-1]
    assert 0.6 < last["validation_auc"] <= 1.0 and 0.55 < last["validation_accuracy"] <= 1.0
    # the same numbers from the dumped model, computed exactly
    model = {}
    for i in (0, 1):
        p = tmp_path / f"model_S{i}"
        if p.exists():
            model.update(read_model_text(str(p)))
    w = np.zeros(1024)
    for k, v in model.items():
        w[k] = v
    rows = np.repeat(np.arange(1600 - h), np.diff(o[h:]))
    xw = np.bincount(rows, weights=w[idx.numpy()[o[h]:]], minlength=1600 - h)
    yv = y.numpy()[h:]
    exact = host().exact_auc(yv.astype(np.float32), xw.astype(np.float32))
    assert last["validation_auc"] == pytest.approx(exact, abs=2e-3)          # histogram bins and the dump's six digits
    assert last["validation_accuracy"] == pytest.approx(float(np.mean((xw >= 0) == (yv > 0))), abs=5e-3)


def test_heartbeats_and_dashboard(tmp_path, capfd):
    """-report_interval: nodes report their resource use, the scheduler prints the table while the job runs."""
    off, idx, vals, y = planted(2000, 2048, 12, 3, True)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=4.0, passes=6, tail=0)
    run_local_threads(cfg.Flags(num_workers=2, num_servers=1, seed=0, report_interval=0.1), text)
    err = capfd.readouterr().err
    head = [l for l in err.splitlines() if l.startswith("Node  Task")]
    assert head and "HostCPU%" in head[0] and "HostName" in head[0]
    rows = [l for l in err.splitlines() if l.startswith(("W0 ", "W1 ", "S0 "))]
    full = [l for l in rows if "no report yet" not in l]
    assert full, err[-2000:]
    cols = full[-1].split()
    assert len(cols) == 15 and "@" in cols[-1]                      # every column filled, host name last
    assert any(int(l.split()[5]) > 0 for l in full)                 # some compute time was reported as busy
    assert max(int(l.split()[1]) for l in full) > 10                # and the task each node was at


def test_model_evaluation_app_on_cpu_nodes(tmp_path):
    """A job file with validation_data + model_input and no solver runs the evaluation app: the scheduler scores the
    validation files with the dumped model; the result equals the validation step of the training job."""
    off, idx, vals, y = planted(1600, 1024, 12, 11, False)
    h = 1200
    o = off.numpy()
    write_libsvm_parts(str(tmp_path / "train"), off[:h + 1], idx[:o[h]], vals[:o[h]], y[:h], 2)
    write_libsvm_parts(str(tmp_path / "valid"), off[h:] - off[h], idx[o[h]:], vals[o[h]:], y[h:], 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.2, ratio=0.5, passes=4, tail=0)
    text = text.replace("local_cache {", 'validation_data { format: TEXT text: LIBSVM file: "%s/part-.*" }\n  local_cache {' % (tmp_path / "valid"))
    trained = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), text)[-1]
    ev = '''
app_name: "eval" parameter_name: "eval_w"
linear_method {
  validation_data { format: TEXT text: LIBSVM file: "%s/part-.*" }
  model_input { format: TEXT file: "%s/model_S.*" }
  model_output { format: TEXT file: "%s/scores" }
}''' % (tmp_path / "valid", tmp_path, tmp_path)
    res = run_local_threads(cfg.Flags(num_workers=1, num_servers=1), ev)[0]
    assert res["examples"] == 400 and res["model_nnz"] > 10
    assert res["auc"] == pytest.approx(trained["validation_auc"], abs=2e-3)         # the dump keeps six digits
    assert res["accuracy"] == pytest.approx(trained["validation_accuracy"], abs=5e-3)
    assert res["auc"] == pytest.approx(res["exact_auc"], abs=2e-3)
    L = np.fromfile(tmp_path / "scores_L", dtype=np.float32)
    P = np.fromfile(tmp_path / "scores_P", dtype=np.float32)
    np.testing.assert_array_equal(L, y.numpy()[h:])
    assert len(P) == 400 and float(np.mean((P >= 0) == (L > 0))) == pytest.approx(res["accuracy"], abs=1e-6)


def test_prior_feature_groups_go_first(tmp_path):
    """solver { prior_fea_group: g num_iter_for_prior_fea_group: n }: the blocks that hold group g's keys (top 10 bits
    of a key) are swept n extra times at the start of the first pass, before the regular order."""
    from parameter_server_b200.apps import linear_cpu

    rows, cols = 800, 600
    off, idx, vals, y = planted(rows, cols, 10, 13, False)
    grp = torch.where(idx % 3 == 0, 127, torch.where(idx % 3 == 1, 120, 5)).to(torch.int64)     # three feature groups
    keys = (grp << 54) | idx
    write_libsvm_parts(str(tmp_path / "train"), off, keys, vals, y, 2)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.5, ratio=1.0, passes=2, tail=0)
    text = text.replace("random_feature_block_order: true", "random_feature_block_order: true prior_fea_group: 127 num_iter_for_prior_fea_group: 3")
    seen = []
    orig = linear_cpu.BatchScheduler._submit

    def spy(self, payload, wait=True, wait_time=-1):
        call = linear_cpu.parse(payload.decode(), cfg.LMCall)
        if call.cmd == "UPDATE_MODEL":
            seen.append((call.key.begin, call.key.end))
        return orig(self, payload, wait, wait_time)

    linear_cpu.BatchScheduler._submit = spy
    try:
        prog = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), text)
    finally:
        linear_cpu.BatchScheduler._submit = orig
    glo, ghi = 127 << 54, 128 << 54
    nblk = len(set(seen))
    in_group = [r for r in set(seen) if max(r[0], glo) < min(r[1], ghi)]
    assert 0 < len(in_group) < nblk
    head = seen[:3 * len(in_group)]
    assert all(r in in_group for r in head) and len(seen) == 3 * len(in_group) + 2 * nblk
    assert all(head.count(r) == 3 for r in in_group)
    assert prog[-1]["objv"] < prog[0]["objv"]


def test_many_servers_own_ranges_in_numeric_order(tmp_path):
    """With more than ten servers S2 must come before S10: server i owns the i-th key range and its dump holds it."""
    off, idx, vals, y = planted(600, 1024, 10, 4, True)           # keys spread over the whole uint64 space
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 1)
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=0.1, ratio=0.5, passes=2, tail=0)
    run_local_threads(cfg.Flags(num_workers=1, num_servers=12, seed=0), text)
    prev = -1
    seen = 0
    for i in range(12):
        p = tmp_path / f"model_S{i}"
        if not p.exists():
            continue
        m = read_model_text(str(p))
        if not m:
            continue
        assert min(m) > prev, (i, min(m), prev)
        assert (i * (2**64 - 1)) // 12 <= min(m) and max(m) < ((i + 1) * (2**64 - 1)) // 12 + 1
        prev = max(m)
        seen += 1
    assert seen >= 10


def test_terafea_groups_are_cut_group_by_group(tmp_path):
    """TERAFEA data: every feature group (top 10 bits of a key) gets blocks of its own, by its own density over its own
    key range, and the important group's blocks are swept first — the schedule of the reference's CTR job — and the run
    equals the oracle's with the same groups."""
    rows, passes, lam, ratio = 900, 3, 0.3, 1.0
    g = torch.Generator().manual_seed(11)
    lines, shard_rows = [], []
    keys_per_row = []
    w_true = {}
    for r in range(rows):
        ks = set()
        ks.add((127 << 54) | int(torch.randint(0, 40, (1,), generator=g)))                     # one feature per example
        ks.update((120 << 54) | int(v) for v in torch.randint(0, 300, (3,), generator=g))
        ks.update((5 << 54) | int(v) for v in torch.randint(0, 500, (6,), generator=g))
        keys_per_row.append(sorted(ks))
    allk = sorted({k for ks in keys_per_row for k in ks})
    wv = torch.randn(len(allk), generator=g) * (torch.rand(len(allk), generator=g) < 0.1)
    w_true = dict(zip(allk, wv.tolist()))
    ys = []
    for r, ks in enumerate(keys_per_row):
        s = sum(w_true[k] for k in ks) + 0.1 * float(torch.randn(1, generator=g))
        ys.append(1 if s > 0 else -1)
        lines.append(f"{1 if ys[-1] > 0 else 0} {r} | " + " ".join(str(k) for k in ks))
    os.makedirs(tmp_path / "train")
    h = rows // 2
    for i, part in enumerate((lines[:h], lines[h:])):
        (tmp_path / "train" / f"part-{i:03d}").write_text("\n".join(part) + "\n")
    text = CONF.format(train=tmp_path / "train", cache=tmp_path / "cache", out=tmp_path, lam=lam, ratio=ratio, passes=passes, tail=0)
    text = text.replace("text: LIBSVM", "text: TERAFEA").replace(
        "random_feature_block_order: true", "random_feature_block_order: true prior_fea_group: 127 num_iter_for_prior_fea_group: 2")
    from parameter_server_b200.apps import linear_cpu

    seen = []
    orig = linear_cpu.BatchScheduler._submit

    def spy(self, payload, wait=True, wait_time=-1):
        call = linear_cpu.parse(payload.decode(), cfg.LMCall)
        if call.cmd == "UPDATE_MODEL":
            seen.append((int(call.fea_grp[0]), call.key.begin, call.key.end))
        return orig(self, payload, wait, wait_time)

    linear_cpu.BatchScheduler._submit = spy
    try:
        prog = run_local_threads(cfg.Flags(num_workers=2, num_servers=2, seed=0), text)
    finally:
        linear_cpu.BatchScheduler._submit = orig
    blocks = sorted(set(seen), key=lambda b: b[1])
    by_group = {gid: [b for b in blocks if b[0] == gid] for gid in (5, 120, 127)}
    # one feature per example: one block; the denser groups: ceil(non-zeros per example x ratio) blocks each
    assert len(by_group[127]) == 1 and len(by_group[120]) == 3 and len(by_group[5]) == 6 and len(blocks) == 10
    for gid, bs in by_group.items():
        assert all(b[1] >> 54 == gid and (b[2] - 1) >> 54 == gid for b in bs)              # a block never crosses groups
    assert seen[:2] == by_group[127] * 2 and len(seen) == 2 + passes * 10                   # the prior sweeps, then the passes

    def shard(lo, hi):
        off = np.concatenate([[0], np.cumsum([len(k) for k in keys_per_row[lo:hi]])]).astype(np.int64)
        cols = np.array([k for ks in keys_per_row[lo:hi] for k in ks], dtype=np.uint64)
        return off, cols, np.ones(len(cols)), np.array(ys[lo:hi], dtype=np.float64)

    ref = DarlinRef([shard(0, h), shard(h, rows)], None,
                    RefConfig(lambda1=lam, max_pass=passes, feature_block_ratio=ratio, epsilon=1e-6, delta_init=1, delta_max=5,
                              kkt_ratio=10, seed=0, feature_group_bits=10, prior_fea_group=(127,), num_iter_for_prior_fea_group=2))
    rprog = ref.run()
    assert len(prog) == len(rprog) == passes
    for p, r in zip(prog, rprog):
        assert p["objv"] == pytest.approx(r.objv, rel=1e-9) and p["nnz_w"] == r.nnz_w
