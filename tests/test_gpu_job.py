"""Job files end to end on one GPU: the same text-format AppConfig a user of the reference would write selects
DARLIN, the plain batch solver, online FTRL or model evaluation; data comes from text files through the native
readers; the model is written as `<file>_S<rank>`."""
import os

import numpy as np
import pytest
import torch

from parameter_server_b200 import config as cfg
from parameter_server_b200.data.synthetic import write_libsvm_parts, zipf_sparse_matrix
from parameter_server_b200.utils.modelio import read_model_text

pytestmark = pytest.mark.gpu

BATCH = '''
app_name: "job" parameter_name: "job_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{d}/train/part-.*" }}
  validation_data {{ format: TEXT text: LIBSVM file: "{d}/valid/part-.*" }}
  local_cache {{ format: BIN file: "{d}/cache/" }}
  model_output {{ format: TEXT file: "{d}/model" }}
  loss {{ type: LOGIT }} penalty {{ type: L1 lambda: 0.5 }} learning_rate {{ type: CONSTANT eta: 1 }}
  solver {{ feature_block_ratio: 1 max_pass_of_data: 6 epsilon: 1e-6 tail_feature_freq: 0 }}
  {darling}
}}
'''


def _data(tmp, rows=3000, cols=2000):
    off, idx, vals, y, _ = zipf_sparse_matrix(rows, cols, 16, seed=3, device="cpu", zipf_s=0.8, wstar_frac=0.1, noise=0.1)
    h = rows * 4 // 5
    write_libsvm_parts(str(tmp / "train"), off[:h + 1], idx[:off[h]], vals[:off[h]], y[:h], 3, one_based=True)
    write_libsvm_parts(str(tmp / "valid"), off[h:] - off[h], idx[off[h]:], vals[off[h]:], y[h:], 1, one_based=True)


def _run(tmp, text, **flag_kw):
    from parameter_server_b200.apps.gpu_job import run_gpu_job

    conf = tmp / "job.conf"
    conf.write_text(text)
    return run_gpu_job(cfg.Flags(app=str(conf), **flag_kw))


def test_darlin_job_then_model_evaluation(tmp_path):
    _data(tmp_path)
    out = _run(tmp_path, BATCH.format(d=tmp_path, darling="darling { delta_init_value: 1 delta_max_value: 5 }"))
    objs = [p["objv"] for p in out["progress"]]
    assert len(objs) == 6 and objs[-1] < objs[0] and out["validation_auc"] > 0.75
    model = read_model_text(out["model"])
    assert out["model"].endswith("model_S0") and len(model) == out["progress"][-1]["nnz_w"] > 10
    assert min(model) >= 1                                   # one-based LIBSVM ids survive as keys
    ev = '''linear_method {{ validation_data {{ format: TEXT text: LIBSVM file: "{d}/valid/part-.*" }}
             model_input {{ format: TEXT file: "{d}/model_S0" }} local_cache {{ format: BIN file: "{d}/cache/" }} }}'''
    res = _run(tmp_path, ev.format(d=tmp_path))
    assert res["auc"] == pytest.approx(out["validation_auc"], abs=1e-6) and res["model_nnz"] == len(model)


def test_checkpoint_resume_gives_the_same_run(tmp_path):
    _data(tmp_path)
    text = BATCH.format(d=tmp_path, darling="darling { delta_init_value: 1 delta_max_value: 5 }")
    full = _run(tmp_path, text)
    ck = str(tmp_path / "ckpt")
    part = _run(tmp_path, text.replace("max_pass_of_data: 6", "max_pass_of_data: 3"), checkpoint_dir=ck, checkpoint_interval=1)
    assert len(part["progress"]) == 3 and len(os.listdir(ck)) == 3
    rest = _run(tmp_path, text, checkpoint_dir=ck, checkpoint_interval=1)      # resumes after pass 2
    assert len(rest["progress"]) == 6
    for a, b in zip(full["progress"], rest["progress"]):
        assert b["objv"] == pytest.approx(a["objv"], rel=2e-4)


def test_warm_start_from_a_model_dump(tmp_path):
    """init_w { type: FILE }: a second job starts from the dump of the first and carries on from its objective."""
    _data(tmp_path)
    text = BATCH.format(d=tmp_path, darling="darling { delta_init_value: 1 delta_max_value: 5 }")
    first = _run(tmp_path, text.replace("max_pass_of_data: 6", "max_pass_of_data: 4"))
    a = [p["objv"] for p in first["progress"]]
    warm = text.replace("max_pass_of_data: 6", "max_pass_of_data: 2").replace(
        "loss {", 'init_w {{ type: FILE file_name: "{d}/model" }} loss {{'.format(d=tmp_path), 1)
    second = _run(tmp_path, warm)
    b = [p["objv"] for p in second["progress"]]
    assert len(b) == 2
    assert b[0] < a[1] and b[0] <= a[-1] * 1.01           # first pass from the dump: at the level the first job had reached
    assert b[-1] <= b[0] * 1.001


def test_darlin_job_under_a_scheduler_node(tmp_path):
    """-gpu_scheduler: the passes are tasks of a scheduler node of the host control plane; same run, same model."""
    _data(tmp_path)
    text = BATCH.format(d=tmp_path, darling="darling { delta_init_value: 1 delta_max_value: 5 }")
    plain = _run(tmp_path, text)
    model_plain = read_model_text(plain["model"])
    ctl = _run(tmp_path, text, gpu_scheduler=True, report_interval=0.05)
    # float atomics sum in a different order from run to run: equal within the tolerance of the resume test
    assert [p["objv"] for p in ctl["progress"]] == pytest.approx([p["objv"] for p in plain["progress"]], rel=2e-4)
    assert [p["objv"] for p in ctl["scheduler_progress"]] == [p["objv"] for p in ctl["progress"]]     # what the ranks replied
    assert [p["nnz_w"] for p in ctl["scheduler_progress"]] == [p["nnz_w"] for p in ctl["progress"]]
    model = read_model_text(ctl["model"])
    common = set(model) & set(model_plain)
    assert ctl["model"].endswith("model_S0") and len(common) >= 0.98 * max(len(model), len(model_plain))
    assert max(abs(model[k] - model_plain[k]) for k in common) < 5e-3
    assert "W0" in ctl["dashboard"] and ("cuda:0" in ctl["dashboard"] or "no report yet" in ctl["dashboard"])
    assert ctl["validation_auc"] == pytest.approx(plain["validation_auc"], abs=2e-3)


def test_plain_batch_solver_job(tmp_path):
    _data(tmp_path)
    out = _run(tmp_path, BATCH.format(d=tmp_path, darling="learner { type: PROXIMAL_GRADIENT }"))
    objs = [p["objv"] for p in out["progress"]]
    assert objs[-1] < objs[0] and out["validation_auc"] > 0.75 and os.path.exists(out["model"])


def test_ftrl_job_from_adfea_text(tmp_path):
    rng = np.random.RandomState(0)
    w = {k: rng.randn() for k in range(300)}
    (tmp_path / "ctr").mkdir()
    for f in range(2):
        lines = []
        for i in range(3000):
            ks = rng.choice(300, size=8, replace=False)
            p = 1 / (1 + np.exp(-(sum(w[k] for k in ks) * 0.8 - 0.5)))
            lines.append(f"{i} 1 {int(rng.rand() < p)} " + " ".join(f"{k * 7919 + 11}:{1 + k % 3}" for k in ks))
        (tmp_path / "ctr" / f"part-{f}").write_text("\n".join(lines) + "\n")
    text = f'''app_name: "ctr" parameter_name: "ctr_w"
      linear_method {{ training_data {{ format: TEXT text: ADFEA file: "{tmp_path}/ctr/part-.*" ignore_feature_group: true }}
        model_output {{ format: TEXT file: "{tmp_path}/ftrl" }} loss {{ type: LOGIT }}
        penalty {{ type: L1 lambda: 0.01 lambda: 0.01 }} learning_rate {{ type: CONSTANT alpha: 0.1 beta: 1 }}
        solver {{ minibatch_size: 500 countmin_n: 100000 eval_interval: 1000 }} ftrl {{ }} }}'''
    out = _run(tmp_path, text)
    assert out["examples"] == 6000 and out["mean_logloss_last"] < 0.69 and out["nnz_w"] > 50
    model = read_model_text(out["model"])
    assert len(model) == out["nnz_w"] and all((k - 11) % 7919 == 0 for k in model)


def test_ftrl_job_checkpoint_resume(tmp_path):
    """A restarted online job reloads the newest checkpoint, skips the minibatches applied before it and
    ends in the model of the uninterrupted run."""
    rng = np.random.RandomState(1)
    w = {k: rng.randn() for k in range(200)}
    (tmp_path / "ctr").mkdir()
    lines = []
    for i in range(4000):
        ks = rng.choice(200, size=6, replace=False)
        p = 1 / (1 + np.exp(-(sum(w[k] for k in ks) * 0.8)))
        lines.append(f"{i} 1 {int(rng.rand() < p)} " + " ".join(f"{k * 7919 + 11}:1" for k in ks))
    (tmp_path / "ctr" / "part-0").write_text("\n".join(lines) + "\n")
    text = f'''app_name: "ctr" parameter_name: "ctr_w"
      linear_method {{ training_data {{ format: TEXT text: ADFEA file: "{tmp_path}/ctr/part-.*" ignore_feature_group: true }}
        model_output {{ format: TEXT file: "{tmp_path}/ftrl" }} loss {{ type: LOGIT }}
        penalty {{ type: L1 lambda: 0.01 lambda: 0.01 }} learning_rate {{ type: CONSTANT alpha: 0.1 beta: 1 }}
        solver {{ minibatch_size: 500 countmin_n: 100000 tail_feature_freq: 2 eval_interval: 1000 }} ftrl {{ }} }}'''
    ck = tmp_path / "ck"
    full = _run(tmp_path, text, checkpoint_dir=str(ck), checkpoint_interval=3)
    model_full = read_model_text(full["model"])
    steps = sorted(int(n.split("step")[1][:-3]) for n in os.listdir(ck))
    assert steps == [3, 6]                                   # 8 minibatches, a checkpoint every 3
    os.remove(ck / "ftrl_rank0_step6.pt")                    # "crash" after minibatch 3..5: resume from step 3
    again = _run(tmp_path, text, checkpoint_dir=str(ck), checkpoint_interval=3)
    model_again = read_model_text(again["model"])
    common = set(model_again) & set(model_full)                # float atomics: a weight at the L1 threshold may flip to 0
    assert again["examples"] == 4000 and len(model_full) > 20 and len(common) >= 0.97 * max(len(model_full), len(model_again))
    for k in common:
        assert model_again[k] == pytest.approx(model_full[k], rel=2e-3, abs=1e-5)
