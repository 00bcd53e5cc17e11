"""The command line on GPUs: `launch -gpus N -app job.conf` runs one rank per GPU; the per-rank model files
together equal the single-GPU model of the same job."""
import os
import subprocess
import sys

import numpy as np
import pytest

from parameter_server_b200.data.synthetic import write_libsvm_parts, zipf_sparse_matrix
from parameter_server_b200.utils.modelio import read_model_text

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONF = '''
app_name: "cli" parameter_name: "cli_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{d}/train/part-.*" }}
  local_cache {{ format: BIN file: "{d}/cache{tag}/" }}
  model_output {{ format: TEXT file: "{d}/model{tag}" }}
  loss {{ type: LOGIT }} penalty {{ type: L1 lambda: 0.5 }} learning_rate {{ type: CONSTANT eta: 1 }}
  solver {{ feature_block_ratio: 1 max_pass_of_data: 5 epsilon: 1e-7 tail_feature_freq: 0 }}
  darling {{ delta_init_value: 1 delta_max_value: 5 }}
}}
'''


def test_launch_gpus_2_matches_single_gpu(tmp_path):
    off, idx, vals, y, _ = zipf_sparse_matrix(4000, 3000, 16, seed=9, device="cpu", zipf_s=0.8, wstar_frac=0.1, noise=0.1)
    write_libsvm_parts(str(tmp_path / "train"), off, idx, vals, y, 4, one_based=True)
    models = {}
    for n in (1, 2):
        conf = tmp_path / f"job{n}.conf"
        conf.write_text(CONF.format(d=tmp_path, tag=n))
        r = subprocess.run([sys.executable, "-m", "parameter_server_b200.launch", "-gpus", str(n), "-app", str(conf)],
                           cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
        m = {}
        for rank in range(n):
            path = tmp_path / f"model{n}_S{rank}"
            assert path.exists()
            part = read_model_text(str(path))
            assert not (set(part) & set(m))               # disjoint key ranges
            m.update(part)
        models[n] = m
    k1, k2 = set(models[1]), set(models[2])
    assert len(k1 & k2) >= 0.97 * max(len(k1), len(k2)) > 30
    err = max(abs(models[1][k] - models[2][k]) for k in k1 & k2)
    assert err < 5e-2
