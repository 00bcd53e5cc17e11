#!/usr/bin/env python
"""Plumbing configuration: L1-LR via DARLIN with 1 scheduler + 2 servers + 2 workers as CPU processes on
localhost (TCP van).  Data: 10,000 rows x 65,536 features, 20 nnz/row with uniform keys mod 2^16, values 1.0,
planted w* (5 % non-zero, N(0,1)), labels sign(X.w* + N(0,0.1)); lambda1 = 1, 10 passes, seed 0.
Prints the objective per pass of the multi-process run and of the single-process fp64 oracle.

  python baseline/run_config0.py [workdir]
"""
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from baseline.cpu_ref.darlin_ref import DarlinConfig, DarlinRef  # noqa: E402
from parameter_server_b200.data.synthetic import write_libsvm_parts  # noqa: E402
from parameter_server_b200.utils.modelio import read_model_text  # noqa: E402


def main():
    work = sys.argv[1] if len(sys.argv) > 1 else "/tmp/psb200_config0"
    os.makedirs(work, exist_ok=True)
    rows, cols, nnz = 10000, 65536, 20
    g = torch.Generator().manual_seed(0)
    keys = torch.randint(0, cols, (rows, nnz), generator=g).sort(1).values
    keep = torch.ones_like(keys, dtype=torch.bool)
    keep[:, 1:] = keys[:, 1:] != keys[:, :-1]
    counts = keep.sum(1)
    off = torch.zeros(rows + 1, dtype=torch.int64)
    off[1:] = counts.cumsum(0)
    idx = keys[keep]
    w = torch.randn(cols, generator=g) * (torch.rand(cols, generator=g) < 0.05)
    xw = torch.zeros(rows).index_add_(0, torch.repeat_interleave(torch.arange(rows), counts), w[idx])
    y = torch.sign(xw + 0.1 * torch.randn(rows, generator=g))
    y[y == 0] = 1
    vals = torch.ones(idx.numel())
    write_libsvm_parts(os.path.join(work, "train"), off, idx, vals, y, 2)
    conf = os.path.join(work, "job.conf")
    with open(conf, "w") as f:
        f.write(f'''app_name: "config0"
parameter_name: "config0_w"
linear_method {{
  training_data {{ format: TEXT text: LIBSVM file: "{work}/train/part-.*" }}
  local_cache {{ format: BIN file: "{work}/cache/" }}
  model_output {{ format: TEXT file: "{work}/model" }}
  loss {{ type: LOGIT }}
  penalty {{ type: L1 lambda: 1 }}
  learning_rate {{ type: CONSTANT eta: 1 }}
  solver {{ feature_block_ratio: 1 max_pass_of_data: 10 max_block_delay: 0 epsilon: 1e-9 tail_feature_freq: 0 }}
  darling {{ delta_init_value: 1 delta_max_value: 5 kkt_filter_threshold_ratio: 10 }}
}}
''')
    t0 = time.time()
    rc = subprocess.call([sys.executable, "-m", "parameter_server_b200.launch", "-num_servers", "2", "-num_workers", "2",
                          "-app", conf, "-seed", "0"], cwd=ROOT)
    t_job = time.time() - t0
    k = idx.numpy().astype(np.uint64)
    o = off.numpy()
    h = rows // 2
    shards = [(o[:h + 1], k[:o[h]], vals.numpy()[:o[h]], y.numpy()[:h]), (o[h:] - o[h], k[o[h]:], vals.numpy()[o[h]:], y.numpy()[h:])]
    t0 = time.time()
    ref = DarlinRef(shards, None, DarlinConfig(lambda1=1.0, max_pass=10, feature_block_ratio=1.0, epsilon=1e-9, seed=0))
    prog = ref.run()
    t_ref = time.time() - t0
    for i, p in enumerate(prog):
        print(f"oracle pass {i}: objective {p.objv:.6f} |w|_0 {p.nnz_w} active {p.nnz_active}")
    model = {}
    for s in ("S0", "S1"):
        path = os.path.join(work, f"model_{s}")
        if os.path.exists(path):
            model.update(read_model_text(path))
    rk, rw = ref.model()
    same = sorted(model) == rk.tolist() and all(abs(model[a] - b) <= 1e-5 * max(1, abs(b)) for a, b in zip(rk.tolist(), rw.tolist()))
    print(f"job rc={rc} wall {t_job:.1f}s ({rows * len(prog) / t_job:.0f} examples/s incl. start-up, load and preprocessing); "
          f"oracle {t_ref:.1f}s; model dump equal to oracle: {same} ({len(model)} non-zero weights)")
    return 0 if (rc == 0 and same) else 1


if __name__ == "__main__":
    sys.exit(main())
