"""FTRL engine on degenerate minibatches against the fp64 oracle (collected late: after the other kernel tests)."""
import numpy as np
import pytest
import torch

from baseline.cpu_ref.ftrl_ref import FTRLRef
from tests.test_ftrl_gpu import _engine

pytestmark = pytest.mark.gpu

@pytest.mark.parametrize("rule", ["count", "sumsq"])
def test_edge_case_minibatches_match_oracle(rule):
    """Single row, the same key twice in a row, the smallest and the largest legal key (2^64 - 2), an empty
    minibatch between two others (what a rank feeds when its files run out before the other ranks')."""
    from parameter_server_b200.models.ftrl import DeviceMinibatch

    eng, hy = _engine(rule=rule)
    ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, rule)
    top = np.uint64(2**64 - 2)
    batches = [
        (np.array([0, 3]), np.array([7, 7, 9], dtype=np.uint64), np.array([1.0])),                       # one row, duplicate key
        (np.array([0]), np.array([], dtype=np.uint64), np.array([])),                                      # empty
        (np.array([0, 2, 2, 5]), np.array([0, top, 7, 9, top], dtype=np.uint64), np.array([-1.0, 1.0, 1.0])),  # a row without features
        (np.array([0, 1]), np.array([top], dtype=np.uint64), np.array([-1.0])),
    ]
    for off, keys, y in batches * 3:
        mb = DeviceMinibatch(torch.from_numpy(off.astype(np.int64)).cuda(), torch.from_numpy(keys.view(np.int64).copy()).cuda(),
                             torch.from_numpy(y.astype(np.float32)).cuda())
        eng.step(mb)
        eng.check_status()
        ref.step([(off.astype(np.int64), keys, y.astype(np.float64))])
    k, w = eng.dump_model()
    rk, rw = ref.nonzero()
    assert np.array_equal(k, rk) and len(rk) >= 2 and int(rk[-1]) == 2**64 - 2
    np.testing.assert_allclose(w, rw, rtol=2e-3, atol=2e-5)
    st = eng.read_stats(reset=False)
    assert st["table_entries"] == len(ref.model) and st["rows"] == 3 * 5
