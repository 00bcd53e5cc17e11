"""AUC kernels: the device histogram equals the host class bin for bin, the exact AUC equals the host's
rank-sum value (ties included)."""
import numpy as np
import pytest
import torch

from parameter_server_b200.runtime import host

pytestmark = pytest.mark.gpu


def _data(n, seed, ties):
    g = torch.Generator(device="cuda").manual_seed(seed)
    y = torch.where(torch.rand(n, generator=g, device="cuda") < 0.3, 1.0, -1.0)
    p = torch.randn(n, generator=g, device="cuda") + 0.8 * y
    if ties:
        p = torch.round(p * 4) / 4          # many equal scores
    return y, p


@pytest.mark.parametrize("ties", [False, True])
def test_auc_histogram_and_exact_auc_match_the_host(ties):
    from parameter_server_b200.ops.evalops import auc_histogram, exact_auc

    H = host()
    y, p = _data(50_000, 5, ties)
    for goodness in (1000, 100000):
        ref = H.AUC()
        ref.set_goodness(goodness)
        ref.add(y.cpu().numpy(), p.cpu().numpy())
        got = auc_histogram(y, p, goodness)
        want = ref.data()
        for a, b in zip(got, want):
            assert list(a) == list(b)
        dev = H.AUC()
        dev.set_goodness(goodness)
        dev.merge_data(*got)
        assert dev.evaluate() == pytest.approx(ref.evaluate(), abs=1e-12)
    want = H.exact_auc(y.cpu().numpy(), p.cpu().numpy())
    assert exact_auc(y, p) == pytest.approx(want, abs=1e-9)
    assert 0.6 < want < 0.9
    # one class only: 0.5 by convention
    assert exact_auc(torch.ones(10, device="cuda"), torch.rand(10, device="cuda")) == 0.5
