import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 257, 100_003, 5_000_000])
def test_reduce_ops_match_fp64(n):
    from parameter_server_b200.ops.reduce import reduce_sum

    g = torch.Generator(device="cuda").manual_seed(n)
    x = torch.randn(n, generator=g, device="cuda") * 3
    xd = x.double()
    dual = torch.exp(x)
    assert reduce_sum(dual, "sum_log1p_inv").item() == pytest.approx(torch.log1p(1 / dual.double()).sum().item(), rel=1e-9)
    assert reduce_sum(x, "sum_logistic").item() == pytest.approx(torch.nn.functional.softplus(-xd).sum().item(), rel=1e-9)
    w = x.clone()
    w[::3] = 0
    w[1::7] = float("nan")
    fin = torch.nan_to_num(w.double(), nan=0.0)
    assert reduce_sum(w, "sum_abs").item() == pytest.approx(fin.abs().sum().item(), rel=1e-9)
    assert reduce_sum(w, "count_nonzero").item() == (fin != 0).sum().item()
    # deterministic: bitwise equal on repeat
    a, b = reduce_sum(dual, "sum_log1p_inv").item(), reduce_sum(dual, "sum_log1p_inv").item()
    assert a == b
