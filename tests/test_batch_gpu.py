"""Plain batch solver kernels (block gradient / curvature for the logistic and the square hinge loss, learner
update, margin update) against an fp64 PyTorch restatement of the same block iteration."""
import math

import numpy as np
import pytest
import torch

from parameter_server_b200.data.synthetic import zipf_sparse_matrix

pytestmark = pytest.mark.gpu


def _reference(off, keys, vals, y, cfg, loss, penalty, learner, passes):
    """The same schedule in plain fp64 torch on the device: returns the objective after every pass and w."""
    from parameter_server_b200.models.darlin import block_order

    f64 = torch.float64
    uk, col = torch.unique(keys, return_inverse=True)
    rows, P = y.numel(), uk.numel()
    row = torch.repeat_interleave(torch.arange(rows, device=y.device), off[1:] - off[:-1])
    v = torch.ones(col.numel(), dtype=f64, device=y.device) if vals is None else vals.to(f64)
    yy, w, xw = y.to(f64), torch.zeros(P, dtype=f64, device=y.device), torch.zeros(rows, dtype=f64, device=y.device)
    per_row = col.numel() / rows
    nblk = max(int(math.ceil(per_row * cfg.feature_block_ratio)), 1)
    kmin, kmax = int(uk[0]), int(uk[-1]) + 1
    bounds = torch.tensor([kmin + (kmax - kmin) * i // nblk for i in range(nblk)] + [kmax], device=y.device)
    c = torch.searchsorted(uk, bounds)
    c[-1] = P
    blk = c.tolist()
    objs = []
    for order in block_order(nblk, passes, cfg.random_block_order, cfg.seed):
        for b in order.tolist():
            c0, c1 = blk[b], blk[b + 1]
            if c1 <= c0:
                continue
            sel = (col >= c0) & (col < c1)
            m = yy * xw
            if loss == "LOGIT":
                tau = torch.sigmoid(-m)
                g, h = -yy * tau, tau * (1 - tau)
            else:
                act = (m < 1).to(f64)
                g, h = -2 * yy * (1 - m) * act, 2 * act
            G = torch.zeros(c1 - c0, dtype=f64, device=y.device).index_add_(0, col[sel] - c0, g[row[sel]] * v[sel])
            U = torch.zeros(c1 - c0, dtype=f64, device=y.device).index_add_(0, col[sel] - c0, h[row[sel]] * v[sel] ** 2)
            wb, eta, lam = w[c0:c1], cfg.eta, cfg.lambda1
            if learner == "GRADIENT_DESCENT":
                d = -eta * (G + (2 * lam * wb if penalty == "L2" else 0.0))
            elif penalty == "L1":
                u = U / eta + 1e-10
                gp, gn = G + lam, G - lam
                d = torch.where(gp <= u * wb, -gp / u, torch.where(gn >= u * wb, -gn / u, -wb)).clamp(-5, 5)
            else:
                d = (-(G + 2 * lam * wb) / (U / eta + 2 * lam + 1e-10)).clamp(-5, 5)
            w[c0:c1] = wb + d
            xw.index_add_(0, row[sel], v[sel] * d[col[sel] - c0])
        m = yy * xw
        lv = torch.nn.functional.softplus(-m).sum() if loss == "LOGIT" else torch.clamp(1 - m, min=0).square().sum()
        objs.append(float(lv) + cfg.lambda1 * float(w.abs().pow(1 if penalty == "L1" else 2).sum()))
    return objs, uk, w


@pytest.mark.parametrize("loss,penalty,learner", [("LOGIT", "L1", "PROXIMAL_GRADIENT"), ("SQUARE_HINGE", "L1", "PROXIMAL_GRADIENT"),
                                                  ("SQUARE_HINGE", "L2", "PROXIMAL_GRADIENT"), ("LOGIT", "L2", "GRADIENT_DESCENT")])
def test_batch_solver_kernels_match_reference(loss, penalty, learner):
    from parameter_server_b200.models.batch import ProxGradientSolver
    from parameter_server_b200.models.darlin import DarlinConfig
    from parameter_server_b200.parallel.peer import PeerGroup

    off, idx, vals, y, _ = zipf_sparse_matrix(1200, 1500, 12, seed=9, device="cuda", zipf_s=0.8)
    keys = idx * 6151 + 5
    cfg = DarlinConfig(lambda1=0.2, eta=0.002 if learner == "GRADIENT_DESCENT" else 1.0, max_pass=4, epsilon=0.0,
                       feature_block_ratio=0.5, seed=2)
    sol = ProxGradientSolver(PeerGroup.single(torch.device("cuda", 0)), cfg, loss=loss, penalty=penalty, learner=learner)
    sol.preprocess(off, keys, vals, y)
    prog = sol.run()
    objs, uk, w = _reference(off, keys, vals, y, cfg, loss, penalty, learner, 4)
    assert sol.nblk > 2 and len(prog) == 4 and sol.kernel_launches > 4 * sol.nblk
    for p, o in zip(prog, objs):
        assert p.objv == pytest.approx(o, rel=1e-3)
    assert prog[-1].objv < prog[0].objv
    assert sol.w.numel() == uk.numel()                      # same global columns, ascending keys
    np.testing.assert_allclose(sol.w.cpu().numpy(), w.cpu().numpy(), rtol=2e-2, atol=2e-3)
    k, wk = sol.model()
    assert len(k) == int((sol.w != 0).sum()) and np.all(np.diff(k.astype(np.float64)) > 0)
