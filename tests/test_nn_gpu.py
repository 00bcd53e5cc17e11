"""Neural-network app: gradients of a 2-layer MLP against torch autograd (fp32) and a short training run."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NET = '''
neural_network {
  train { name: "train"
    layer { type: DATA name: "data" out: "x" out: "y" minibatch_size: %d }
    layer { type: FULLY_CONNECTED name: "fc1" in: "x" out: "h" size: 64 activation { type: %s } }
    layer { type: FULLY_CONNECTED name: "fc2" in: "h" out: "s" size: 4 activation { type: IDENTITY } lr_scale: 1 }
    layer { type: LOGISTIC_LOSS name: "loss" in: "s1" in: "y" }
  }
  test { name: "test"
    layer { type: DATA name: "tdata" out: "x" out: "y" }
    layer { type: FULLY_CONNECTED name: "fc1" in: "x" out: "h" size: 64 activation { type: %s } }
    layer { type: FULLY_CONNECTED name: "fc2" in: "h" out: "s" size: 4 activation { type: IDENTITY } }
    layer { type: AUC name: "auc" in: "s1" in: "y" }
  }
  solver { type: SGD update: %s lr { alpha: %g beta: 1 } max_iteration: %d display: 50 validation: %d }
}
'''


def _data(n, d, seed):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(n, d, generator=g)
    w1 = torch.randn(d, 8, generator=torch.Generator().manual_seed(99))
    s = torch.tanh(X @ w1).sum(1) + 0.3 * X[:, 0] * X[:, 1]
    y = torch.where(s > 0, 1.0, -1.0)
    return X, y


class _FirstColumn:
    """Loss/AUC layers take the first output unit: exposed as edge "s1" sharing storage with "s"."""


def _solver(act, update, alpha, iters, batch=256, valid=0):
    from parameter_server_b200 import config as cfg
    from parameter_server_b200.models.nn import SGDSolver
    from parameter_server_b200.parallel.peer import PeerGroup

    conf = cfg.parse_app_config((NET % (batch, act, act, update, alpha, iters, valid)).replace('"s1"', '"s"').replace("size: 4", "size: 1"))
    return SGDSolver(conf.neural_network, PeerGroup.single(torch.device("cuda", 0)))


@pytest.mark.parametrize("act", ["RELU", "SCALED_TANH"])
def test_gradients_match_autograd(act):
    sol = _solver(act, "NORMAL", 0.1, 1, batch=0)
    X, y = _data(512, 32, 1)
    sol.train.layer("data").set_data(X, y, normalize=False)
    sol.train.forward()
    sol.train.backward()
    w1 = sol.train.layer("fc1").model.value.clone().requires_grad_(True)
    w2 = sol.train.layer("fc2").model.value.clone().requires_grad_(True)
    xd, yd = X.cuda(), y.cuda()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    pre = xd @ w1.T
    h = torch.relu(pre) if act == "RELU" else 1.7159 * torch.tanh(2.0 / 3.0 * pre)
    s = (h @ w2.T).reshape(-1)
    loss = torch.nn.functional.softplus(-s * yd).sum()
    loss.backward()
    torch.backends.cuda.matmul.allow_tf32 = prev
    assert sol.train.layer("loss").loss.item() == pytest.approx(loss.item(), rel=2e-3)
    for name, ref in (("fc1", w1.grad), ("fc2", w2.grad)):
        got = sol.train.layer(name).model.gradient
        assert (got - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("update", ["NORMAL", "ADAGRAD"])
def test_training_reduces_loss_and_test_net_shares_the_model(update):
    sol = _solver("RELU", update, 0.05 if update == "NORMAL" else 0.1, 300, batch=256, valid=100)
    Xtr, ytr = _data(4096, 32, 2)
    Xte, yte = _data(1024, 32, 3)
    sol.train.layer("data").set_data(Xtr, ytr, normalize=False)
    sol.test.layer("tdata").set_data(Xte, yte, normalize=False)
    hist = sol.run(verbose=False)
    first = sum(h["loss"] for h in hist[:10]) / 10
    last = sum(h["loss"] for h in hist[-10:]) / 10
    assert last < 0.8 * first
    aucs = [h["test_auc"] for h in hist if h.get("test_auc") is not None]
    assert len(aucs) == 3 and aucs[-1] > 0.8
    assert sol.test.layer("fc1").model is sol.train.layer("fc1").model


SPARSE_NET = '''
neural_network {
  train { name: "train"
    layer { type: DATA name: "data" out: "x" out: "y" minibatch_size: %d }
    layer { type: SPARSE_FULLY_CONNECTED name: "emb" in: "x" out: "h" size: 32 activation { type: %s } }
    layer { type: FULLY_CONNECTED name: "fc2" in: "h" out: "s" size: 1 activation { type: IDENTITY } }
    layer { type: LOGISTIC_LOSS name: "loss" in: "s" in: "y" }
  }
  solver { type: SGD update: ADAGRAD lr { alpha: 0.1 beta: 1 } max_iteration: %d display: 50 }
}
'''


def _sparse_data(n, vocab, per_row, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, vocab, (n, per_row), generator=g).sort(1).values
    vals = torch.rand(n, per_row, generator=g) + 0.5
    off = torch.arange(n + 1, dtype=torch.int64) * per_row
    wtrue = torch.randn(vocab, generator=torch.Generator().manual_seed(7))
    y = torch.where((wtrue[idx] * vals).sum(1) > 0, 1.0, -1.0)
    return off, idx.reshape(-1).int(), vals.reshape(-1), y


@pytest.mark.parametrize("act", ["RELU", "SCALED_TANH", "SIGMOID"])
def test_sparse_fully_connected_layer_matches_autograd(act):
    """Embedding-bag forward and the model gradient against a dense fp32 torch restatement."""
    from parameter_server_b200 import config as cfg
    from parameter_server_b200.models.nn import SGDSolver
    from parameter_server_b200.parallel.peer import PeerGroup

    conf = cfg.parse_app_config(SPARSE_NET % (0, act, 1))
    sol = SGDSolver(conf.neural_network, PeerGroup.single(torch.device("cuda", 0)))
    n, vocab, per_row = 300, 500, 9
    off, idx, vals, y = _sparse_data(n, vocab, per_row, 4)
    sol.train.layer("data").set_sparse_data(off, idx, vals, y, vocab)
    sol.train.forward()
    sol.train.backward()
    emb, fc2 = sol.train.layer("emb"), sol.train.layer("fc2")
    W = emb.model.value.clone().requires_grad_(True)          # [vocab, 32]
    w2 = fc2.model.value.clone().requires_grad_(True)
    X = torch.zeros(n, vocab, device="cuda")
    X.index_put_((torch.arange(n, device="cuda").repeat_interleave(per_row), idx.cuda().long()), vals.cuda(), accumulate=True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    pre = X @ W
    h = {"RELU": torch.relu, "SIGMOID": torch.sigmoid, "SCALED_TANH": lambda t: 1.7159 * torch.tanh(2.0 / 3.0 * t)}[act](pre)
    s = (h @ w2.T).reshape(-1)
    loss = torch.nn.functional.softplus(-s * y.cuda()).sum()
    loss.backward()
    torch.backends.cuda.matmul.allow_tf32 = prev
    assert (emb.outputs[0].value - h).abs().max().item() < 1e-4 * max(1.0, h.abs().max().item())
    assert sol.train.layer("loss").loss.item() == pytest.approx(loss.item(), rel=2e-3)
    got, ref = emb.model.gradient, W.grad
    assert (got - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())


def test_sparse_net_trains():
    from parameter_server_b200 import config as cfg
    from parameter_server_b200.models.nn import SGDSolver
    from parameter_server_b200.parallel.peer import PeerGroup

    conf = cfg.parse_app_config(SPARSE_NET % (256, "RELU", 200))
    sol = SGDSolver(conf.neural_network, PeerGroup.single(torch.device("cuda", 0)))
    off, idx, vals, y = _sparse_data(4096, 300, 8, 5)
    sol.train.layer("data").set_sparse_data(off, idx, vals, y, 300)
    hist = sol.run(verbose=False)
    assert sum(h["loss"] for h in hist[-10:]) < 0.8 * sum(h["loss"] for h in hist[:10])
