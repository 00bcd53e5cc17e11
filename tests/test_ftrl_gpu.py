"""FTRL fused kernels on one GPU against the fp64 CPU restatement of the reference."""
import numpy as np
import pytest
import torch

from baseline.cpu_ref.ftrl_ref import FTRLRef
from parameter_server_b200.data.synthetic import ctr_minibatch

pytestmark = pytest.mark.gpu


def _engine(impl="fused", rule="count", **kw):
    from parameter_server_b200.models.ftrl import FTRLEngine, FTRLHyper
    from parameter_server_b200.parallel.peer import PeerGroup

    hyper = FTRLHyper(alpha=0.02, beta=1.0, lambda1=0.05, lambda2=0.1, rule=rule)
    args = dict(table_capacity=1 << 16, max_rows=4096, max_nnz=1 << 19, local_capacity=1 << 16)
    args.update(kw)
    return FTRLEngine(PeerGroup.single(torch.device("cuda", 0)), hyper, impl=impl, **args), hyper


def _batches(n, rows=700, log2=13):
    return [ctr_minibatch(rows, seed=100 + i, device="cuda", key_space_log2=log2, bias=-0.5, wstar_frac=0.2,
                          wstar_std=1.0) for i in range(n)]


@pytest.mark.parametrize("impl,rule,counts", [("fused", "count", None), ("fused", "sumsq", None),
                                              ("fused", "sumsq", True), ("nccl", "count", None)])
def test_ftrl_matches_oracle(impl, rule, counts):
    from parameter_server_b200.models.ftrl import DeviceMinibatch

    eng, hy = _engine(impl, rule, track_counts=counts)
    assert eng.track_counts == (rule == "count" or bool(counts))
    ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, rule)
    for off, keys, y in _batches(6):
        eng.step(DeviceMinibatch(off, keys, y))
        st = eng.read_stats()
        eng.check_status()
        loss = ref.step([(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64), y.cpu().numpy().astype(np.float64))])
        assert st["rows"] == y.numel()
        assert st["loss_sum"] == pytest.approx(loss, rel=2e-4)
    k, w = eng.dump_model()
    rk, rw = ref.nonzero()
    assert len(rk) > 50
    assert np.array_equal(k, rk)
    np.testing.assert_allclose(w, rw, rtol=2e-3, atol=2e-5)
    st = eng.read_stats(reset=False)
    assert st["nnz_w"] == ref.nnz
    assert st["norm1"] == pytest.approx(ref.norm1, rel=1e-3)
    assert st["table_entries"] == len(ref.model)
    assert eng.penalty(st) == pytest.approx(ref.objv(), rel=1e-3)


@pytest.mark.parametrize("rule", ["count", "sumsq"])
def test_ftrl_valued_features_and_predict(rule):
    from parameter_server_b200.models.ftrl import DeviceMinibatch

    eng, hy = _engine(rule=rule)
    ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, rule)
    g = torch.Generator(device="cuda").manual_seed(3)
    for off, keys, y in _batches(4, rows=300, log2=10):
        vals = torch.rand(keys.numel(), generator=g, device="cuda") + 0.5
        eng.step(DeviceMinibatch(off, keys, y, vals))
        ref.step([(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64), y.cpu().numpy().astype(np.float64),
                   vals.cpu().numpy())])
    off, keys, y = _batches(1, rows=200, log2=10)[0]
    xw = eng.predict(DeviceMinibatch(off, keys, y)).cpu().numpy()
    _, _, _, _, _, rxw = ref.worker_gradient(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64),
                                             y.cpu().numpy().astype(np.float64))
    np.testing.assert_allclose(xw, rxw, rtol=2e-3, atol=2e-4)
    # predict leaves training state untouched: one more step still matches
    eng.step(DeviceMinibatch(off, keys, y))
    ref.step([(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64), y.cpu().numpy().astype(np.float64))])
    k, w = eng.dump_model()
    rk, rw = ref.nonzero()
    assert np.array_equal(k, rk)
    np.testing.assert_allclose(w, rw, rtol=2e-3, atol=2e-5)
    eng.check_status()


@pytest.mark.parametrize("impl", ["fused", "nccl"])
def test_tail_feature_filter_matches_oracle(impl):
    """Keys enter the model only once their count-min estimate exceeds tail_feature_freq."""
    from parameter_server_b200.models.ftrl import DeviceMinibatch, FTRLEngine, FTRLHyper
    from parameter_server_b200.parallel.peer import PeerGroup

    hy = FTRLHyper(alpha=0.02, beta=1.0, lambda1=0.05, lambda2=0.1, tail_feature_freq=3, countmin_n=1 << 15, countmin_k=2)
    eng = FTRLEngine(PeerGroup.single(torch.device("cuda", 0)), hy, impl=impl, table_capacity=1 << 16, max_rows=4096,
                     max_nnz=1 << 19, local_capacity=1 << 16)
    ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, tail_freq=3, countmin_n=hy.countmin_n, countmin_k=2)
    seen = set()
    for off, keys, y in _batches(4, rows=300, log2=14):
        eng.step(DeviceMinibatch(off, keys, y))
        eng.check_status()
        hk = keys.cpu().numpy().view(np.uint64)
        seen.update(hk.tolist())
        ref.step([(off.cpu().numpy(), hk, y.cpu().numpy().astype(np.float64))])
    st = eng.read_stats(reset=False)
    assert st["table_entries"] == len(ref.model)
    assert 50 < len(ref.model) < 0.8 * len(seen)      # the filter kept a real share of the keys out
    k, w = eng.dump_model()
    rk, rw = ref.nonzero()
    assert np.array_equal(k, rk)
    np.testing.assert_allclose(w, rw, rtol=2e-3, atol=2e-5)


def test_ftrl_reports_local_table_overflow():
    from parameter_server_b200.models.ftrl import DeviceMinibatch

    eng, _ = _engine(local_capacity=256, max_probe=64)
    off, keys, y = _batches(1, rows=200)[0]
    eng.step(DeviceMinibatch(off, keys, y))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="dedup table full"):
        eng.check_status()


def test_model_text_dump(tmp_path):
    from parameter_server_b200.models.ftrl import DeviceMinibatch
    from parameter_server_b200.utils.modelio import read_model_text

    eng, _ = _engine()
    for off, keys, y in _batches(3):
        eng.step(DeviceMinibatch(off, keys, y))
    path = eng.save_model(str(tmp_path / "ftrl"))
    assert path.endswith("_S0")
    k, w = eng.dump_model()
    m = read_model_text(path)
    assert len(m) == len(k)
    for kk, ww in zip(k[:50], w[:50]):
        assert m[int(kk)] == pytest.approx(float(ww), rel=1e-5)



def test_compact_inputs_give_the_same_model():
    """32-bit feature ids hashed on the device + 32-bit row offsets == the same minibatches as uint64 keys."""
    from parameter_server_b200.models.ftrl import KEY_U32, KEY_U32_HASHED, DeviceMinibatch

    a, _ = _engine(rule="sumsq")
    b, _ = _engine(rule="sumsq")
    c, _ = _engine(rule="sumsq")
    d, _ = _engine(rule="sumsq")
    for i in range(4):
        off, keys, y, fid = ctr_minibatch(500, seed=40 + i, device="cuda", key_space_log2=13, bias=-0.5, wstar_frac=0.2,
                                          wstar_std=1.0, return_ids=True)
        a.step(DeviceMinibatch(off, keys, y))
        b.step(DeviceMinibatch(off.to(torch.int32), fid, y, None, KEY_U32_HASHED))
        c.step(DeviceMinibatch(off, fid.to(torch.int64), y))             # the ids themselves as keys, 64 bits wide
        d.step(DeviceMinibatch(off.to(torch.int32), fid, y, None, KEY_U32))
    for e in (a, b, c, d):
        e.check_status()
    (ka, wa), (kb, wb), (kc, wc), (kd, wd) = a.dump_model(), b.dump_model(), c.dump_model(), d.dump_model()
    assert len(ka) > 50 and np.array_equal(ka, kb) and np.array_equal(kc, kd)
    np.testing.assert_allclose(wa, wb, rtol=1e-5, atol=1e-7)     # same arithmetic, different summation order of atomics
    np.testing.assert_allclose(wc, wd, rtol=1e-5, atol=1e-7)
    with pytest.raises(ValueError, match="32-bit keys"):
        a.step(DeviceMinibatch(off, fid, y))


@pytest.mark.parametrize("rule", ["count", "sumsq"])
def test_shard_table_grows_instead_of_filling_up(rule):
    """A shard that starts far too small doubles between steps; the model stays the oracle's."""
    from parameter_server_b200.models.ftrl import DeviceMinibatch

    eng, hy = _engine(rule=rule, table_capacity=1 << 11, local_capacity=1 << 13)
    assert eng.cap == 1 << 14                       # room for one worst-case step from the start
    ref = FTRLRef(hy.alpha, hy.beta, hy.lambda1, hy.lambda2, rule)
    for off, keys, y in _batches(6, rows=120, log2=13):
        eng.step(DeviceMinibatch(off, keys, y))
        eng.check_status()
        eng.maybe_grow()
        ref.step([(off.cpu().numpy(), keys.cpu().numpy().view(np.uint64), y.cpu().numpy().astype(np.float64))])
    assert eng.grown >= 1 and eng.cap > 1 << 14
    st = eng.read_stats(reset=False)
    assert st["table_entries"] == len(ref.model) and st["table_entries"] + eng.lcap <= eng.GROW_AT * eng.cap
    k, w = eng.dump_model()
    rk, rw = ref.nonzero()
    assert np.array_equal(k, rk)
    np.testing.assert_allclose(w, rw, rtol=2e-3, atol=2e-5)
