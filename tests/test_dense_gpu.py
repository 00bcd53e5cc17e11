"""tcgen05 TF32 GEMM and the NN elementwise kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_act(x, act):
    if act == "RELU":
        return torch.relu(x)
    if act == "SCALED_TANH":
        return 1.7159 * torch.tanh(2.0 / 3.0 * x)
    if act == "SIGMOID":
        return torch.sigmoid(x)
    return x


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (128, 128, 256), (256, 384, 96), (200, 130, 72), (1000, 520, 1024), (64, 8, 4),
                                   # >= 148 tiles of 128x256: the persistent kernel (several tiles per CTA, ragged edges, short K)
                                   (2048, 4096, 512), (1925, 2563, 260), (4096, 4224, 36), (9000, 2100, 64)])
@pytest.mark.parametrize("act", ["IDENTITY", "RELU", "SCALED_TANH"])
def test_gemm_tn_matches_fp32(M, N, K, act):
    from parameter_server_b200.ops import dense

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g, device="cuda")
    b = torch.randn(N, K, generator=g, device="cuda") / K ** 0.5
    out = dense.gemm_tn(a, b, act)
    torch.cuda.synchronize()
    dense.check_status(a.device)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = _ref_act(a.double() @ b.double().T, act).float()
    torch.backends.cuda.matmul.allow_tf32 = prev
    err = (out - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err        # TF32: 10-bit mantissa
    assert (out - ref).abs().mean().item() < 2e-3


def test_gemm_strided_views_and_repeat():
    from parameter_server_b200.ops import dense

    big = torch.randn(300, 256, device="cuda")
    a, b = big[:260, :128], big[4:132, 128:]            # row stride 256, offsets keep 16-byte alignment
    o1 = dense.gemm_tn(a, b)
    o2 = dense.gemm_tn(a, b)
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)
    assert (o1 - a @ b.T).abs().max().item() < 0.2
    with pytest.raises(ValueError):
        dense.gemm_tn(big[:, :127], big[:, 1:128])


def test_elementwise_kernels():
    from parameter_server_b200.ops import dense

    x = torch.randn(333, 77, device="cuda")
    assert torch.equal(dense.transpose(x), x.T.contiguous())
    g = torch.randn_like(x)
    for act in ("IDENTITY", "RELU", "SCALED_TANH", "SIGMOID"):
        xr = x.clone().requires_grad_(True)
        y = _ref_act(xr, act)
        y.backward(g)
        z = dense.act_backward(g, y.detach(), act)
        torch.testing.assert_close(z, xr.grad, rtol=1e-4, atol=1e-5)
    yl = torch.where(torch.rand(1000, device="cuda") < 0.5, 1.0, -1.0)
    s = torch.randn(1000, device="cuda")
    loss, grad = dense.logistic_loss(s, yl)
    sr = s.clone().requires_grad_(True)
    ref = torch.nn.functional.softplus(-sr * yl).sum()
    ref.backward()
    assert loss.item() == pytest.approx(ref.item(), rel=1e-5)
    torch.testing.assert_close(grad, sr.grad, rtol=1e-4, atol=1e-6)
    w, gw, h = torch.randn(500, device="cuda"), torch.randn(500, device="cuda"), torch.zeros(500, device="cuda")
    w0 = w.clone()
    dense.sgd_update(w, gw, None, 0.1, 1.0, 9)
    torch.testing.assert_close(w, w0 - 0.1 * gw / (1.0 + 3.0))
    w1 = w.clone()
    dense.sgd_update(w, gw, h, 0.1, 1.0, 9)
    torch.testing.assert_close(h, gw * gw)
    torch.testing.assert_close(w, w1 - 0.1 * gw / (1.0 + gw.abs()))
    m = torch.randn(200, 9, device="cuda") * 3 + 1
    dense.col_normalize(m)
    torch.testing.assert_close(m.mean(0), torch.zeros(9, device="cuda"), atol=1e-5, rtol=0)
    torch.testing.assert_close(m.norm(dim=0), torch.full((9,), 200 ** 0.5, device="cuda"), rtol=1e-4, atol=1e-4)
