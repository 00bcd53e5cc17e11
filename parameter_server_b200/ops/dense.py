"""Dense-layer operators of the neural-network app on the sm_100a kernels
(``csrc/gemm_tcgen05.cu``): TF32 tcgen05 GEMM with fused activation, tiled transpose,
activation backward, logistic loss, SGD / AdaGrad update, column normalisation."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _native as N

ACT = {"IDENTITY": 0, "RELU": 1, "SCALED_TANH": 2, "SIGMOID": 3}
_status = {}


def _status_for(dev) -> torch.Tensor:
    k = (dev.type, dev.index)
    if k not in _status:
        _status[k] = torch.zeros(8, dtype=torch.int32, device=dev)
    return _status[k]


def check_status(dev) -> None:
    st = _status_for(dev).tolist()
    if st[0] != 0:
        _status_for(dev).zero_()
        raise RuntimeError(f"GEMM kernel gave up waiting (code {st[0]}, tile {st[1]},{st[2] - 100})")


def gemm_tn(a: torch.Tensor, b: torch.Tensor, act: str = "IDENTITY", out: Optional[torch.Tensor] = None,
            pad_k: bool = False) -> torch.Tensor:
    """``act(a @ b.T)`` for row-major fp32 ``a`` [M,K] and ``b`` [N,K] on the tcgen05 tensor cores (TF32)."""
    assert a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape[1] == b.shape[1]
    assert a.stride(1) == 1 and b.stride(1) == 1
    M, K = a.shape
    Nn = b.shape[0]
    if pad_k and K % 4:
        # TMA needs row strides that are multiples of 16 bytes: zero-pad the contraction dimension
        kp = (K + 3) // 4 * 4
        a = torch.nn.functional.pad(a, (0, kp - K))
        b = torch.nn.functional.pad(b, (0, kp - K))
        K = kp
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.float32, device=a.device)
    rc = N.lib().psb_gemm_tn_tf32(N.ptr(a), N.ptr(b), N.ptr(out), M, Nn, K, a.stride(0), b.stride(0), out.stride(0), ACT[act],
                                  N.ptr(_status_for(a.device)), N.stream_ptr())
    if rc == 1:
        raise ValueError("gemm_tn needs 16-byte aligned operands whose row strides are multiples of 4 floats")
    N.check(rc, "gemm_tn_tf32")
    return out


def transpose(x: torch.Tensor) -> torch.Tensor:
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    out = torch.empty((x.shape[1], x.shape[0]), dtype=torch.float32, device=x.device)
    N.check(N.lib().psb_transpose(N.ptr(x), N.ptr(out), x.shape[0], x.shape[1], N.stream_ptr()), "transpose")
    return out


def act_backward(g: torch.Tensor, y: torch.Tensor, act: str) -> torch.Tensor:
    z = torch.empty_like(g)
    N.check(N.lib().psb_act_backward(N.ptr(g), N.ptr(y), N.ptr(z), C.c_size_t(g.numel()), ACT[act], N.stream_ptr()), "act_backward")
    return z


def logistic_loss(x: torch.Tensor, y: torch.Tensor, want_grad: bool = True):
    """(Σ log(1+e^{-x·y}) as a 1-element fp64 tensor, −y/(1+e^{x·y}) or None)."""
    loss = torch.zeros(1, dtype=torch.float64, device=x.device)
    grad = torch.empty_like(x) if want_grad else None
    N.check(N.lib().psb_logistic_loss(N.ptr(x), N.ptr(y), N.ptr(grad), C.c_size_t(x.numel()), N.ptr(loss), N.stream_ptr()), "logistic_loss")
    return loss, grad


def sgd_update(w: torch.Tensor, g: torch.Tensor, h: Optional[torch.Tensor], alpha: float, beta: float, it: int) -> None:
    N.check(N.lib().psb_sgd_update(N.ptr(w), N.ptr(g), N.ptr(h), C.c_size_t(w.numel()), C.c_float(alpha), C.c_float(beta),
                                   C.c_float(float(it)), 0 if h is None else 1, N.stream_ptr()), "sgd_update")


def col_normalize(x: torch.Tensor) -> None:
    assert x.is_contiguous() and x.dim() == 2
    N.check(N.lib().psb_col_normalize(N.ptr(x), x.shape[0], x.shape[1], N.stream_ptr()), "col_normalize")


def sparse_fc_forward(off: torch.Tensor, idx: torch.Tensor, vals: Optional[torch.Tensor], w: torch.Tensor, act: str = "IDENTITY") -> torch.Tensor:
    """Y = act(X·W) for CSR X (int64 offsets, int32 column ids, float32 values or None = ones) and W [in, out]
    (out a multiple of 4): the embedding-bag sum of the sparse fully connected layer."""
    rows, (in_dim, out_dim) = off.numel() - 1, w.shape
    y = torch.empty((rows, out_dim), dtype=torch.float32, device=w.device)
    N.check(N.lib().psb_spfc_forward(N.ptr(off), N.ptr(idx), N.ptr(vals), N.ptr(w), N.ptr(y), rows, in_dim, out_dim, ACT[act],
                                     N.ptr(_status_for(w.device)), N.stream_ptr()), "spfc_forward")
    return y


def sparse_fc_backward(off: torch.Tensor, idx: torch.Tensor, vals: Optional[torch.Tensor], y: torch.Tensor, gy: torch.Tensor,
                       in_dim: int, act: str = "IDENTITY") -> torch.Tensor:
    """Wg = Xᵀ·(dY ∘ act'(Y)) as [in, out]."""
    rows, out_dim = y.shape
    wg = torch.zeros((in_dim, out_dim), dtype=torch.float32, device=y.device)
    N.check(N.lib().psb_spfc_backward(N.ptr(off), N.ptr(idx), N.ptr(vals), N.ptr(y), N.ptr(gy.contiguous()), N.ptr(wg), rows, in_dim,
                                      out_dim, ACT[act], N.stream_ptr()), "spfc_backward")
    return wg
