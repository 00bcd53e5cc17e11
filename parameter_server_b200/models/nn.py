"""The neural-network application: a DAG of layers built from a ``NetConfig``, trained by SGD or
AdaGrad, with the dense layers on the tcgen05 tensor cores.

Reference: ``Net`` (src/neural_network/net.h:34-65), ``Layer`` + factory
(src/neural_network/layer.h:26-73, layer_inl.h:12-36), ``FullyConnectedLayer``
(fully_connected_layer.h:27-65), ``DataLayer`` (data_layer.h:11-52), ``LogisticLossLayer``
(loss_layer.h:33-59), ``AUCLayer`` (auc_layer.h:8-42), activations
(activation_function.h:16-99), ``Parameter`` (parameter.h:14-28), ``SGDSolver``
(sgd_solver.h:11-67).  The reference's solver never distributes (its ``process()`` is empty); here
ranks train data-parallel: every rank draws its own minibatches and the weight gradients are
all-reduced over NCCL before the update.

Layout: activations are ``[batch, features]``, weights are stored ``[out, in]`` so that both GEMM
operands of the forward pass are K-major; the two products of the backward pass get their
operands from the tiled transpose kernel.  ``scaled tanh`` is 1.7159·tanh(⅔·x) — the reference
writes ``2/3`` in integer arithmetic, which evaluates to 0; the documented formula is used.
"""
from __future__ import annotations

import math
import sys
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from ..ops import dense
from ..parallel.peer import PeerGroup
from ..config import data_files
from ..runtime import host


@dataclass
class Parameter:
    """Edge or model tensor of the net: value, gradient, AdaGrad accumulator."""
    name: str
    value: Optional[torch.Tensor] = None
    gradient: Optional[torch.Tensor] = None
    hession: Optional[torch.Tensor] = None


def init_tensor(shape, init, device, seed: int) -> torch.Tensor:
    """ParameterInitConfig → tensor (ZERO / CONSTANT / GAUSSIAN).  The reference's Gaussian re-seeds per
    element and therefore yields a constant (src/base/shared_array_inl.h:115-120); a real Gaussian is drawn here."""
    kind = init.type if init is not None else "GAUSSIAN"
    if kind == "ZERO":
        return torch.zeros(shape, device=device)
    if kind == "CONSTANT":
        return torch.full(shape, float(init.constant), device=device)
    g = torch.Generator(device=device).manual_seed(seed)
    mean, std = (init.mean, init.std) if init is not None and init.has("std") else (0.0, 1.0 / math.sqrt(shape[-1]))
    return torch.randn(shape, generator=g, device=device) * std + mean


class Layer:
    def __init__(self, conf, net: "Net"):
        self.conf, self.net, self.name = conf, net, conf.name
        self.inputs = [net.edge(n) for n in conf.get("in")]
        self.outputs = [net.edge(n) for n in conf.out]
        self.model: Optional[Parameter] = None
        self.lr_scale = conf.lr_scale

    def init(self) -> None: ...
    def forward(self) -> float: return 0.0
    def backward(self) -> None: ...


class DataLayer(Layer):
    """Holds a data set (features, labels), normalises the columns, emits random row minibatches."""

    def init(self) -> None:
        self.gen = torch.Generator(device="cpu").manual_seed(1234 + self.net.group.rank)
        if self.conf.has("data") and self.conf.data.file and getattr(self, "X", None) is None:
            self.load_files()

    def load_files(self) -> None:
        H = host()
        dc = self.conf.data
        files = H.divide_files(H.search_files(data_files(dc, H)), self.net.group.world, 0)[self.net.group.rank]
        r = H.SlotReader()
        r.init(files, getattr(H.TextFormat, dc.text if dc.has("text") else "LIBSVM"), f"/tmp/psb200_cache/nn{self.net.group.rank}/", True)
        info, _ = r.read(2)
        rows = info["num_ex"]
        off, idx, val = r.offset(1).astype(np.int64), r.index(1).astype(np.int64), r.value(1)
        cols = int(idx.max()) + 1 if len(idx) else 1
        X = torch.zeros(rows, cols)
        rr = np.repeat(np.arange(rows), np.diff(off))
        X[torch.from_numpy(rr), torch.from_numpy(idx)] = torch.from_numpy(val if len(val) else np.ones(len(idx), np.float32))
        self.set_data(X, torch.from_numpy(np.where(r.value(0) > 0, 1.0, -1.0).astype(np.float32)))

    def set_data(self, X: torch.Tensor, y: torch.Tensor, normalize: bool = True) -> None:
        self.X = X.to(self.net.device).contiguous().float()
        self.y = y.to(self.net.device).float()
        if normalize:
            dense.col_normalize(self.X)

    def set_sparse_data(self, off: torch.Tensor, idx: torch.Tensor, vals: Optional[torch.Tensor], y: torch.Tensor,
                        in_dim: int) -> None:
        """Keep the examples as CSR rows (for a SPARSE_FULLY_CONNECTED consumer): minibatches are row subsets."""
        d = self.net.device
        self.X = None
        self.csr = (off.to(d).long(), idx.to(d).int(), None if vals is None else vals.to(d).float(), int(in_dim))
        self.y = y.to(d).float()

    def _sparse_minibatch(self):
        off, idx, vals, in_dim = self.csr
        n, b = self.y.numel(), self.conf.minibatch_size
        if b <= 0 or b >= n:
            return (off, idx, vals, in_dim), self.y
        sel = torch.randperm(n, generator=self.gen)[:b].to(self.net.device)
        lens = off[sel + 1] - off[sel]
        noff = torch.zeros(b + 1, dtype=torch.int64, device=off.device)
        noff[1:] = lens.cumsum(0)
        # position p of the new matrix comes from row sel[r] at offset p - noff[r]
        src = torch.repeat_interleave(off[sel] - noff[:-1], lens) + torch.arange(int(noff[-1]), device=off.device)
        return (noff, idx[src].contiguous(), None if vals is None else vals[src].contiguous(), in_dim), self.y[sel].contiguous()

    def forward(self) -> float:
        if getattr(self, "csr", None) is not None and self.X is None:
            xb, yb = self._sparse_minibatch()
            self.outputs[0].value = xb
            if len(self.outputs) > 1:
                self.outputs[1].value = yb
            return 0.0
        n = self.X.shape[0]
        b = self.conf.minibatch_size
        if b <= 0 or b >= n:
            xb, yb = self.X, self.y
        else:
            b -= b % 4        # GEMM operand strides are multiples of 4 floats
            sel = torch.randperm(n, generator=self.gen)[:b].to(self.net.device)
            xb, yb = self.X[sel].contiguous(), self.y[sel].contiguous()
        self.outputs[0].value = xb
        if len(self.outputs) > 1:
            self.outputs[1].value = yb
        return 0.0


class FullyConnectedLayer(Layer):
    """Y = act(X·W): forward GEMM with the activation fused in the epilogue; backward
    Z = dY∘act'(Y), Wg = Zᵀ·X, Xg = Z·W."""

    def init(self) -> None:
        self.act = self.conf.activation.type if self.conf.has("activation") else "IDENTITY"
        if self.act not in dense.ACT:
            raise ValueError(f"activation {self.act} is not implemented")
        self.out_dim = int(self.conf.size)
        self.model = None

    def _ensure_model(self, in_dim: int) -> None:
        if self.model is None:
            shared = self.net.shared_models.get(self.name)
            if shared is not None:
                self.model = shared                      # CLONE: the test net shares the training net's model
                return
            w = init_tensor((self.out_dim, in_dim), self.conf.init if self.conf.has("init") else None, self.net.device,
                            seed=zlib.crc32(self.name.encode()) % (1 << 30))   # same weights in every process
            self.model = Parameter(self.name, w, torch.zeros_like(w), None)
            self.net.shared_models[self.name] = self.model

    def forward(self) -> float:
        x = self.inputs[0].value
        self._ensure_model(x.shape[1])
        self.x = x
        self.outputs[0].value = dense.gemm_tn(x, self.model.value, self.act, pad_k=True)
        return 0.0

    def backward(self) -> None:
        y, gy = self.outputs[0].value, self.outputs[0].gradient
        z = gy if self.act == "IDENTITY" else dense.act_backward(gy, y, self.act)
        zt, xt = dense.transpose(z), dense.transpose(self.x)
        self.model.gradient = dense.gemm_tn(zt, xt, pad_k=True)                       # [out, in] = Zᵀ · X
        if self.inputs[0].needs_grad:
            wt = dense.transpose(self.model.value)                        # [in, out]
            self.inputs[0].gradient = dense.gemm_tn(z, wt, pad_k=True)                # [batch, in] = Z · W


class SparseFullyConnectedLayer(Layer):
    """Y = act(X·W) for a sparse minibatch: the input edge carries a CSR triple ``(offsets int64, column ids
    int32, values float32 | None)`` (``DataLayer.set_sparse_data``), the model is one row of ``size`` floats per
    input feature — the per-key vectors of the reference's layer (sparse_fully_connected_layer.h:31-88, which
    adds the vectors of an example's features; its admission rule "a feature gets a vector once it was seen
    50 times" is left to the data pipeline's tail filter).  No gradient flows into the data."""

    def init(self) -> None:
        self.act = self.conf.activation.type if self.conf.has("activation") else "IDENTITY"
        if self.act not in dense.ACT:
            raise ValueError(f"activation {self.act} is not implemented")
        self.out_dim = int(self.conf.size)
        if self.out_dim % 4:
            raise ValueError("the size of a sparse fully connected layer must be a multiple of 4")
        self.model = None

    def forward(self) -> float:
        off, idx, vals, in_dim = self.inputs[0].value
        if self.model is None:
            shared = self.net.shared_models.get(self.name)
            if shared is None:
                w = init_tensor((in_dim, self.out_dim), self.conf.init if self.conf.has("init") else None, self.net.device,
                                seed=zlib.crc32(self.name.encode()) % (1 << 30))
                shared = Parameter(self.name, w, torch.zeros_like(w), None)
                self.net.shared_models[self.name] = shared
            self.model = shared
        self.x = (off, idx, vals, in_dim)
        self.outputs[0].value = dense.sparse_fc_forward(off, idx, vals, self.model.value, self.act)
        return 0.0

    def backward(self) -> None:
        off, idx, vals, in_dim = self.x
        self.model.gradient = dense.sparse_fc_backward(off, idx, vals, self.outputs[0].value, self.outputs[0].gradient, in_dim,
                                                       self.act)


class LogisticLossLayer(Layer):
    def forward(self) -> float:
        x, y = self.inputs[0].value, self.inputs[1].value
        loss, grad = dense.logistic_loss(x.reshape(-1), y, want_grad=self.net.training)
        self.loss, self.grad, self.n = loss, grad, y.numel()
        return 0.0

    def backward(self) -> None:
        self.inputs[0].gradient = self.grad.reshape(self.inputs[0].value.shape)


class AUCLayer(Layer):
    def forward(self) -> float:
        x, y = self.inputs[0].value.reshape(-1), self.inputs[1].value
        from ..ops.evalops import exact_auc

        self.auc = exact_auc(y, x) if x.is_cuda else host().exact_auc(y.cpu().numpy(), x.cpu().numpy())
        return self.auc


LAYERS = {"DATA": DataLayer, "FULLY_CONNECTED": FullyConnectedLayer, "SPARSE_FULLY_CONNECTED": SparseFullyConnectedLayer,
          "LOGISTIC_LOSS": LogisticLossLayer, "AUC": AUCLayer}


class Edge(Parameter):
    needs_grad: bool = True


class Net:
    """Layers wired by edge names, executed in the listed (topological) order."""

    def __init__(self, conf, group: PeerGroup, shared_models: Optional[Dict[str, Parameter]] = None, training: bool = True):
        self.conf, self.group, self.device, self.training = conf, group, group.device, training
        self.edges: Dict[str, Edge] = {}
        self.shared_models = shared_models if shared_models is not None else {}
        self.layers: List[Layer] = []
        for lc in conf.layer:
            if lc.type not in LAYERS:
                raise ValueError(f"unknown layer type {lc.type}")
            self.layers.append(LAYERS[lc.type](lc, self))
        for l in self.layers:
            l.init()
            if isinstance(l, DataLayer):
                for e in l.outputs:
                    e.needs_grad = False

    def edge(self, name: str) -> Edge:
        if name not in self.edges:
            self.edges[name] = Edge(name)
        return self.edges[name]

    def layer(self, name: str) -> Layer:
        return next(l for l in self.layers if l.name == name)

    def forward(self) -> None:
        for l in self.layers:
            l.forward()

    def backward(self) -> None:
        for l in reversed(self.layers):
            if not isinstance(l, (DataLayer, AUCLayer)):
                l.backward()

    def models(self) -> List[Parameter]:
        return [l.model for l in self.layers if l.model is not None]


class SGDSolver:
    """w ← w − α·g/(β+√t) or AdaGrad w ← w − α·g/(β+√Σg²); periodic evaluation of the test net."""

    def __init__(self, nn_conf, group: PeerGroup):
        self.conf, self.group = nn_conf, group
        self.train = Net(nn_conf.train, group)
        self.test = Net(nn_conf.test, group, self.train.shared_models, training=False) if nn_conf.has("test") else None
        s = nn_conf.solver
        self.alpha, self.beta = s.lr.alpha, s.lr.beta
        self.adagrad = s.update == "ADAGRAD"
        self.history: List[dict] = []

    def step(self, it: int) -> float:
        self.train.forward()
        self.train.backward()
        for l in self.train.layers:
            p = l.model
            if p is None or p.gradient is None:
                continue
            if self.group.world > 1:
                import torch.distributed as dist

                dist.all_reduce(p.gradient, group=self.group.group)
                p.gradient /= self.group.world
            if self.adagrad and p.hession is None:
                p.hession = torch.zeros_like(p.value)
            dense.sgd_update(p.value, p.gradient, p.hession if self.adagrad else None, self.alpha * l.lr_scale, self.beta, it + 1)
        loss_layer = next((l for l in self.train.layers if isinstance(l, LogisticLossLayer)), None)
        return float(loss_layer.loss.item()) / max(loss_layer.n, 1) if loss_layer else 0.0

    def evaluate(self) -> Optional[float]:
        if self.test is None:
            return None
        self.test.forward()
        auc_layer = next((l for l in self.test.layers if isinstance(l, AUCLayer)), None)
        return auc_layer.auc if auc_layer else None

    def run(self, verbose: bool = True) -> List[dict]:
        s = self.conf.solver
        for it in range(s.max_iteration):
            loss = self.step(it)
            rec = {"iter": it, "loss": loss}
            if s.validation > 0 and (it + 1) % s.validation == 0:
                rec["test_auc"] = self.evaluate()
            if verbose and self.group.rank == 0 and ((it + 1) % max(s.display, 1) == 0 or "test_auc" in rec):
                print(f"iter {it + 1:6d}  loss {loss:.5f}" + (f"  test auc {rec['test_auc']:.5f}" if rec.get("test_auc") is not None else ""),
                      file=sys.stderr)
            self.history.append(rec)
        dense.check_status(self.group.device)
        return self.history


def run_nn_job(app_conf, flags, group: PeerGroup) -> dict:
    solver = SGDSolver(app_conf.neural_network, group)
    hist = solver.run(verbose=True)
    return {"history": hist, "final_loss": hist[-1]["loss"] if hist else None}
