"""Minibatch gradient, regularisation and the two optimizers (host/torch path).

Reference: ml/objective/GradientDescent.scala:19-132 and ml/objective/Adam.scala:15-110.
* batch = ``(size * ratio).toInt`` consecutive cyclic rows; gradient = mean over the batch
  of x * (-loss.grad); L2 adds lambda * w on the gradient's own coordinates only.
* SGD: lr = lr0 / sqrt(1 + decay * epoch).
* Adam: beta1 = 0.9, beta2 = 0.999, eps = 1e-8, constant lr; the beta powers advance once
  per epoch (on the first update after an epoch's last gradient), and the sparse update
  touches only the gradient's coordinates (lazy Adam).
The GPU path implements the same rules in csrc/cuda (gradient and update kernels).
"""
from __future__ import annotations

import math

import torch

from .gradient.kinds import DenseDoubleGradient, Gradient, Kind, SparseDoubleGradient

EPS = 1e-8


class GradientDescent:
    name = "sgd"

    def __init__(self, dim: int, lr_0: float, decay: float, batch_sp_ratio: float, device="cpu",
                 dtype=torch.float64):
        self.dim, self.lr_0, self.decay, self.batch_sp_ratio = dim, lr_0, decay, batch_sp_ratio
        self.epoch = 0
        self.batch = 0
        self.batch_num = int(math.ceil(1.0 / batch_sp_ratio))
        self.device, self.dtype = device, dtype

    # GradientDescent.scala:23-51
    def mini_batch_gradient_descent(self, weight: torch.Tensor, data_set, loss):
        batch_size = data_set.batch_size(self.batch_sp_ratio)
        dense = DenseDoubleGradient(self.dim)
        obj_loss = 0.0
        if batch_size > 0:
            b = data_set.looping_read(batch_size)
            w64 = weight.double().cpu()
            b = b.to("cpu")
            pre = loss.predict(w64, b)
            y = b.labels.double()
            coef = -loss.grad(pre, y)
            dense.plus_by_features(b.cols, coef[b.row_ids()] * b.dense_values(torch.float64))
            obj_loss = float(loss.loss(pre, y).sum())
        grad = dense.to_auto()
        if batch_size > 0:
            grad.times_by(1.0 / batch_size)
        if loss.is_l1_reg:
            self.l1_reg(grad, 0.0, loss.get_reg_param())
        if loss.is_l2_reg:
            self.l2_reg(grad, weight, loss.get_reg_param())
        reg_loss = loss.get_reg(weight)
        self.advance()
        return grad, batch_size, obj_loss, reg_loss

    def advance(self) -> None:
        self.batch += 1
        if self.batch == self.batch_num:
            self.epoch += 1
            self.batch = 0

    @staticmethod
    def l1_reg(grad: Gradient, alpha: float, theta: float) -> None:
        v = grad.values
        pos = (v >= 0) & (v <= theta)
        neg = (v < 0) & (v >= -theta)
        v[pos] = (v[pos] - alpha).clamp(min=0)
        v[neg] = (v[neg] - alpha).clamp(max=0)

    @staticmethod
    def l2_reg(grad: Gradient, weight: torch.Tensor, lam: float) -> None:
        w = weight.double().cpu()
        if grad.kind is Kind.DenseDouble:
            grad.values += w * lam
        elif grad.kind is Kind.SparseDouble:
            grad.values += w[grad.indices.long()] * lam
        else:
            raise ValueError(f"Cannot regularize {grad.kind} kind of gradients")

    def learning_rate(self) -> float:
        return self.lr_0 / math.sqrt(1.0 + self.decay * self.epoch)

    # GradientDescent.scala:89-132
    def update(self, grad: Gradient, weight: torch.Tensor) -> None:
        g = self._plain(grad)
        if g is None:
            return
        lr = self.learning_rate()
        if hasattr(g, "indices"):
            idx = g.indices.long().to(weight.device)
            weight[idx] -= (g.values.to(weight.device) * lr).to(weight.dtype)
        else:
            weight -= (g.values.to(weight.device) * lr).to(weight.dtype)

    @staticmethod
    def _plain(grad: Gradient):
        if grad.kind is Kind.ZeroGradient:
            return None
        if grad.kind in (Kind.Sketch, Kind.FixedPoint, Kind.Zip):
            grad = grad.to_auto()
            if grad.kind is Kind.ZeroGradient:
                return None
        return grad

    def state_dict(self) -> dict:
        return {"name": self.name, "epoch": self.epoch, "batch": self.batch}

    def load_state_dict(self, sd: dict) -> None:
        self.epoch, self.batch = int(sd["epoch"]), int(sd["batch"])


class Adam(GradientDescent):
    name = "adam"
    beta1, beta2 = 0.9, 0.999

    def __init__(self, dim, lr_0, decay, batch_sp_ratio, device="cpu", dtype=torch.float64):
        super().__init__(dim, lr_0, decay, batch_sp_ratio, device, dtype)
        self.beta1_t, self.beta2_t = 0.9, 0.999
        self.m = torch.zeros(dim, dtype=dtype, device=device)
        self.v = torch.zeros(dim, dtype=dtype, device=device)

    def advance_betas(self) -> None:
        """Adam.scala:29-32: the powers move once per epoch."""
        if self.epoch > 0 and self.batch == 0:
            self.beta1_t *= self.beta1
            self.beta2_t *= self.beta2

    def step_scale(self) -> float:
        return math.sqrt(1.0 - self.beta2_t) / (1.0 - self.beta1_t)

    def update(self, grad: Gradient, weight: torch.Tensor) -> None:
        self.advance_betas()
        g = self._plain(grad)
        if g is None:
            return
        gv = g.values.to(weight.device).to(self.m.dtype)
        if hasattr(g, "indices"):
            idx = g.indices.long().to(weight.device)
            m_t = self.beta1 * self.m[idx] + (1 - self.beta1) * gv
            v_t = self.beta2 * self.v[idx] + (1 - self.beta2) * gv * gv
            new = (math.sqrt(1 - self.beta2_t) * m_t) / ((1 - self.beta1_t) * (v_t.sqrt() + EPS))
            weight[idx] -= (new * self.lr_0).to(weight.dtype)
            self.m[idx] = m_t
            self.v[idx] = v_t
        else:
            self.m.mul_(self.beta1).add_(gv, alpha=1 - self.beta1)
            self.v.mul_(self.beta2).addcmul_(gv, gv, value=1 - self.beta2)
            new = (math.sqrt(1 - self.beta2_t) * self.m) / ((1 - self.beta1_t) * (self.v.sqrt() + EPS))
            weight -= (new * self.lr_0).to(weight.dtype)

    def state_dict(self) -> dict:
        sd = super().state_dict()
        sd.update(beta1_t=self.beta1_t, beta2_t=self.beta2_t, m=self.m.detach().cpu(), v=self.v.detach().cpu())
        return sd

    def load_state_dict(self, sd: dict) -> None:
        super().load_state_dict(sd)
        self.beta1_t, self.beta2_t = float(sd["beta1_t"]), float(sd["beta2_t"])
        self.m.copy_(sd["m"].to(self.m.dtype))
        self.v.copy_(sd["v"].to(self.v.dtype))
