"""Loss functions of the three generalized linear models (vectorised torch).

Reference: ml/objective/Loss.scala:6-137. ``grad`` is the NEGATIVE derivative of the
loss with respect to the prediction (the caller multiplies by -1,
ml/objective/GradientDescent.scala:33). The regularisation "loss" is the un-squared
norm times lambda (Loss.scala:31-36,48-53) and is active iff lambda > 1e-8.
"""
from __future__ import annotations

import torch

EPS = 1e-8
LOSS_LOG, LOSS_HINGE, LOSS_SQUARE = 0, 1, 2   # ids shared with the CUDA kernels


class Loss:
    loss_id = -1
    name = "loss"

    def __init__(self, lam: float = 0.0):
        self.lam = float(lam)

    def loss(self, pre: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def grad(self, pre: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def predict(self, w: torch.Tensor, batch) -> torch.Tensor:
        """Margins w.x of every row of a CSRMatrix."""
        vals = batch.dense_values(w.dtype)
        prod = w[batch.cols.long()] * vals
        out = torch.zeros(batch.rows, dtype=w.dtype, device=w.device)
        return out.index_add_(0, batch.row_ids(), prod)

    @property
    def is_l1_reg(self) -> bool:
        return False

    @property
    def is_l2_reg(self) -> bool:
        return False

    def get_reg_param(self) -> float:
        return self.lam

    def get_reg(self, w: torch.Tensor) -> float:
        return 0.0


class L1Loss(Loss):
    @property
    def is_l1_reg(self) -> bool:
        return self.lam > EPS

    def get_reg(self, w):
        return float(w.abs().sum()) * self.lam if self.is_l1_reg else 0.0


class L2Loss(Loss):
    @property
    def is_l2_reg(self) -> bool:
        return self.lam > EPS

    def get_reg(self, w):
        return float(torch.linalg.vector_norm(w.double())) * self.lam if self.is_l2_reg else 0.0


def _log_loss(pre, y):
    z = pre * y
    mid = torch.log1p(torch.exp(-z.clamp(-18, 18)))
    return torch.where(z > 18, torch.exp(-z), torch.where(z < -18, -z, mid))


def _log_grad(pre, y):
    z = pre * y
    mid = y / (1.0 + torch.exp(z.clamp(-18, 18)))
    return torch.where(z > 18, y * torch.exp(-z), torch.where(z < -18, y, mid))


class L1LogLoss(L1Loss):
    """Defined by the reference, never wired to a model (Loss.scala:56-80)."""
    loss_id, name = LOSS_LOG, "L1LogLoss"
    loss = staticmethod(_log_loss)
    grad = staticmethod(_log_grad)


class L2LogLoss(L2Loss):
    loss_id, name = LOSS_LOG, "L2LogLoss"
    loss = staticmethod(_log_loss)
    grad = staticmethod(_log_grad)


class L2HingeLoss(L2Loss):
    loss_id, name = LOSS_HINGE, "L2HingeLoss"

    def loss(self, pre, y):
        z = pre * y
        return torch.where(z < 1.0, 1.0 - z, torch.zeros_like(z))

    def grad(self, pre, y):
        return torch.where(pre * y <= 1.0, y, torch.zeros_like(y))


class L2SquareLoss(L2Loss):
    loss_id, name = LOSS_SQUARE, "L2SquareLoss"

    def loss(self, pre, y):
        return 0.5 * (pre - y) * (pre - y)

    def grad(self, pre, y):
        return y - pre
