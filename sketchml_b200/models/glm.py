"""The three model families: replicated dense weights, a loss and an optimizer.

Reference: ml/algorithm/LRModel.scala:21-27, SVMModel.scala:21-27,
LinearRegModel.scala:21-27 (zero weights, Adam, L2 loss with lambda = reg.l2 on
every worker). The optimizer here follows ``conf.optimizer``; the reference always
constructs Adam.
"""
from __future__ import annotations

import torch

from ..config import MLConf, ML_LINEAR_REGRESSION, ML_LOGISTIC_REGRESSION, ML_SUPPORT_VECTOR_MACHINE
from ..optim import Adam, GradientDescent
from .loss import L2HingeLoss, L2LogLoss, L2SquareLoss, Loss


class GLModel:
    name = "GeneralizedLinearModel"
    loss_cls = Loss
    task = "logistic"

    def __init__(self, conf: MLConf, device="cpu", dtype=None):
        self.conf = conf
        self.dtype = dtype or (torch.float64 if conf.dtype == "float64" else torch.float32)
        self.device = torch.device(device)
        self.init_model()

    def init_model(self) -> None:
        c = self.conf
        self.weights = torch.zeros(c.feature_num, dtype=self.dtype, device=self.device)
        opt_cls = Adam if c.optimizer == "adam" else GradientDescent
        self.optimizer = opt_cls(c.feature_num, c.learn_rate, c.learn_decay, c.batch_sample_ratio,
                                 device=self.device, dtype=self.dtype)
        self.loss = self.loss_cls(c.l2_reg)

    def get_name(self) -> str:
        return self.name

    def predict(self, batch) -> torch.Tensor:
        return self.loss.predict(self.weights, batch)

    def state_dict(self) -> dict:
        return {"weights": self.weights.detach().cpu(), "optimizer": self.optimizer.state_dict(),
                "model": self.name}

    def load_state_dict(self, sd: dict) -> None:
        self.weights.copy_(sd["weights"].to(self.weights.dtype))
        self.optimizer.load_state_dict(sd["optimizer"])


class LRModel(GLModel):
    name, loss_cls, task = "LR", L2LogLoss, "logistic"


class SVMModel(GLModel):
    name, loss_cls, task = "SVM", L2HingeLoss, "svm"


class LinearRegModel(GLModel):
    name, loss_cls, task = "LinearReg", L2SquareLoss, "regression"


def build_model(conf: MLConf, device="cpu") -> GLModel:
    """Model selection by ``algo`` (ml/SketchML.scala:13-18)."""
    cls = {ML_LOGISTIC_REGRESSION: LRModel, ML_SUPPORT_VECTOR_MACHINE: SVMModel,
           ML_LINEAR_REGRESSION: LinearRegModel}.get(conf.algo)
    if cls is None:
        raise ValueError("Unrecognizable algorithm: " + conf.algo)
    return cls(conf, device)
