"""Model families (logistic regression, linear SVM, least squares) and their losses."""
from .glm import GLModel, LRModel, SVMModel, LinearRegModel, build_model  # noqa: F401
from .loss import (Loss, L1Loss, L2Loss, L1LogLoss, L2LogLoss, L2HingeLoss, L2SquareLoss,  # noqa: F401
                   LOSS_LOG, LOSS_HINGE, LOSS_SQUARE)
