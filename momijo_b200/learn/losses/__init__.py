"""Losses (``momijo.learn.losses``)."""
from .losses import (  # noqa: F401
    softmax_cross_entropy, cross_entropy_from_logits, cross_entropy_from_probs, mse, mae, huber,
    smooth_l1, bce, bce_with_logits, kl_div, nll_loss, focal, dice, triplet, cosine_embedding,
)
from .classification import cross_entropy, binary_cross_entropy, hinge, focal_loss, label_smoothing_cross_entropy  # noqa: F401
from .regression import (  # noqa: F401
    mse_loss, mae_loss, rmse_loss, huber_loss, smooth_l1_loss, log_cosh_loss, quantile_loss,
    msle_loss, mape_loss,
)
from . import ranking, segmentation  # noqa: F401
