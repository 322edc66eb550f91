"""Losses (``momijo.learn.losses``)."""
from .losses import (  # noqa: F401
    softmax_cross_entropy, cross_entropy_from_logits, cross_entropy_from_probs, mse, mae, huber,
    smooth_l1, bce, bce_with_logits, kl_div, nll_loss, focal, dice, triplet, cosine_embedding,
    triplet_loss, cosine_embedding_loss,
)
from .classification import (  # noqa: F401
    cross_entropy, binary_cross_entropy, hinge, focal_loss, label_smoothing_cross_entropy,
    focal_loss_binary_with_logits, focal_loss_multiclass_with_logits,
)
from .regression import (  # noqa: F401
    mse_loss, mae_loss, rmse_loss, huber_loss, smooth_l1_loss, log_cosh_loss, quantile_loss,
    msle_loss, mape_loss,
)
from . import ranking, segmentation  # noqa: F401
from .ranking import hinge_loss, triplet_loss_from_dist  # noqa: F401,E402
from .segmentation import dice_loss_mc, dice_loss_mc_vec, iou_loss_mc, iou_loss_mc_vec  # noqa: F401,E402
