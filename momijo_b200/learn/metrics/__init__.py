"""Metrics (``momijo.learn.metrics``)."""
from .classification import (  # noqa: F401
    accuracy, f1_score, confusion_matrix, precision_recall_f1, argmax_index, confusion_matrix_from_labels,
    f1_score_binary,
)
from .metrics import accuracy_approx, iou, psnr, ssim  # noqa: F401
from .regression import mse, rmse, mae, mape, r2_score, explained_variance  # noqa: F401
from .streaming import StreamingMetric, WeightedStreamingMetric, ConfusionMatrixBinary  # noqa: F401
