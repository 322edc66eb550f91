"""Metrics (``momijo.learn.metrics``)."""
from .classification import accuracy, f1_score, confusion_matrix, precision_recall_f1  # noqa: F401
from .metrics import accuracy_approx, iou, psnr, ssim  # noqa: F401
from .regression import mse, rmse, mae, mape, r2_score, explained_variance  # noqa: F401
from .streaming import StreamingMetric, WeightedStreamingMetric, ConfusionMatrixBinary  # noqa: F401
