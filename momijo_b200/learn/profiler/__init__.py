from .core import Profiler, ProfRow  # noqa: F401
from .estimators import est_ops_linear, est_ops_relu, est_ops_attention, est_ops_conv2d  # noqa: F401
