"""Optimizers and schedulers (``momijo.learn.optim``)."""
from .sgd import SGD  # noqa: F401
from .adam import Adam  # noqa: F401
from .adamw import AdamW  # noqa: F401
from .rmsprop import RMSprop  # noqa: F401
from .adagrad import Adagrad  # noqa: F401
from . import schedulers  # noqa: F401
from .schedulers import (  # noqa: F401
    ExponentialLR, PolynomialLR, CosineAnnealingWarmRestarts, LinearWarmup, WarmupThen, ChainedLR,
    ReduceLROnPlateau,
)
from .scheduler_steplr import StepLR  # noqa: F401
from .scheduler_multistep import MultiStepLR  # noqa: F401
from .scheduler_cosine import CosineAnnealingLR  # noqa: F401
