"""Callbacks (``momijo.learn.callbacks``)."""
from .early_stopping import EarlyStopping  # noqa: F401
from .model_checkpoint import ModelCheckpoint  # noqa: F401
from .lr_monitor import LRMonitor, LRRecord  # noqa: F401
from .logger import CSVLogger, CSVTableLogger, JSONLLogger  # noqa: F401
