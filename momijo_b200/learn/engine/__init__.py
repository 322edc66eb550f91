"""Training / evaluation loops (``momijo.learn.engine``)."""
from .hooks import Hooks, TrainState, BatchInfo, LRUpdateInfo  # noqa: F401
from .trainer import Trainer  # noqa: F401
from .evaluator import Evaluator, EvalResult  # noqa: F401
from .jit_compile import JITOptions, GraphExecutor, compile, compile_with, dry_trace  # noqa: F401
