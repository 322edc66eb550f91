from .registry import Backend, BackendKind, KernelRegistry, default_registry  # noqa: F401
from .schedule import Schedule, auto_schedule, default_schedule  # noqa: F401
from . import cpu  # noqa: F401
