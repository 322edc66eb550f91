from .registry import BackendKind, KernelRegistry, default_registry  # noqa: F401
from .schedule import Schedule, default_schedule  # noqa: F401
