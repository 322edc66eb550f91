from .autocast import AMPPrecision, autocast, AutocastGuard, GradScaler  # noqa: F401
