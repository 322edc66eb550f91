from . import runtime  # noqa: F401
