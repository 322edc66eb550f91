from .registry import (  # noqa: F401
    register_model, has_model, get_constructor_path, list_models, unregister_model, clear_registry,
    dump_registry,
)
from .download import DownloadOptions, cached_download  # noqa: F401
