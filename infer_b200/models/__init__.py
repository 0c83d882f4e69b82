"""Architectures. Importing this package registers them with ``config.registry``."""
from . import qwen2  # noqa: F401
