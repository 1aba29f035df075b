"""Architectures known to the library; importing this package registers them."""
from . import qwen3, suvazen  # noqa: F401
