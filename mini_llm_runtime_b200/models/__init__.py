"""Importing this package registers the architectures."""
from . import qwen3  # noqa: F401
