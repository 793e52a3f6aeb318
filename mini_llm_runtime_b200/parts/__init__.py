"""Importing this package registers the built-in parts."""
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401
