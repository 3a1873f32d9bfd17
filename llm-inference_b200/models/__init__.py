"""Architectures this engine knows; importing the package registers them."""

from . import qwen2  # noqa: F401
