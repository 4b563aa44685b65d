"""Architectures this library knows; importing the package registers them."""
from . import qwen3, kadodra, tusasun, bagasun, bolisun  # noqa: F401
