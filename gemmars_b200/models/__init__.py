"""Architectures.  Importing this package registers each of them under its config.json names."""
from . import qwen3  # noqa: F401
