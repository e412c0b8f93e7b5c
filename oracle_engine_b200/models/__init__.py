"""Architectures: importing this package registers each one under its config.json name."""
from . import llama  # noqa: F401
