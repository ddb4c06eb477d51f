"""Architectures that register themselves when the package is imported."""
from . import llama  # noqa: F401
