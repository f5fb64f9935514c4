"""Architectures.  Importing this package registers each of them."""
from . import nevurax, qwen2  # noqa: F401
from .nevurax import NevuraxConfig
from .qwen2 import Qwen2Config

__all__ = ["NevuraxConfig", "Qwen2Config"]
