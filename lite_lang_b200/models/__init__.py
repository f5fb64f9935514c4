"""Architectures.  Importing this package registers each of them."""
from . import nevurax, qwen2, redirax  # noqa: F401
from .nevurax import NevuraxConfig
from .qwen2 import Qwen2Config
from .redirax import RediraxConfig

__all__ = ["NevuraxConfig", "Qwen2Config", "RediraxConfig"]
