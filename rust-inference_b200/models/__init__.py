"""Architectures.  Importing this package registers them."""
from . import qwen3, ranudra  # noqa: F401
from .qwen3 import Qwen3Config
from .ranudra import RanudraConfig

__all__ = ["Qwen3Config", "RanudraConfig"]
