"""Architectures.  Importing this package registers them."""
from . import pitenex, qwen3, ranudra  # noqa: F401
from .pitenex import PitenexConfig
from .qwen3 import Qwen3Config
from .ranudra import RanudraConfig

__all__ = ["PitenexConfig", "Qwen3Config", "RanudraConfig"]
