"""Architectures of the package; importing a module registers its architecture."""

from . import gumapel, qwen3  # noqa: F401
from .gumapel import GumapelConfig
from .qwen3 import Qwen3Config

__all__ = ["GumapelConfig", "Qwen3Config"]
