"""Architectures of the package; importing a module registers its architecture."""

from . import gumapel, kelasun, qwen3  # noqa: F401
from .gumapel import GumapelConfig
from .kelasun import KelasunConfig
from .qwen3 import Qwen3Config

__all__ = ["GumapelConfig", "KelasunConfig", "Qwen3Config"]
