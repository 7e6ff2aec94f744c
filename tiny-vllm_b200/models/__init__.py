"""Architectures of the package; importing a module registers its architecture."""

from . import bimolix, fezavik, gumapel, kelasun, qwen3  # noqa: F401
from .bimolix import BimolixConfig
from .fezavik import FezavikConfig
from .gumapel import GumapelConfig
from .kelasun import KelasunConfig
from .qwen3 import Qwen3Config

__all__ = ["BimolixConfig", "FezavikConfig", "GumapelConfig", "KelasunConfig", "Qwen3Config"]
