"""Architectures of the package; importing a module registers its architecture."""

from . import bimolix, gumapel, kelasun, qwen3  # noqa: F401
from .bimolix import BimolixConfig
from .gumapel import GumapelConfig
from .kelasun import KelasunConfig
from .qwen3 import Qwen3Config

__all__ = ["BimolixConfig", "GumapelConfig", "KelasunConfig", "Qwen3Config"]
