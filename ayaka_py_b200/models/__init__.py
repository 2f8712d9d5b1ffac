"""Architectures.  Importing this package registers them."""

from . import gpt2, luporax, rakalix, tesozen, vedadra  # noqa: F401
from .model import Model

__all__ = ["Model"]
