"""The generic decoder built from a model plan."""

from .model import Model

__all__ = ["Model"]
