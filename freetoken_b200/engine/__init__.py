"""The engine (one step function) and the scheduler above it."""

from .engine import Engine, EngineArgs, StepEntry

__all__ = ["Engine", "EngineArgs", "StepEntry"]
