"""freetoken_b200: a single-GPU inference engine for the MiniMax-M3 decoder on B200."""

from .version import __version__

__all__ = ["__version__", "LLM", "SamplingParams", "Engine", "EngineArgs", "StepEntry"]


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM
        return LLM
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    if name in ("Engine", "EngineArgs", "StepEntry"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
