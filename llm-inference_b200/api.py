"""Public entry points (filled in by engine.engine)."""

from .engine.engine import Engine, SamplingParams, SequenceState, TokenEvent, build_info, create_engine

__all__ = ["Engine", "SamplingParams", "SequenceState", "TokenEvent", "build_info", "create_engine"]
