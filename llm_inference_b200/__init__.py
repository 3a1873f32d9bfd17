"""Import name of the ``llm-inference_b200`` source folder.

The folder name has a hyphen, which Python cannot import, so this package only
extends its search path into that folder and re-exports the public entry points.
"""

from pathlib import Path as _Path

__path__.append(str(_Path(__file__).resolve().parent.parent / "llm-inference_b200"))

from .engine.engine import (  # noqa: E402
    SamplingParams,
    SequenceState,
    TokenEvent,
    build_info,
    create_engine,
)

__all__ = ["SamplingParams", "SequenceState", "TokenEvent", "build_info", "create_engine"]
