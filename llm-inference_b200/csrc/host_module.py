"""Loads the compiled C++ host runtime (page pools, cache manager, scheduler)."""

from __future__ import annotations

import importlib.util
import os
import sys
from functools import lru_cache

from . import build


@lru_cache(maxsize=1)
def host():
    """The ``b200_host`` extension module; built first if its sources changed. With
    ``LLM_INFERENCE_B200_SANITIZE=1`` in the environment (see ``build.sanitizer_environment``)
    the build checked by AddressSanitizer and UndefinedBehaviorSanitizer is loaded instead."""
    path = build.build_host(sanitize=os.environ.get("LLM_INFERENCE_B200_SANITIZE") == "1")
    if "b200_host" in sys.modules:
        return sys.modules["b200_host"]
    spec = importlib.util.spec_from_file_location("b200_host", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["b200_host"] = module
    spec.loader.exec_module(module)
    return module
