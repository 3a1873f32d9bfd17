"""Loads the compiled C++ host runtime (page pools, cache manager, scheduler)."""

from __future__ import annotations

import importlib.util
import sys
from functools import lru_cache

from . import build


@lru_cache(maxsize=1)
def host():
    """The ``b200_host`` extension module; built first if its sources changed."""
    path = build.build_host()
    if "b200_host" in sys.modules:
        return sys.modules["b200_host"]
    spec = importlib.util.spec_from_file_location("b200_host", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["b200_host"] = module
    spec.loader.exec_module(module)
    return module
