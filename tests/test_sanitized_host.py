"""The C++ host runtime (page pools, cache manager, scheduler, bindings) under AddressSanitizer
and UndefinedBehaviorSanitizer: the cache-manager and scheduler tests are run once more in a
child interpreter that loads the checked build, as the reference's CI runs its host code under
the same two sanitizers (.github/workflows/ci.yml:62-79). compute-sanitizer cannot be used for
the device side here; this covers the host side."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

from helpers import ROOT


def test_cache_manager_and_scheduler_under_address_and_ub_sanitizers():
    from llm_inference_b200.csrc import build

    try:
        extra = build.sanitizer_environment()
        build.build_host(sanitize=True)
    except build.BuildError as error:
        pytest.skip(f"no sanitizer build on this machine: {error}")
    env = dict(os.environ, **extra)
    result = subprocess.run(
        [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", "tests/test_cache_manager.py", "tests/test_scheduler.py"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=900,
    )
    report = result.stdout[-3000:] + result.stderr[-3000:]
    assert result.returncode == 0, report
    assert "passed" in result.stdout and "failed" not in result.stdout, report
    for sign in ("AddressSanitizer", "runtime error:", "UndefinedBehaviorSanitizer"):
        assert sign not in result.stdout and sign not in result.stderr, report
    # The child really loaded the checked build.
    probe = subprocess.run(
        [sys.executable, "-c", "from llm_inference_b200.csrc.host_module import host; print(host().__file__)"],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=300,
    )
    assert probe.returncode == 0 and "sanitize" in probe.stdout, probe.stdout + probe.stderr
