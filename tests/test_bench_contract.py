"""What bench.py promises without a GPU: its refusals, the reference arm's line, where the
peaks come from, the flop counts behind its fractions and how it reads the clock samples."""

from __future__ import annotations

import importlib.util
import json
import subprocess
import sys
from types import SimpleNamespace

import pytest

from helpers import ROOT


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def run(*args: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    result = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert result.returncode == 2
    assert result.stdout.strip().count("\n") == 0 and "one GPU" in result.stdout


def test_reference_arm_prints_one_line_and_says_why_when_it_cannot_run():
    """Without a GPU (or without the reference installed under baseline/_ref) the arm prints one
    line that says why and exits 0. Where it can run, that takes minutes and is the driver's job."""
    import torch

    if torch.cuda.is_available() and (ROOT / "baseline" / "_ref" / "instinct").is_dir():
        pytest.skip("the reference is installed and a GPU is visible: the arm would run in full")
    result = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert result.returncode == 0
    line = json.loads(result.stdout.strip())
    assert line["impl"] == "reference" and "\n" not in line["unavailable"] and len(line["unavailable"]) > 20


def test_peaks_come_from_the_measured_file_when_it_is_there(bench, tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", tmp_path)
    assert bench.peaks() == bench.FALLBACK_PEAKS and bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6400.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1390.0}))
    assert bench.peaks() == {"source": "measured", "hbm_gbs": 6400.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1390.0}
    (tmp_path / "MEASURED_PEAKS.json").write_text("{ not json")
    assert bench.peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": {"nested": 1}}))
    assert bench.peaks()["source"] == "fallback"


def test_flop_counts_of_the_headline_shape(bench):
    """A 2,048-token prefill of the 1.5B shape: 5.37 TFLOP in the layers' products and 0.36 in
    causal attention."""
    shape = bench.MODEL
    config = SimpleNamespace(
        hidden_size=shape["hidden_size"], intermediate_size=shape["intermediate_size"], head_dim=shape["head_dim"],
        num_attention_heads=shape["num_attention_heads"], num_key_value_heads=shape["num_key_value_heads"],
    )
    layers = shape["num_hidden_layers"]
    linear = 2048 * bench.linear_flops_per_token(config, layers)
    attention = bench.attention_flops(config, layers, 2048)
    assert linear == pytest.approx(5.37e12, rel=5e-3)
    assert attention == pytest.approx(0.36e12, rel=2e-2)
    # Per token and layer: q/k/v 2048 x 1536, o 1536 x 1536, gate, up and down 8960 x 1536 each.
    assert bench.linear_flops_per_token(config, 1) == 2 * (2048 * 1536 + 1536 * 1536 + 3 * 8960 * 1536)


def test_clock_samples_are_summarised(bench):
    sampler = bench.ClockSampler()
    sampler.lines = [
        "1965, 1965, Not Active, Not Active, Not Active, Active",
        "1800, 1965, Not Active, Not Active, Not Active, Not Active",
        "garbage",
        "1900, 1965, Not Active, Active, Not Active, Active",
        "[N/A], 1965, Not Active, Not Active, Not Active, Not Active",
    ]
    assert sampler.summary() == {"sm_mhz": 1900.0, "sm_max_mhz": 1965.0, "reasons": ["hw_thermal_slowdown", "sw_power_cap"], "samples": 3}
    assert sampler.summary(0, 2)["reasons"] == ["sw_power_cap"]
    assert sampler.summary(2, 3) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
