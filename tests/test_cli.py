"""Command-line entry points."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

from helpers import ROOT, plain_weights
from plain import qwen2_plain as plain


def run(module: str, *args: str, check: bool = True) -> subprocess.CompletedProcess:
    result = subprocess.run(
        [sys.executable, "-m", f"llm_inference_b200.cli.{module}", *args], capture_output=True, text=True, cwd=ROOT, timeout=600
    )
    if check:
        assert result.returncode == 0, result.stderr[-3000:]
    return result


def test_random_model_and_inspect(tmp_path):
    folder = tmp_path / "tiny"
    run("random_model", "--preset", "tiny-b", "--seed", "4", "--out", str(folder))
    assert json.loads((folder / "config.json").read_text())["sliding_window"] == 24
    out = run("inspect_model", str(folder)).stdout
    assert "architecture: Qwen2ForCausalLM" in out and "lm_head.weight  bfloat16  [311, 96]" in out and "valid" in out
    (folder / "config.json").write_text(json.dumps({"architectures": ["Nope"]}))
    bad = run("inspect_model", str(folder), check=False)
    assert bad.returncode == 1 and "no model registered for 'Nope'" in bad.stderr


@pytest.mark.gpu
def test_generate_and_benchmark(tmp_path):
    folder = tmp_path / "tiny"
    run("random_model", "--preset", "tiny-a", "--seed", "9", "--out", str(folder))
    config, weights = plain_weights(folder)
    prompt = [5, 17, 3, 200, 41]
    out = run("generate", "--model", str(folder), "--prompt-ids", "5,17,3,200,41", "--max-new-tokens", "6",
              "--dtype", "float32", "--max-model-length", "128", "--kv-cache-mib", "1", "--page-size", "16").stdout
    assert json.loads(out.strip().splitlines()[-1])["tokens"] == plain.greedy(config, weights, prompt, 6)
    prompts = tmp_path / "prompts.json"
    prompts.write_text(json.dumps([[1, 2, 3], list(range(40)), [9] * 17]))
    result = tmp_path / "bench.json"
    run("benchmark", "--model", str(folder), "--prompts", str(prompts), "--output", str(result), "--output-length", "8",
        "--warmups", "1", "--repetitions", "2", "--max-sequences", "2", "--max-model-length", "128", "--kv-cache-mib", "1",
        "--page-size", "16")
    report = json.loads(result.read_text())
    assert report["aggregate"]["generated_tokens_per_second"] > 0
    assert len(report["requests"]) == 6 and all(r["output_tokens"] == 8 for r in report["requests"])
    assert set(report["aggregate"]["ttft_ms"]) == {"p50", "p95", "p99"}


@pytest.mark.gpu
def test_benchmark_with_a_random_shape_and_a_synthetic_mix(tmp_path):
    result = tmp_path / "mix.json"
    run("benchmark", "--random", "tiny-b", "--mix", "5", "--mix-prompt-lengths", "3", "40", "--mix-output-lengths", "2", "9",
        "--output", str(result), "--warmups", "1", "--repetitions", "1", "--max-sequences", "3", "--max-model-length", "64",
        "--kv-cache-mib", "1", "--page-size", "8", "--prefill-chunk-size", "16")
    report = json.loads(result.read_text())
    requests = report["requests"]
    assert len(requests) == 5
    assert all(3 <= r["prompt_tokens"] <= 40 and 2 <= r["output_tokens"] <= 9 for r in requests)
    assert len({r["prompt_tokens"] for r in requests}) > 1
    assert report["configuration"]["model_path"] == "random:tiny-b"
    neither = run("benchmark", "--mix", "2", "--output", str(result), check=False)
    assert neither.returncode != 0 and "--model DIR or --random SHAPE" in neither.stderr


def test_replay_checks_its_options_and_needs_a_gpu(tmp_path):
    """Options are checked before anything is loaded; without a CUDA device the tool says so
    and exits (there is no CPU path to fall back to)."""
    import torch

    from helpers import TRACE_RUN

    folder = tmp_path / "tiny"
    run("random_model", "--preset", "tiny-a", "--seed", "2", "--out", str(folder))
    base = [sys.executable, str(TRACE_RUN), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out")]
    step = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}], "end": ["a"]}) + "\n"
    for extra, message in (
        (["--max-tokens", "0"], "--max-tokens must be positive"),
        (["--max-tokens", "64", "--page-size", "48"], "--page-size must divide 64"),
        (["--max-tokens", "64", "--dtype", "float16"], "invalid choice"),
    ):
        bad = subprocess.run(base + extra, input=step, capture_output=True, text=True, timeout=300)
        assert bad.returncode == 2 and message in bad.stderr
    if not torch.cuda.is_available():
        result = subprocess.run(base + ["--max-tokens", "64"], input=step, capture_output=True, text=True, timeout=300)
        assert result.returncode == 2 and "no CUDA device" in result.stderr and "done" not in result.stdout


def test_benchmark_percentiles_interpolate_as_the_reference_does():
    """The reference's rule (python/instinct/benchmark.py:94-107): rank q (n - 1), linear between
    the neighbours. Checked on values whose percentiles are easy to state."""
    import math

    from llm_inference_b200.cli.benchmark import percentiles

    values = [float(v) for v in range(101)]  # rank q * 100 is the value itself
    assert percentiles(values[::-1]) == {"p50": 50.0, "p95": 95.0, "p99": 99.0}
    got = percentiles([1.0, 2.0, 3.0, 4.0, 10.0])
    assert got["p50"] == 3.0 and math.isclose(got["p95"], 4.0 + 0.8 * 6.0) and math.isclose(got["p99"], 4.0 + 0.96 * 6.0)
    assert percentiles([7.0]) == {"p50": 7.0, "p95": 7.0, "p99": 7.0}
    assert all(math.isnan(v) for v in percentiles([]).values())
