"""Shared test fixtures: the two tiny configurations, model folders, the replay driver."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
TRACE_RUN = ROOT / "bin" / "trace_run"

# Two tiny Qwen2 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "intermediate_size": 176,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "max_position_embeddings": 128,
    "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "intermediate_size": 272,
    "vocab_size": 311,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "use_sliding_window": True,
    "sliding_window": 24,
    "max_window_layers": 1,
    "max_position_embeddings": 256,
    "eos_token_id": [5, 7],
}
TINY = {"A": TINY_A, "B": TINY_B}
PAGE_SIZE = {"A": 16, "B": 8}


def make_model_folder(folder: Path, raw_config: dict, seed: int, std: float = 0.02) -> Path:
    """config.json + model.safetensors with seeded random bfloat16 weights."""
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.weights import write_model_folder

    _, config = parse_config(raw_config)
    return write_model_folder(folder, config, seed, std=std)


def plain_weights(folder: Path) -> tuple[dict, dict]:
    """(config dict, weights as float64 arrays) read with the safetensors package, not the engine."""
    import torch
    from safetensors.torch import load_file

    config = json.loads((Path(folder) / "config.json").read_text())
    tensors = load_file(str(Path(folder) / "model.safetensors"))
    return config, {name: t.to(torch.float64).numpy() for name, t in tensors.items()}


def run_trace(
    model: Path, dtype: str, steps: list[dict], out: Path, max_tokens: int, page_size: int | None = None, timeout: int = 600
) -> dict[int, np.ndarray]:
    """Drive bin/trace_run with ``steps``; returns step -> float32 logits ``[wanted, vocab]``."""
    vocab = json.loads((Path(model) / "config.json").read_text())["vocab_size"]
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model), "--dtype", dtype, "--out", str(out), "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    text = "".join(json.dumps(step) + "\n" for step in steps)
    result = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=dict(os.environ))
    assert result.returncode == 0, f"trace_run failed ({result.returncode}):\n{result.stdout[-2000:]}\n{result.stderr[-4000:]}"
    done = [line for line in result.stdout.splitlines() if line.startswith("done ")]
    assert [int(line.split()[1]) for line in done] == [s["step"] for s in steps], result.stdout[-2000:]
    logits = {}
    for step in steps:
        wanted = sum(len(e.get("want", [])) for e in step["entries"])
        path = Path(out) / f"{step['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {step['step']}: {data.size} floats for {wanted} rows"
            logits[step["step"]] = data.reshape(wanted, vocab)
        else:
            assert not path.exists()
    return logits


def random_tokens(rng: np.random.Generator, vocab: int, count: int) -> list[int]:
    return [int(t) for t in rng.integers(0, vocab, size=count)]


# Largest absolute logit error allowed against the plain float64 implementation. Logits of
# these models are of order 0.1 to 1; the float32 bound is a few hundred float32 roundings,
# the bfloat16 bound a few bfloat16 roundings of values of that size.
TOLERANCE = {"float32": 2e-5, "bfloat16": 2e-2}
