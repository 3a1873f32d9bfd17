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


# Sizes far from the two tiny configurations: many heads over a narrow width with wide heads
# (the output projection's inner size is a hundred times its outer one), the smallest heads, and
# heads of 128 and 64, which in bfloat16 run the tensor-core attention kernels (prompt portions
# on tcgen05 or mma.sync, single tokens on the split-key kernels fed by TMA or cp.async) where
# the others run the plain kernel; one of them with a window that ends inside a page.
OTHER_SIZES = {
    "heads_of_128": dict(
        TINY["B"], hidden_size=136, head_dim=128, num_attention_heads=6, num_key_value_heads=2, intermediate_size=200,
        vocab_size=401, num_hidden_layers=2, sliding_window=70, max_window_layers=1, max_position_embeddings=512,
    ),
    "heads_of_64": dict(
        TINY["A"], hidden_size=88, head_dim=64, num_attention_heads=5, num_key_value_heads=5, intermediate_size=120,
        vocab_size=333, num_hidden_layers=2, max_position_embeddings=512,
    ),
    "wide_heads": dict(
        TINY["B"], hidden_size=40, head_dim=192, num_attention_heads=21, num_key_value_heads=3, intermediate_size=520,
        vocab_size=257, num_hidden_layers=2, sliding_window=17, max_window_layers=1, rms_norm_eps=3e-6,
    ),
    "small_heads": dict(
        TINY["A"], hidden_size=264, head_dim=16, num_attention_heads=5, num_key_value_heads=1, intermediate_size=56,
        vocab_size=1537, num_hidden_layers=1, rope_theta=500000.0, max_position_embeddings=256,
    ),
}


# Factor by which `sharpen_attention` scales queries and keys of the models whose bfloat16 steps
# run the tensor-core attention kernels.
SHARPENED = {"heads_of_128": 8.0, "heads_of_64": 8.0}


def make_model_folder(folder: Path, raw_config: dict, seed: int, std: float = 0.02) -> Path:
    """config.json + model.safetensors with seeded random bfloat16 weights."""
    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.weights import write_model_folder

    _, config = parse_config(raw_config)
    return write_model_folder(folder, config, seed, std=std)


def sharpen_attention(folder: Path, factor: float) -> None:
    """Multiply every query and key projection (weights and biases) of a model folder by
    ``factor``. With N(0, 0.02) weights all scores are nearly equal and one wrong key among a
    hundred moves a logit by less than bfloat16 rounding; with queries and keys scaled up the
    softmax picks few keys, and a wrong key, page or mask edge moves the logits by their own
    spread. Everything else keeps its scale, so the logits stay of order 0.1 to 1."""
    from llm_inference_b200.weights import SafetensorsFile, write_safetensors

    path = Path(folder) / "model.safetensors"
    with SafetensorsFile(path) as file:
        tensors = {name: file.read(name).clone() for name in file.tensors}
    for name, tensor in tensors.items():
        if ".q_proj." in name or ".k_proj." in name:
            tensors[name] = (tensor.float() * factor).to(tensor.dtype)
    write_safetensors(path, tensors)


class LazyWeights:
    """Weights that live on the GPU, handed to the plain implementation one tensor at a time as
    float32 NumPy (it widens them to float64 itself): models of the benchmark's sizes would not
    fit the host twice over in float64."""

    def __init__(self, tensors: dict) -> None:
        self.tensors = tensors

    def __getitem__(self, name: str):
        return self.tensors[name].float().cpu().numpy()

    def get(self, name: str, default=None):
        return self[name] if name in self.tensors else default

    def __contains__(self, name: str) -> bool:
        return name in self.tensors


def device_model(settings: dict, seed: int, dtype: str | None, std: float, sharpen: float = 1.0):
    """(model on cuda:0 with seeded random weights, raw config dict, the same weights for the
    plain implementation). Nothing is written to disk. With ``dtype=None`` the model is built
    but not loaded (only the weights are wanted)."""
    import torch

    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.engine.loading import parse_dtype
    from llm_inference_b200.parts.model import Model
    from llm_inference_b200.weights import random_weights

    entry, config = parse_config(settings)
    model = Model(entry.recipe(config))
    tensors = random_weights(model.tensor_specs(), seed, std=std, dtype=torch.bfloat16, device="cuda:0")
    if sharpen != 1.0:
        for name in tensors:
            if ".q_proj." in name or ".k_proj." in name:
                tensors[name] = (tensors[name].float() * sharpen).to(torch.bfloat16)
    if dtype is not None:
        model.load(tensors, parse_dtype(dtype), torch.device("cuda:0"))
    return model, dict(settings), LazyWeights(tensors)


def plain_weights(folder: Path) -> tuple[dict, dict]:
    """(config dict, weights as float64 arrays) read with the safetensors package, not the engine."""
    import torch
    from safetensors.torch import load_file

    config = json.loads((Path(folder) / "config.json").read_text())
    tensors = load_file(str(Path(folder) / "model.safetensors"))
    return config, {name: t.to(torch.float64).numpy() for name, t in tensors.items()}


def run_trace(
    model: Path, dtype: str, steps: list[dict], out: Path, max_tokens: int, page_size: int | None = None, timeout: int = 600,
    extra: list[str] | None = None,
) -> dict[int, np.ndarray]:
    """Drive bin/trace_run with ``steps``; returns step -> float32 logits ``[wanted, vocab]``."""
    vocab = json.loads((Path(model) / "config.json").read_text())["vocab_size"]
    cmd = [sys.executable, str(TRACE_RUN), "--model", str(model), "--dtype", dtype, "--out", str(out), "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    cmd += list(extra or [])
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
