"""The recorded outputs of the reference's own model code (tests/golden/reference_outputs.json,
made by tests/golden/make_golden.py) against the plain implementation and against the engine."""

from __future__ import annotations

import importlib.util
import json
from pathlib import Path

import numpy as np
import pytest

from plain import qwen2_plain as plain

GOLDEN = Path(__file__).resolve().parent / "golden"


def _maker():
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.fixture(scope="module")
def golden():
    maker = _maker()
    record = json.loads((GOLDEN / "reference_outputs.json").read_text())
    assert record["seed"] == maker.SEED and record["prompt_lengths"] == maker.PROMPT_LENGTHS
    return maker, record


@pytest.mark.parametrize("name", ["full", "window"])
def test_plain_implementation_matches_the_reference_outputs(golden, name):
    maker, record = golden
    case = record["cases"][name]["case"]
    tensors = maker.make_weights(case)
    config = maker.plain_config(case)
    weights = {k: v.astype(np.float64) for k, v in tensors.items()}
    prompts = maker.prompts_for(case)
    for prompt, logits in zip(prompts, record["cases"][name]["prefill_logits"]):
        assert np.abs(plain.forward(config, weights, prompt)[-1] - np.asarray(logits)).max() < 5e-6
    for prompt, tokens in zip(prompts[:4], record["cases"][name]["greedy"]):
        assert plain.greedy(config, weights, prompt, 10) == tokens
    for prompt, tokens in zip(prompts[2:7], record["cases"][name]["batched"]):
        assert plain.greedy(config, weights, prompt, 6) == tokens


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["full", "window"])
def test_engine_matches_the_reference_outputs(golden, name, tmp_path):
    """The float32 engine against what the reference's engine produced for the same weights:
    chunked prefill over small pages, greedy generation, batched requests."""
    import torch

    from llm_inference_b200 import create_engine
    from llm_inference_b200.weights import write_safetensors

    maker, record = golden
    case = record["cases"][name]["case"]
    tensors = maker.make_weights(case)
    config = dict(maker.plain_config(case), architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                  max_position_embeddings=128, eos_token_id=2)
    (tmp_path / "config.json").write_text(json.dumps(config))
    # Stored in float16, the reference's own storage format (python/instinct/format.py:204-207):
    # the float32 engine must compute with these values unrounded.
    stored = {k: torch.from_numpy(v.astype(np.float16)) for k, v in tensors.items()}
    assert all(np.array_equal(stored[k].numpy().astype(v.dtype), v) for k, v in tensors.items()), "weights are float16-exact"
    write_safetensors(tmp_path / "model.safetensors", stored)
    prompts = maker.prompts_for(case)
    with create_engine(tmp_path, dtype="float32", max_num_sequences=3, kv_cache_bytes=1 << 20, prefill_chunk_size=5,
                       prefill_burst_size=8, page_size=4) as engine:
        for prompt, logits in zip(prompts, record["cases"][name]["prefill_logits"]):
            assert np.abs(engine.prefill_logits(prompt) - np.asarray(logits)).max() < 2e-5
        for prompt, tokens in zip(prompts[:4], record["cases"][name]["greedy"]):
            assert engine.generate(prompt, 10) == tokens
        ids = [engine.submit(p, 6) for p in prompts[2:7]]
        while engine.has_work():
            engine.step()
        assert [engine.request(i).output for i in ids] == record["cases"][name]["batched"]
