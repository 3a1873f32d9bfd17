"""Layers of the benchmark's size (Qwen2.5-1.5B: 12/2 heads of 128, hidden 1536, intermediate
8960, vocabulary 151936), three of them with random weights: a 700-token prompt in two
portions and three decoded tokens. First the 32-bit path against the plain implementation
(and the same for two layers of the 7B and 14B sizes), then bfloat16 with each attention
kernel against the 32-bit path. The tiny test configurations never reach the tile counts,
cluster sizes and split factors these sizes do."""

from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "eos_token_id": 151643, "max_window_layers": 1,
}


def logits_of(dtype: str, attention: str, window: int, gemm: str = "auto", shape: dict | None = None) -> np.ndarray:
    import torch

    from llm_inference_b200 import models  # noqa: F401  (registers the architecture)
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.engine.engine import Engine
    from llm_inference_b200.engine.loading import random_model
    from llm_inference_b200.engine.runner import StepEntry

    settings = dict(shape or SHAPE, use_sliding_window=window > 0, sliding_window=window if window else 32768)
    _, config = parse_config(settings)
    model = random_model(config, 5, dtype, "cuda:0", std=0.05)
    engine = Engine(
        model=model, max_num_sequences=4, max_model_length=2048, kv_cache_bytes=1 << 30, prefill_chunk_size=1024,
        prefill_burst_size=1024, max_batch_tokens=1100, dtype=dtype, cuda_graphs=False,
    )
    engine.runner.options.update(attention=attention, gemm=gemm)
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, settings["vocab_size"], 700)]
    engine.cache.open(1)
    # A step's logits live in a scratch buffer that the next step overwrites: copy them.
    rows = [engine.runner.step([StepEntry(1, prompt[:517], (516,))]).clone()]
    rows.append(engine.runner.step([StepEntry(1, prompt[517:], (len(prompt) - 518,))]).clone())
    for token in (11, 222, 3333):
        rows.append(engine.runner.step([StepEntry(1, (token,), (0,))]).clone())
    engine.runner.check()
    out = torch.cat(rows).float().cpu().numpy()
    engine.close()
    return out


PROMPT_SEED, PROMPT_LENGTH, FIRST_PORTION, DECODED = 0, 700, 517, (11, 222, 3333)


def plain_logits(shape: dict, window: int = 0) -> np.ndarray:
    """What `logits_of` returns, from the plain implementation: the same seeded weights (drawn on
    the GPU as bfloat16, handed over tensor by tensor), the whole sequence at once, logits at the
    five places the engine is asked for."""
    from helpers import device_model
    from plain import qwen2_plain as plain

    settings = dict(shape, use_sliding_window=window > 0, sliding_window=window if window else 32768)
    _, config, weights = device_model(settings, seed=5, dtype=None, std=0.05)
    prompt = [int(t) for t in np.random.default_rng(PROMPT_SEED).integers(0, settings["vocab_size"], PROMPT_LENGTH)]
    tokens = prompt + list(DECODED)
    hidden = plain.hidden_states(config, weights, tokens)
    rows = [FIRST_PORTION - 1, PROMPT_LENGTH - 1, PROMPT_LENGTH, PROMPT_LENGTH + 1, PROMPT_LENGTH + 2]
    return plain.output_logits(config, weights, hidden[rows])


def test_32_bit_path_at_benchmark_sizes_matches_plain():
    """The float32 path (own FMA products over inner sizes up to 18,944, plain attention over 700
    keys) against the plain float64 implementation: within a thousandth of the logits' range."""
    import gc

    import torch

    for name, shape in {"1.5B": SHAPE, **LARGER}.items():
        want = plain_logits(shape)
        got = logits_of("float32", "auto", 0, shape=shape)
        span = float(want.max() - want.min())
        error = np.abs(got - want)
        assert error.max() <= 1e-3 * span, (name, error.max(), span)
        assert (got.argmax(axis=1) == want.argmax(axis=1)).all(), name
        print(f"{name}: float32 path max |logit error| {error.max():.3e}, logits' range {span:.2f}")
        gc.collect()
        torch.cuda.empty_cache()
    # A window that ends inside the prompt, on the 1.5B size.
    want = plain_logits(SHAPE, window=300)
    got = logits_of("float32", "auto", 300)
    assert np.abs(got - want).max() <= 1e-3 * float(want.max() - want.min())


def assert_same_greedy_tokens(got: np.ndarray, reference: np.ndarray, name: str = "") -> None:
    """Every row picks the token the 32-bit path picks, except at a near-tie: where the 32-bit
    logits of the two picks lie closer together than four times the row's own mean rounding
    error, either may win (among 150,000 random logits the best two are often that close)."""
    assert len({row.tobytes() for row in reference}) == len(reference), "rows must be distinct positions"
    for r, (mine, theirs) in enumerate(zip(got.argmax(axis=1), reference.argmax(axis=1))):
        if mine != theirs:
            margin = float(reference[r, theirs] - reference[r, mine])
            rounding = float(np.abs(got[r] - reference[r]).mean())
            assert margin <= 4.0 * rounding, (name, r, int(mine), int(theirs), margin, rounding)


@pytest.mark.parametrize("window", [0, 300], ids=["full", "window300"])
def test_benchmark_sized_layers_in_bfloat16_follow_the_32_bit_path(window):
    reference = logits_of("float32", "auto", window)
    scale = float(reference.std())
    results = {
        name: logits_of("bfloat16", attention, window, gemm)
        for name, (attention, gemm) in {
            "tcgen05": ("tcgen05", "auto"), "flash": ("flash", "auto"), "plain+library": ("plain", "library"),
        }.items()
    }
    for name, got in results.items():
        error = np.abs(got - reference)
        # bfloat16 keeps 8 bits: activations rounded a few dozen times on the way cost a few
        # per cent of the logits' spread, whichever kernels run; a wrong tile costs the spread.
        assert error.mean() <= 0.03 * scale and error.max() <= 0.2 * scale, (name, error.mean(), error.max(), scale)
        assert_same_greedy_tokens(got, reference, name)
    # The engine's own kernels are no further from 32-bit than the library product with the
    # plain attention kernel is.
    baseline = np.abs(results["plain+library"] - reference).mean()
    for name in ("tcgen05", "flash"):
        assert np.abs(results[name] - reference).mean() <= 1.1 * baseline, name


LARGER = {
    "7B": dict(SHAPE, num_hidden_layers=2, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False),
    "14B": dict(SHAPE, num_hidden_layers=2, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=13824, vocab_size=152064, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", list(LARGER))
def test_layers_of_the_larger_shapes_follow_the_32_bit_path(name):
    """Two layers of the Qwen2.5-7B and -14B sizes, the kernels the engine picks by itself."""
    reference = logits_of("float32", "auto", 0, shape=LARGER[name])
    got = logits_of("bfloat16", "auto", 0, shape=LARGER[name])
    scale = float(reference.std())
    error = np.abs(got - reference)
    # What bfloat16 itself costs at this size is measured, not assumed: the same model with the
    # plain attention kernel and the library's products. Sums over 13,824 and 18,944 terms leave
    # the largest of 760,000 rounding errors at a fifth of the logits' spread on that path too
    # (0.21 at the 14B size); the engine's own kernels must not be further off than that, and a
    # wrong tile, which costs the spread, is.
    baseline = np.abs(logits_of("bfloat16", "plain", 0, "library", shape=LARGER[name]) - reference)
    assert error.mean() <= 0.03 * scale, (error.mean(), scale)
    assert error.mean() <= 1.1 * baseline.mean(), (error.mean(), baseline.mean())
    assert error.max() <= 1.25 * baseline.max() and error.max() <= 0.3 * scale, (error.max(), baseline.max(), scale)
    assert_same_greedy_tokens(got, reference, name)
