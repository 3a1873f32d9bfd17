"""Decode steps as one resident kernel (csrc/kernels/resident_decode.cu) against the plain
implementation and against the chain of kernels it replaces.

The model is small but has every size the kernel cuts work by: heads of 128 in groups of two
over two kv heads, a hidden width of two row tiles, a feed-forward width that is no multiple of
128, a vocabulary that is no multiple of anything, one layer with a window, and pages of 64.
Queries and keys are scaled up so that attention picks few keys. The requests hold between 1
and 330 keys: shorter than a tile, ending on a page's edge and just past it, longer than the
window."""

from __future__ import annotations

import numpy as np
import pytest

from helpers import device_model
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "hidden_size": 256,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 576,
    "vocab_size": 1003, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 1024, "eos_token_id": 2, "use_sliding_window": True, "sliding_window": 100,
    "max_window_layers": 2,
}
LENGTHS = [5, 64, 65, 128, 129, 200, 330, 77, 1 + 4, 256, 257, 191, 192, 193, 300, 40]
DECODED = 4


@pytest.fixture(scope="module")
def setting():
    model, config, weights = device_model(SHAPE, seed=13, dtype="bfloat16", std=0.05, sharpen=1.5)
    rng = np.random.default_rng(21)
    sequences = [[int(t) for t in rng.integers(0, SHAPE["vocab_size"], n)] for n in LENGTHS]
    expected = [plain.forward(config, weights, tokens)[-DECODED:] for tokens in sequences]
    return model, sequences, expected


def decode_logits(model, sequences, decode_kernel: str, cuda_graphs: bool, fold_norms: bool = False):
    import torch

    from llm_inference_b200.engine.engine import Engine
    from llm_inference_b200.engine.runner import StepEntry

    engine = Engine(
        model=model, max_num_sequences=16, max_model_length=1024, kv_cache_bytes=64 << 20, prefill_chunk_size=512,
        prefill_burst_size=512, max_batch_tokens=600, dtype="bfloat16", cuda_graphs=cuda_graphs, decode_kernel=decode_kernel,
        fold_norms=fold_norms,
    )
    runner = engine.runner
    assert (runner.options["resident"] is not None) == (decode_kernel == "resident")
    for rid, tokens in enumerate(sequences, start=1):
        engine.cache.open(rid)
        if len(tokens) > DECODED:
            runner.step([StepEntry(rid, tokens[:-DECODED], ())])
    got = []
    launches = []
    for d in range(DECODED, 0, -1):
        entries = [StepEntry(rid, (tokens[-d],), (0,)) for rid, tokens in enumerate(sequences, start=1)]
        before = runner.lib.calls
        got.append(runner.step(entries).clone())
        launches.append(runner.lib.calls - before)
    runner.check()
    out = torch.stack(got).float().cpu().numpy()  # [DECODED, requests, vocab]
    engine.close()
    return out, launches


@pytest.mark.parametrize("graphs", [False, True], ids=["launched", "captured"])
@pytest.mark.parametrize("live", [1, 3, 8, 16])
def test_resident_decode_steps_match_plain_and_the_chain(setting, live, graphs):
    model, sequences, expected = setting
    sequences, expected = sequences[:live], expected[:live]
    got, launches = decode_logits(model, sequences, "resident", graphs)
    chain, chain_launches = decode_logits(model, sequences, "chain", graphs)
    if not graphs:
        # One launch per step (the first step also builds the plan) against the chain's dozens.
        assert launches[-1] == 1 and max(launches) <= 2 and min(chain_launches) > 20, (launches, chain_launches)
    ratios = []
    for step in range(DECODED):
        for i in range(live):
            want = expected[i][step]
            error = np.abs(got[step, i] - want)
            floor = np.abs(chain[step, i] - want)
            spread = float(want.std())
            where = (live, step, i, LENGTHS[i])
            assert floor.max() <= 0.6 * spread and floor.mean() <= 0.15 * spread, (where, floor.max() / spread, floor.mean() / spread)
            # The two paths round at different places (the resident kernel takes q, k and v from the
            # 32-bit product straight through bias and rotation, and applies 1 / rms after the
            # product instead of before it), so a single row may come out up to twice as far from
            # the plain implementation as the chain's, or half as far; a wrong key, page or split
            # costs the logits' spread, ten times that.
            assert error.mean() <= 2.0 * floor.mean() + 0.002 * spread and error.max() <= 2.0 * floor.max() + 0.01 * spread, (
                where, error.max() / spread, floor.max() / spread, error.mean() / spread, floor.mean() / spread)
            ratios.append(error.mean() / floor.mean())
    # Over all rows the two paths are equally far from the plain implementation.
    print(f"live={live}: mean error of the resident kernel over the chain's, per row: mean {np.mean(ratios):.3f}, "
          f"min {np.min(ratios):.3f}, max {np.max(ratios):.3f}")
    assert np.mean(ratios) <= 1.05, ratios  # measured: 0.90 to 0.94


@pytest.mark.parametrize("live", [1, 5, 16])
def test_norms_folded_into_the_products_match_plain_and_the_chain(setting, live):
    """The option that folds every RMSNorm of a short step into the products around it (the
    product before adds into the residual stream itself, the product after applies 1 / rms):
    fewer launches, the same logits to rounding."""
    model, sequences, expected = setting
    sequences, expected = sequences[:live], expected[:live]
    got, launches = decode_logits(model, sequences, "chain", False, fold_norms=True)
    chain, chain_launches = decode_logits(model, sequences, "chain", False)
    layers = SHAPE["num_hidden_layers"]
    assert launches[-1] == chain_launches[-1] - (2 * layers - 1), (launches, chain_launches)  # all norms but the first
    ratios = []
    for step in range(DECODED):
        for i in range(live):
            want = expected[i][step]
            error, floor = np.abs(got[step, i] - want), np.abs(chain[step, i] - want)
            spread = float(want.std())
            assert error.mean() <= 2.0 * floor.mean() + 0.002 * spread and error.max() <= 2.0 * floor.max() + 0.01 * spread, (
                live, step, i, error.max() / spread, floor.max() / spread)
            ratios.append(error.mean() / floor.mean())
    assert np.mean(ratios) <= 1.1, ratios


def test_generation_through_the_engine_uses_the_resident_kernel(setting):
    """Greedy generation with run-ahead and captured graphs: the scheduler's path over the
    resident kernel gives the tokens of the chain of kernels, up to a near-tie."""
    from llm_inference_b200.engine.engine import Engine

    model, sequences, _ = setting
    prompts = [sequences[6][:150], sequences[5][:70], sequences[14][:201]]
    outputs = {}
    for kernel in ("resident", "chain"):
        with Engine(model=model, max_num_sequences=4, max_model_length=1024, kv_cache_bytes=64 << 20, prefill_chunk_size=96,
                    prefill_burst_size=96, dtype="bfloat16", decode_kernel=kernel) as engine:
            ids = [engine.submit(p, 24) for p in prompts]
            while engine.has_work():
                engine.step()
            outputs[kernel] = [engine.request(i).output for i in ids]
            assert engine.stats()["steps_ahead_used"] > 10
    same = sum(a == b for a, b in zip(outputs["resident"], outputs["chain"]))
    first_difference = [next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), len(a)) for a, b in zip(outputs["resident"], outputs["chain"])]
    assert same >= 2 or min(first_difference) >= 8, (outputs, first_difference)
