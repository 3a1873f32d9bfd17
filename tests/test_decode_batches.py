"""Decode steps with many live requests, replayed from captured CUDA graphs, at the benchmark's
layer sizes (Qwen2.5-1.5B: 12/2 heads of 128, hidden 1536, intermediate 8960, vocabulary
151936; three layers), in bfloat16, every request's logits against the plain implementation
of its own sequence.

The batch sizes cross the engine's three regimes of matrix products (up to 16 rows: the
mma.sync and tcgen05 weight-streaming kernels; up to 32: everything on the tcgen05 kernel
with 32 padded columns; 64: the library's products except the down projection) and the padded
batch-size buckets of the captured graphs. The engine is built for a context of 4,096 while
the requests hold 130 to 700 keys, so the captured steps are launched for a longer reach, and
cut the keys into more pieces, than the live requests need.

The 64 requests are prefixes, all of different lengths, of eight random sequences: the plain
implementation runs each sequence once, and its rows at a prefix's last positions are what a
request with that prefix must produce."""

from __future__ import annotations

import numpy as np
import pytest

from helpers import device_model
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "eos_token_id": 151643, "use_sliding_window": False, "sliding_window": 32768,
}
BASES, LONGEST, DECODED = 8, 700, 4


@pytest.fixture(scope="module")
def setting():
    """The model, 64 requests (prefixes of eight base sequences) and the plain logits at each
    request's last ``DECODED`` positions."""
    model, config, weights = device_model(SHAPE, seed=5, dtype="bfloat16", std=0.05)
    rng = np.random.default_rng(3)
    bases = [[int(t) for t in rng.integers(0, SHAPE["vocab_size"], LONGEST)] for _ in range(BASES)]
    # 64 different lengths between 130 and 700, spread over the bases; page edges (multiples of
    # 64) and their neighbours among them.
    lengths = sorted({130 + (i * 571) // 63 for i in range(64)} | {192, 193, 256, 257, 448, 449, 640, 641, 700})
    lengths = [n for n in lengths if n <= LONGEST]
    picks = rng.permutation(len(lengths))[:64]
    requests = [(int(i % BASES), lengths[int(p)]) for i, p in enumerate(picks)]
    assert len({n for _, n in requests}) == 64
    rows_needed = {b: sorted({n - 1 - d for bb, n in requests if bb == b for d in range(DECODED)}) for b in range(BASES)}
    expected = {}
    for b, tokens in enumerate(bases):
        hidden = plain.hidden_states(config, weights, tokens)
        logits = plain.output_logits(config, weights, hidden[rows_needed[b]])
        for row, values in zip(rows_needed[b], logits):
            expected[(b, row)] = values
    return model, bases, requests, expected


def decode_logits(model, bases, requests, kernels: str):
    """The logits of the last ``DECODED`` steps, ``[DECODED, live, vocab]``, and how many steps
    were replayed from a graph."""
    import torch

    from llm_inference_b200.engine.engine import Engine
    from llm_inference_b200.engine.runner import StepEntry

    engine = Engine(
        model=model, max_num_sequences=64, max_model_length=4096, kv_cache_bytes=1 << 30, prefill_chunk_size=1024,
        prefill_burst_size=1024, max_batch_tokens=1100, dtype="bfloat16", cuda_graphs=True, kernels=kernels,
    )
    runner = engine.runner
    assert runner.use_graphs
    # Prompts: everything but the last DECODED tokens, a few requests per step.
    pending = []
    for rid, (b, n) in enumerate(requests, start=1):
        engine.cache.open(rid)
        pending.append(StepEntry(rid, bases[b][: n - DECODED], ()))
    batch, held = [], 0
    for entry in pending + [None]:
        if entry is None or held + len(entry.tokens) > 1100:
            runner.step(batch)
            batch, held = [], 0
        if entry is not None:
            batch.append(entry)
            held += len(entry.tokens)
    # The last tokens one by one, all requests in every step. The logits live in scratch that
    # the next step reuses: copy them.
    got = []
    for d in range(DECODED, 0, -1):
        entries = [StepEntry(rid, (bases[b][n - d],), (0,)) for rid, (b, n) in enumerate(requests, start=1)]
        got.append(runner.step(entries).clone())
    runner.check()
    replays = runner.graph_replays
    out = torch.stack(got).float().cpu().numpy()
    engine.close()
    return out, replays


@pytest.mark.parametrize("live", [8, 17, 32, 64])
def test_decode_steps_of_many_requests_from_captured_graphs(setting, live):
    model, bases, requests, expected = setting
    requests = requests[:live]
    got, replays = decode_logits(model, bases, requests, "tuned")
    assert replays >= 1, "no decode step was replayed from a captured graph"
    # What bfloat16 itself costs at these sizes is measured, not assumed: the same steps with the
    # plain attention kernel and the library's products.
    base, _ = decode_logits(model, bases, requests, "plain")

    ratios_mean, ratios_max, flips = [], [], 0
    for step, d in enumerate(range(DECODED, 0, -1)):
        for i, (b, n) in enumerate(requests):
            want = expected[(b, n - d)]
            error = np.abs(got[step, i] - want)
            floor = np.abs(base[step, i] - want)
            scale = float(want.std())
            where = (live, step, i, b, n)
            # Rounding to bfloat16 a few dozen times on the way costs a few per cent of the logits'
            # spread whichever kernels run; a wrong key, page, split or padded row costs the spread.
            assert floor.mean() <= 0.05 * scale, (where, floor.mean() / scale)
            assert error.mean() <= 1.3 * floor.mean() and error.max() <= 2.0 * floor.max(), (
                where, error.mean() / scale, floor.mean() / scale, error.max() / scale, floor.max() / scale)
            ratios_mean.append(error.mean() / floor.mean())
            ratios_max.append(error.max() / floor.max())
            mine, theirs = int(got[step, i].argmax()), int(want.argmax())
            if mine != theirs:
                # Only a near-tie of the plain logits may be decided the other way.
                assert want[theirs] - want[mine] <= 4.0 * error.mean(), (where, want[theirs] - want[mine], error.mean())
                flips += 1
    print(f"live={live}: error of the tuned kernels over that of the plain ones: mean {np.mean(ratios_mean):.3f} "
          f"(worst {np.max(ratios_mean):.3f}), max {np.mean(ratios_max):.3f} (worst {np.max(ratios_max):.3f}); {flips} near-ties")
