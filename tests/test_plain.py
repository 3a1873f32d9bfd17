"""The plain implementation checked on its own (no GPU): parts against closed forms."""

from __future__ import annotations

import numpy as np

from helpers import TINY_A, TINY_B
from plain import qwen2_plain as plain


def test_rms_norm_and_rope_closed_forms():
    x = np.array([[3.0, 4.0]])
    out = plain.rms_norm(x, np.array([2.0, 0.5]), 0.0)
    assert np.allclose(out, [[2 * 3 / np.sqrt(12.5), 0.5 * 4 / np.sqrt(12.5)]])
    # Position 0 leaves the vector alone; a rotation keeps each pair's length.
    v = np.arange(8, dtype=np.float64).reshape(1, 1, 8)
    assert np.allclose(plain.rope(v, [0], 10000.0), v)
    r = plain.rope(np.repeat(v, 3, axis=0), [1, 7, 100], 10000.0)
    for i in range(4):
        assert np.allclose(r[:, 0, i] ** 2 + r[:, 0, i + 4] ** 2, v[0, 0, i] ** 2 + v[0, 0, i + 4] ** 2)
    # The first pair turns by exactly `position` radians.
    assert np.allclose(r[0, 0, 0], 0 * np.cos(1.0) - 4 * np.sin(1.0))
    inverse = plain.rope_inverse_frequencies(8, 10000.0)
    assert inverse.dtype == np.float32 and np.allclose(inverse, 10000.0 ** (-np.arange(4) / 4), rtol=1e-6)


def test_attention_mask_window_and_groups():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((6, 4, 8)), rng.standard_normal((6, 2, 8)), rng.standard_normal((6, 2, 8))
    out = plain.attention(q, k, v, 8**-0.5).reshape(6, 4, 8)
    assert np.allclose(out[0], np.repeat(v[0], 2, axis=0))  # the first token sees only itself
    # Heads 0,1 use kv head 0 and heads 2,3 kv head 1.
    scores = (q[5, 2] * 8**-0.5) @ k[:6, 1].T
    p = np.exp(scores - scores.max())
    assert np.allclose(out[5, 2], (p / p.sum()) @ v[:6, 1])
    # Window 1 sees only itself; window >= length equals full attention.
    assert np.allclose(plain.attention(q, k, v, 1.0, window=1).reshape(6, 4, 8)[3], np.repeat(v[3], 2, axis=0))
    assert np.allclose(plain.attention(q, k, v, 1.0, window=6), plain.attention(q, k, v, 1.0))
    windowed = plain.attention(q, k, v, 1.0, window=3).reshape(6, 4, 8)
    scores = q[5, 0] @ k[3:6, 0].T
    p = np.exp(scores - scores.max())
    assert np.allclose(windowed[5, 0], (p / p.sum()) @ v[3:6, 0])


def test_layer_windows_of_the_tiny_configs():
    assert [plain.layer_window(TINY_A, i) for i in range(2)] == [0, 0]
    assert [plain.layer_window(TINY_B, i) for i in range(3)] == [0, 24, 24]


def test_prefix_property_of_the_whole_model():
    """Causality: logits at a position do not change when tokens are appended."""
    rng = np.random.default_rng(1)
    config = TINY_B
    heads, kv, hidden, inter, vocab = 3, 1, 96, 272, 311
    weights = {"model.embed_tokens.weight": rng.normal(0, 0.05, (vocab, hidden)), "model.norm.weight": np.ones(hidden),
               "lm_head.weight": rng.normal(0, 0.05, (vocab, hidden))}
    for layer in range(3):
        p = f"model.layers.{layer}."
        weights[p + "input_layernorm.weight"] = np.ones(hidden)
        weights[p + "post_attention_layernorm.weight"] = np.ones(hidden)
        for name, rows in (("q_proj", heads * 32), ("k_proj", kv * 32), ("v_proj", kv * 32)):
            weights[p + f"self_attn.{name}.weight"] = rng.normal(0, 0.05, (rows, hidden))
            weights[p + f"self_attn.{name}.bias"] = rng.normal(0, 0.05, rows)
        weights[p + "self_attn.o_proj.weight"] = rng.normal(0, 0.05, (hidden, heads * 32))
        weights[p + "mlp.gate_proj.weight"] = rng.normal(0, 0.05, (inter, hidden))
        weights[p + "mlp.up_proj.weight"] = rng.normal(0, 0.05, (inter, hidden))
        weights[p + "mlp.down_proj.weight"] = rng.normal(0, 0.05, (hidden, inter))
    tokens = [int(t) for t in rng.integers(0, vocab, 40)]
    full = plain.forward(config, weights, tokens)
    assert full.shape == (40, vocab)
    assert np.allclose(plain.forward(config, weights, tokens[:29]), full[:29], atol=1e-12)
    # The window matters from position 24 on (layer 0 is full, layers 1-2 see 24 positions).
    unwindowed = plain.forward({**config, "use_sliding_window": False}, weights, tokens)
    assert np.allclose(unwindowed[:24], full[:24], atol=1e-12) and not np.allclose(unwindowed[24:], full[24:], atol=1e-6)


def test_sampling_filters():
    logits = np.log(np.array([0.5, 0.2, 0.2, 0.06, 0.04]))
    assert np.allclose(plain.surviving_probabilities(logits, 1.0), [0.5, 0.2, 0.2, 0.06, 0.04])
    assert np.allclose(plain.surviving_probabilities(logits, 1.0, top_k=1), [1, 0, 0, 0, 0])
    # top_k = 2 lands on a tie: both 0.2 tokens stay.
    assert np.allclose(plain.surviving_probabilities(logits, 1.0, top_k=2), np.array([0.5, 0.2, 0.2, 0, 0]) / 0.9)
    # top_p 0.6: mass before the 0.2s is 0.5 < 0.6 (kept), before 0.06 it is 0.9 (dropped).
    assert np.allclose(plain.surviving_probabilities(logits, 1.0, top_p=0.6), np.array([0.5, 0.2, 0.2, 0, 0]) / 0.9)
    assert np.allclose(plain.surviving_probabilities(logits, 1.0, min_p=0.3), np.array([0.5, 0.2, 0.2, 0, 0]) / 0.9)
    sharp = plain.surviving_probabilities(logits, 0.5)
    assert np.allclose(sharp, np.array([0.25, 0.04, 0.04, 0.0036, 0.0016]) / 0.3352)
    assert plain.draw_key(3, 2) == 3_000_011 and 0.0 <= plain.uniform_from_key(5) < 1.0


def test_how_decode_attention_cuts_the_key_range():
    """The split rule is a pure function of the batch and the longest request: never more
    splits than 64-key tiles, 16 at most at ordinary lengths, up to 64 only for very few
    (request, kv head) pairs with many keys, and no split once the batch fills the GPU."""
    from llm_inference_b200.parts.ops import MAX_DECODE_SPLITS, decode_splits

    for tma in (False, True):
        for seqs in (1, 2, 8, 64, 300):
            for kv_heads in (1, 2, 8):
                for keys in (1, 64, 65, 1000, 4096, 32768, 131072):
                    splits = decode_splits(seqs, kv_heads, keys, tma)
                    assert 1 <= splits <= min(MAX_DECODE_SPLITS, (keys + 63) // 64)
                    if keys <= 4096:
                        assert splits <= 16
    assert decode_splits(1, 2, 4096, True) == 16 and decode_splits(8, 2, 4096, True) == 13  # 222 blocks / 16 pairs
    assert decode_splits(1, 2, 32768, True) == 64 and decode_splits(8, 2, 32768, True) == 16
    assert decode_splits(6, 2, 4096, True) == 14 and decode_splits(16, 2, 4096, True) == 9  # 296 / 32
    assert decode_splits(1, 8, 32768, True) == 37  # 296 resident blocks / 8 pairs
    assert decode_splits(64, 2, 2048, True) == 2 and decode_splits(64, 8, 2048, True) == 1
    assert decode_splits(1, 2, 100, True) == 2
