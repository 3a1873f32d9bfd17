"""A plain, slow Qwen2 forward pass in NumPy: whole sequences, no cache, one function per part.

Written from the reference's formulas (paths are within KavinP21/LLM-Inference); it imports
nothing from the engine and the engine imports nothing from here. Arithmetic is float64
unless a function says otherwise, so it stands above both the engine's float32 path and its
bfloat16 path. It is compared once with the reference's own model code run on the CPU
(tests/golden/make_golden.py).
"""

from __future__ import annotations

import numpy as np

F64 = np.float64


def linear(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """``x @ W.T (+ b)`` with ``W`` stored ``[out, in]`` - python/instinct/backends/base.py:83-101."""
    out = x.astype(F64) @ weight.astype(F64).T
    return out if bias is None else out + bias.astype(F64)


def embed(table: np.ndarray, tokens) -> np.ndarray:
    """``table[tokens]``, no scaling for Qwen2 - python/instinct/backends/dense.py:82-84,
    python/instinct/backends/base.py:103-107."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F64)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``x * rsqrt(mean(x^2) + eps) * w`` - python/instinct/backends/portable.py:144-149."""
    x = x.astype(F64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight.astype(F64)


def rope_inverse_frequencies(dims: int, theta: float) -> np.ndarray:
    """``theta ** (-2 i / dims)`` for ``i < dims / 2``, in float32 as the reference computes it -
    python/instinct/backends/portable.py:117-119."""
    half = dims // 2
    return np.float32(theta) ** (-np.arange(0, half, dtype=np.float32) * np.float32(2) / np.float32(dims))


def rope(x: np.ndarray, positions, theta: float) -> np.ndarray:
    """Rotate ``[tokens, heads, head_dim]`` at ``positions``: dim i pairs with i + d/2,
    ``x'[i] = x[i] cos a - x[i+d/2] sin a``, ``x'[i+d/2] = x[i+d/2] cos a + x[i] sin a``,
    ``a = position * inv_freq[i]`` formed in float32 -
    python/instinct/backends/portable.py:115-132 (also tests/test_mlx_engine.py:105-115)."""
    dims = x.shape[-1]
    half = dims // 2
    inverse = rope_inverse_frequencies(dims, theta)
    angles = (np.asarray(positions, dtype=np.float32)[:, None] * inverse[None, :]).astype(np.float32)
    cos = np.cos(angles.astype(F64))[:, None, :]
    sin = np.sin(angles.astype(F64))[:, None, :]
    x = x.astype(F64)
    first, second = x[..., :half], x[..., half:]
    return np.concatenate([first * cos - second * sin, second * cos + first * sin], axis=-1)


def softmax(scores: np.ndarray) -> np.ndarray:
    shifted = scores - np.max(scores, axis=-1, keepdims=True)
    e = np.exp(shifted)
    return e / np.sum(e, axis=-1, keepdims=True)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int = 0) -> np.ndarray:
    """Causal attention of a whole sequence: ``q [T, nh, d]``, ``k, v [T, nkv, d]`` -> ``[T, nh*d]``.

    Query head h reads kv head ``h // (nh / nkv)`` (python/instinct/backends/portable.py:175-178);
    scores are ``(q * scale) @ k.T`` (:179); a key is visible when ``key <= query`` and, with a
    window, ``key > query - window`` (python/instinct/batches.py:110-113); hidden scores are
    -inf before the softmax (portable.py:186-188)."""
    tokens, q_heads, dim = q.shape
    groups = q_heads // k.shape[1]
    k = np.repeat(k.astype(F64), groups, axis=1).transpose(1, 0, 2)
    v = np.repeat(v.astype(F64), groups, axis=1).transpose(1, 0, 2)
    qh = q.astype(F64).transpose(1, 0, 2) * scale
    scores = qh @ k.transpose(0, 2, 1)
    query = np.arange(tokens)[:, None]
    key = np.arange(tokens)[None, :]
    mask = key <= query
    if window:
        mask &= key > query - window
    scores = np.where(mask[None], scores, -np.inf)
    out = softmax(scores) @ v
    return out.transpose(1, 0, 2).reshape(tokens, q_heads * dim)


def swiglu(h: np.ndarray, gate_w: np.ndarray, up_w: np.ndarray, down_w: np.ndarray) -> np.ndarray:
    """``down(gate * sigmoid(gate) * up)`` - python/instinct/backends/dense.py:124-128."""
    gate = linear(h, gate_w)
    up = linear(h, up_w)
    return linear(gate / (1.0 + np.exp(-gate)) * up, down_w)


def layer_window(config: dict, layer: int) -> int:
    """Window of a layer: with ``use_sliding_window`` the layers ``>= max_window_layers`` see the
    last ``sliding_window`` positions; an explicit ``layer_types`` list overrides the rule. The
    reference's window semantics ("the last w positions, the query's included") are in
    python/instinct/batches.py:56-57,110-113 and python/instinct/backends/metal_kernels.py:33."""
    types = config.get("layer_types")
    if types:
        return int(config["sliding_window"]) if types[layer] == "sliding_attention" else 0
    if config.get("use_sliding_window") and layer >= int(config.get("max_window_layers", 0)):
        return int(config["sliding_window"])
    return 0


def attention_block(config: dict, weights: dict, layer: int, h: np.ndarray, positions) -> np.ndarray:
    """Projections with bias, rotary encoding, attention, output projection without bias -
    python/instinct/backends/dense.py:88-104."""
    p = f"model.layers.{layer}.self_attn."
    heads, kv_heads = int(config["num_attention_heads"]), int(config["num_key_value_heads"])
    dim = int(config.get("head_dim") or config["hidden_size"] // heads)
    tokens = h.shape[0]
    q = linear(h, weights[p + "q_proj.weight"], weights[p + "q_proj.bias"]).reshape(tokens, heads, dim)
    k = linear(h, weights[p + "k_proj.weight"], weights[p + "k_proj.bias"]).reshape(tokens, kv_heads, dim)
    v = linear(h, weights[p + "v_proj.weight"], weights[p + "v_proj.bias"]).reshape(tokens, kv_heads, dim)
    q = rope(q, positions, float(config["rope_theta"]))
    k = rope(k, positions, float(config["rope_theta"]))
    out = attention(q, k, v, dim**-0.5, layer_window(config, layer))
    return linear(out, weights[p + "o_proj.weight"])


def hidden_states(config: dict, weights: dict, tokens) -> np.ndarray:
    """The residual stream after the last layer - python/instinct/backends/dense.py:80-129."""
    x = embed(weights["model.embed_tokens.weight"], tokens)
    positions = np.arange(len(tokens))
    eps = float(config["rms_norm_eps"])
    for layer in range(int(config["num_hidden_layers"])):
        p = f"model.layers.{layer}."
        h = rms_norm(x, weights[p + "input_layernorm.weight"], eps)
        x = x + attention_block(config, weights, layer, h, positions)
        h = rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu(
            h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"]
        )
    return x


def output_logits(config: dict, weights: dict, x: np.ndarray) -> np.ndarray:
    """Last norm and output head; a tied head is the embedding table -
    python/instinct/backends/dense.py:132-134, python/instinct/export.py:38-41."""
    head = weights.get("lm_head.weight")
    if head is None:
        if not config.get("tie_word_embeddings"):
            raise KeyError("lm_head.weight")
        head = weights["model.embed_tokens.weight"]
    return linear(rms_norm(x, weights["model.norm.weight"], float(config["rms_norm_eps"])), head)


def forward(config: dict, weights: dict, tokens) -> np.ndarray:
    """Logits ``[tokens, vocab]`` at every position of one whole sequence."""
    return output_logits(config, weights, hidden_states(config, weights, tokens))


def greedy(config: dict, weights: dict, prompt, count: int) -> list[int]:
    """Greedy continuation by re-running the whole sequence (tests/test_mlx_engine.py:213-222);
    ties go to the lowest id (cuda/kernels.cu:333)."""
    tokens = list(prompt)
    out = []
    for _ in range(count):
        token = int(np.argmax(forward(config, weights, tokens)[-1]))
        out.append(token)
        tokens.append(token)
    return out


# --- sampling (python/instinct/sampling.py:47-101) ---------------------------------------------

CANDIDATES = 1024


def surviving_probabilities(
    logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0
) -> np.ndarray:
    """Probability of each token after the reference's filters, renormalised over survivors.

    Candidates are the 1024 largest logits (sampling.py:67-72); ``probs`` is the softmax of
    ``logit / temperature`` over the candidates (:76-77); a candidate survives if its rank is
    below ``top_k`` (:79-80), ``probs >= min_p * probs.max()`` (:81-82) and the mass before it
    in descending order is ``< top_p`` (:83-85). Equal logits are ranked together here."""
    logits = np.asarray(logits, dtype=F64)
    vocab = logits.shape[0]
    count = min(CANDIDATES, vocab)
    order = np.argsort(-logits, kind="stable")[:count]
    candidate_floor = logits[order[-1]]
    candidates = logits >= candidate_floor
    scaled = logits / temperature
    probs = np.where(candidates, np.exp(scaled - scaled.max()), 0.0)
    probs = probs / probs.sum()
    keep = candidates.copy()
    if top_k and top_k < count:
        keep &= logits >= logits[order[top_k - 1]]
    keep &= probs >= min_p * probs.max()
    if top_p < 1.0:
        mass_before = np.array([probs[logits > value].sum() for value in logits])
        keep &= mass_before < top_p
    kept = np.where(keep, probs, 0.0)
    return kept / kept.sum()


def splitmix64(x: int) -> int:
    mask = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & mask
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & mask
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & mask
    return x ^ (x >> 31)


def draw_key(seed: int, generated: int) -> int:
    """``(seed * 1_000_003 + tokens generated so far) mod 2^63`` - sampling.py:94-98."""
    return (seed * 1_000_003 + generated) % (1 << 63)


def uniform_from_key(key: int) -> float:
    """The engine's own draw: the top 24 bits of splitmix64(key) as a fraction."""
    return (splitmix64(key) >> 40) / float(1 << 24)
