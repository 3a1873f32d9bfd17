"""Runs the reference's own Qwen2 model code on the CPU and records its outputs.

    python tests/golden/make_golden.py --reference PATH_TO_THE_REFERENCE_CHECKOUT

The reference's tested engine (python/instinct/mlx_engine.py + backends/dense.py + batches.py +
paged_kv.py) is written against MLX, which exists only for Apple hardware. Its model code is
plain array arithmetic, though, so this script registers a small NumPy stand-in under the
name ``mlx.core`` (32-bit floats throughout, ``float16`` mapped to ``float32``), selects the
reference's plain operators (INSTINCT_KERNELS=plain), writes a tiny random model with the
reference's own ``write_engine``, and drives the reference's ``MlxEngine``: chunked prefill
over pages of four positions, greedy generation, batched requests. The outputs go to
``reference_outputs.json`` beside this file together with the weights' seed, and are compared
with tests/plain/qwen2_plain.py here and again, without the reference, in
tests/test_golden.py.

Nothing of the reference is copied: it is imported from its own checkout at run time.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def numpy_mlx() -> types.ModuleType:
    """The few dozen names of mlx.core the reference's Qwen2 path touches, over NumPy."""
    mx = types.ModuleType("mlx.core")

    def array(value, dtype=None):
        out = np.array(value, dtype=dtype)
        if out.dtype == np.float16:
            out = out.astype(np.float32)
        return out

    mx.array = array
    mx.float16 = mx.bfloat16 = mx.float32 = np.float32
    mx.int8, mx.int32, mx.int64, mx.uint32, mx.bool_ = np.int8, np.int32, np.int64, np.uint32, np.bool_
    mx.inf = np.inf
    mx.zeros = lambda shape, dtype=np.float32: np.zeros(shape, dtype=dtype)
    mx.ones = lambda shape, dtype=np.float32: np.ones(shape, dtype=dtype)
    mx.arange = lambda *a, dtype=None, **k: np.arange(*a, dtype=dtype, **k)
    mx.concatenate = lambda arrays, axis=0: np.concatenate(arrays, axis=axis)
    mx.cos, mx.sin, mx.tanh, mx.exp, mx.abs = np.cos, np.sin, np.tanh, np.exp, np.abs
    mx.where, mx.maximum, mx.minimum, mx.clip, mx.round = np.where, np.maximum, np.minimum, np.clip, np.round
    mx.repeat = lambda x, repeats, axis=None: np.repeat(x, repeats, axis=axis)
    mx.take_along_axis = lambda x, idx, axis: np.take_along_axis(x, idx, axis=axis)
    mx.mean = lambda x, axis=None, keepdims=False: np.mean(x, axis=axis, keepdims=keepdims)
    mx.max = lambda x, axis=None, keepdims=False: np.max(x, axis=axis, keepdims=keepdims)
    mx.argmax = lambda x, axis=None: np.argmax(x, axis=axis)
    mx.rsqrt = lambda x: (1.0 / np.sqrt(x)).astype(np.float32)
    mx.sigmoid = lambda x: (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
    mx.cumsum = lambda x, axis=None: np.cumsum(x, axis=axis)

    def softmax(x, axis=-1):
        shifted = x - np.max(x, axis=axis, keepdims=True)
        e = np.exp(shifted)
        return (e / np.sum(e, axis=axis, keepdims=True)).astype(np.float32)

    mx.softmax = softmax
    mx.eval = lambda *a, **k: None
    mx.disable_compile = lambda: None
    mx.enable_compile = lambda: None
    mx.gpu, mx.cpu = "gpu", "cpu"
    mx.default_device = lambda: "cpu"
    mx.metal = types.SimpleNamespace(is_available=lambda: False)
    mx.device_info = lambda: {"device_name": "numpy", "architecture": "cpu"}
    mx.get_active_memory = lambda: 0
    mx.fast = types.SimpleNamespace()
    return mx


def install_stand_in() -> None:
    os.environ["INSTINCT_KERNELS"] = "plain"
    package = types.ModuleType("mlx")
    core = numpy_mlx()
    package.core = core
    sys.modules["mlx"] = package
    sys.modules["mlx.core"] = core


CASES = {
    # Full attention, tied head: the plain Qwen2 path.
    "full": dict(vocab=48, hidden=64, inter=40, layers=2, heads=4, kv_heads=2, theta=10000.0, eps=1e-6, window=0, pattern=0),
    # The reference's layer pattern with a window of 6: layers 0 and 1 see the last six
    # positions, layer 2 all of them (python/instinct/format.py:70-75).
    "window": dict(vocab=37, hidden=48, inter=56, layers=3, heads=3, kv_heads=1, theta=1000000.0, eps=1e-5, window=6, pattern=3),
}
PROMPT_LENGTHS = [1, 3, 4, 5, 9, 16, 17, 33]
SEED = 17


def make_weights(case: dict) -> dict[str, np.ndarray]:
    """Random weights whose values are exact in float16 (the reference's file format)."""
    rng = np.random.default_rng(SEED)
    head_dim = case["hidden"] // case["heads"]

    def w(*shape, scale=0.12):
        return (rng.standard_normal(shape) * scale).astype(np.float16)

    def norm():
        return (1.0 + rng.standard_normal(case["hidden"]) * 0.05).astype(np.float16)

    tensors = {"model.embed_tokens.weight": w(case["vocab"], case["hidden"]), "model.norm.weight": norm()}
    for layer in range(case["layers"]):
        p = f"model.layers.{layer}."
        tensors[p + "input_layernorm.weight"] = norm()
        tensors[p + "post_attention_layernorm.weight"] = norm()
        for name, heads in (("q_proj", case["heads"]), ("k_proj", case["kv_heads"]), ("v_proj", case["kv_heads"])):
            tensors[p + f"self_attn.{name}.weight"] = w(heads * head_dim, case["hidden"])
            tensors[p + f"self_attn.{name}.bias"] = w(heads * head_dim, scale=0.05)
        tensors[p + "self_attn.o_proj.weight"] = w(case["hidden"], case["heads"] * head_dim)
        tensors[p + "mlp.gate_proj.weight"] = w(case["inter"], case["hidden"])
        tensors[p + "mlp.up_proj.weight"] = w(case["inter"], case["hidden"])
        tensors[p + "mlp.down_proj.weight"] = w(case["hidden"], case["inter"])
    return tensors


def plain_config(case: dict) -> dict:
    config = dict(
        vocab_size=case["vocab"], hidden_size=case["hidden"], intermediate_size=case["inter"],
        num_hidden_layers=case["layers"], num_attention_heads=case["heads"], num_key_value_heads=case["kv_heads"],
        rope_theta=case["theta"], rms_norm_eps=case["eps"], tie_word_embeddings=True, sliding_window=case["window"],
    )
    if case["pattern"]:
        config["layer_types"] = [
            "sliding_attention" if (layer + 1) % case["pattern"] else "full_attention" for layer in range(case["layers"])
        ]
    return config


def prompts_for(case: dict) -> list[list[int]]:
    return [[(i * 5 + 3 + n) % case["vocab"] for i in range(n)] for n in PROMPT_LENGTHS]


def run_reference(case: dict, tensors: dict[str, np.ndarray]) -> dict:
    from instinct.format import ModelConfig, write_engine
    from instinct.mlx_engine import MlxEngine

    config = ModelConfig(
        vocab_size=case["vocab"], hidden_size=case["hidden"], intermediate_size=case["inter"],
        num_hidden_layers=case["layers"], num_attention_heads=case["heads"], num_key_value_heads=case["kv_heads"],
        max_position_embeddings=128, eos_token_id=2, rope_theta=case["theta"], rms_norm_eps=case["eps"],
        sliding_window=case["window"], sliding_window_pattern=case["pattern"],
    )
    stored = dict(tensors)
    stored["lm_head.weight"] = stored["model.embed_tokens.weight"]
    out: dict = {"prefill_logits": [], "greedy": [], "batched": []}
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "tiny.engine"
        write_engine(path, config, stored, aliases={"lm_head.weight": "model.embed_tokens.weight"})
        with MlxEngine(path, max_num_sequences=3, kv_cache_bytes=1 << 20, prefill_chunk_size=5,
                       prefill_burst_size=8, page_size=4) as engine:
            for prompt in prompts_for(case):
                out["prefill_logits"].append(np.asarray(engine.prefill_logits(prompt), dtype=np.float32).tolist())
            prompts = prompts_for(case)
            out["greedy"] = [[int(t) for t in engine.generate(p, 10)] for p in prompts[:4]]
            ids = [engine.submit(p, 6) for p in prompts[2:7]]
            while engine.has_work():
                engine.step()
            out["batched"] = [[int(t) for t in engine.request(i).output] for i in ids]
            pools = engine.stats()["kv_pools"]
            assert all(p["used_pages"] == 0 and p["reserved_pages"] == 0 for p in pools.values())
    return out


def compare_with_plain(case: dict, tensors: dict[str, np.ndarray], reference: dict) -> float:
    from plain import qwen2_plain as plain

    config = plain_config(case)
    weights = {name: value.astype(np.float64) for name, value in tensors.items()}
    worst = 0.0
    prompts = prompts_for(case)
    for prompt, logits in zip(prompts, reference["prefill_logits"]):
        mine = plain.forward(config, weights, prompt)[-1]
        worst = max(worst, float(np.abs(mine - np.asarray(logits)).max()))
    for prompt, tokens in zip(prompts[:4], reference["greedy"]):
        assert plain.greedy(config, weights, prompt, 10) == tokens, "greedy tokens differ from the reference"
    for prompt, tokens in zip(prompts[2:7], reference["batched"]):
        assert plain.greedy(config, weights, prompt, 6) == tokens, "batched tokens differ from the reference"
    return worst


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--reference", required=True, help="checkout of KavinP21/LLM-Inference")
    args = parser.parse_args()
    install_stand_in()
    sys.path.insert(0, str(Path(args.reference) / "python"))
    record = {"seed": SEED, "prompt_lengths": PROMPT_LENGTHS, "cases": {}}
    for name, case in CASES.items():
        tensors = make_weights(case)
        reference = run_reference(case, tensors)
        worst = compare_with_plain(case, tensors, reference)
        print(f"{name}: max |plain - reference| over {len(PROMPT_LENGTHS)} prompts = {worst:.3e}; greedy and batched tokens equal")
        assert worst < 5e-6
        record["cases"][name] = {"case": case, "max_abs_difference": worst, **reference}
    (HERE / "reference_outputs.json").write_text(json.dumps(record) + "\n")
    print(f"wrote {HERE / 'reference_outputs.json'}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
