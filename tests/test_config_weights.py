"""Configuration, registry and weight loading (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_folder
from llm_inference_b200 import models  # noqa: F401
from llm_inference_b200.config import ConfigError, Qwen2Config, parse_config, registered_architectures
from llm_inference_b200.engine.loading import load_model
from llm_inference_b200.parts import Model
from llm_inference_b200.weights import SafetensorsFile, WeightsError, load_weights, write_safetensors


def test_registry_maps_architecture_name_to_model():
    assert "Qwen2ForCausalLM" in registered_architectures()
    entry, config = parse_config(TINY_A)
    assert isinstance(config, Qwen2Config)
    assert entry.name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="no model registered for 'LlamaForCausalLM'"):
        parse_config({**TINY_A, "architectures": ["LlamaForCausalLM"]})
    # Without "architectures" the model_type decides.
    raw = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert parse_config(raw)[0].name == "Qwen2ForCausalLM"


def test_config_reads_every_size_from_json():
    _, a = parse_config(TINY_A)
    _, b = parse_config(TINY_B)
    assert (a.head_dim, b.head_dim) == (16, 32)
    assert a.eos_token_ids == (2,) and b.eos_token_ids == (5, 7)
    assert [a.layer_window(i) for i in range(2)] == [0, 0]
    assert [b.layer_window(i) for i in range(3)] == [0, 24, 24]
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    # rope_theta may live in rope_parameters; sliding_window is inert unless switched on.
    raw = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    raw["rope_parameters"] = {"rope_theta": 5e5}
    raw["sliding_window"] = 32
    _, c = parse_config(raw)
    assert c.rope_theta == 5e5 and c.layer_window(1) == 0
    # An explicit per-layer list overrides max_window_layers.
    _, d = parse_config({**TINY_B, "layer_types": ["sliding_attention", "full_attention", "sliding_attention"]})
    assert [d.layer_window(i) for i in range(3)] == [24, 0, 24]
    assert parse_config(d.to_json_dict())[1] == d


@pytest.mark.parametrize(
    "change, message",
    [
        ({"hidden_size": None}, "missing required key 'hidden_size'"),
        ({"rms_norm_eps": None}, "missing required key 'rms_norm_eps'"),
        ({"rope_theta": None}, "rope_theta"),
        ({"num_key_value_heads": 3}, "not a multiple"),
        ({"vocab_size": 2_000_000}, "vocab_size"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"eos_token_id": 999}, "outside the vocabulary"),
        ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
        ({"head_dim": 15}, "head_dim"),
        ({"use_sliding_window": True, "sliding_window": 0, "max_window_layers": 0}, "sliding_window"),
        ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
        ({"rope_theta": None, "rope_parameters": {"rope_theta": 1e6, "rope_type": "yarn", "factor": 4}}, "rope_parameters"),
        ({"rope_scaling": "linear"}, "must be an object"),
        ({"num_hidden_layers": "two"}, "must be an integer"),
    ],
)
def test_config_errors(change, message):
    raw = {**TINY_A, **change}
    raw = {k: v for k, v in raw.items() if v is not None}
    with pytest.raises(ConfigError, match=message):
        parse_config(raw)


def test_random_folder_round_trip(tmp_path):
    folder = make_model_folder(tmp_path / "a", TINY_A, seed=3)
    assert sorted(p.name for p in folder.iterdir()) == ["config.json", "model.safetensors"]
    again = make_model_folder(tmp_path / "b", TINY_A, seed=3)
    other = make_model_folder(tmp_path / "c", TINY_A, seed=4)
    assert (folder / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    assert (folder / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    model = load_model(folder, "float32", "cpu")
    # Tied head: no lm_head tensor in the file, the head is the embedding table.
    with SafetensorsFile(folder / "model.safetensors") as file:
        assert "lm_head.weight" not in file.tensors
        assert all(info.dtype == torch.bfloat16 for info in file.tensors.values())
        norm = file.read("model.norm.weight").float()
        assert abs(float(norm.mean()) - 1.0) < 0.02 and 0.005 < float(norm.std()) < 0.04
        embed = file.read("model.embed_tokens.weight").float()
        assert abs(float(embed.mean())) < 0.002 and 0.015 < float(embed.std()) < 0.025
    assert model.head.weight is model.embedding.table
    # q, k and v are one matrix in the model.
    attention = model.blocks[0].mixer
    assert attention.w_qkv.shape == ((4 + 2 * 2) * 16, 64) and attention.b_qkv.dtype == torch.float32
    untied = load_model(make_model_folder(tmp_path / "d", TINY_B, seed=3), "bfloat16", "cpu")
    assert untied.head.weight is not untied.embedding.table and untied.head.weight.dtype == torch.bfloat16


def test_loader_keeps_stored_precision(tmp_path):
    from llm_inference_b200.weights import TensorSpec

    tensors = {
        "half": torch.randn(4, 3).to(torch.float16),
        "brain": torch.randn(4, 3).to(torch.bfloat16),
        "single": torch.randn(5),
        "table": torch.arange(6, dtype=torch.int64),
    }
    write_safetensors(tmp_path / "model.safetensors", tensors)
    specs = [
        TensorSpec("half", (4, 3)),
        TensorSpec("brain", (4, 3)),
        TensorSpec("single", (5,)),
        TensorSpec("table", (6,), integer=True),
        TensorSpec("absent", (2,), optional=True),
    ]
    loaded = load_weights(tmp_path, specs)
    assert loaded["half"].dtype == torch.float16 and torch.equal(loaded["half"], tensors["half"])
    assert loaded["brain"].dtype == torch.bfloat16 and torch.equal(loaded["brain"], tensors["brain"])
    assert loaded["single"].dtype == torch.float32 and torch.equal(loaded["single"], tensors["single"])
    assert loaded["table"].dtype == torch.int32 and loaded["table"].tolist() == list(range(6))
    assert "absent" not in loaded


def test_float16_checkpoint_reaches_a_float32_model_unrounded(tmp_path):
    """A float32 model computes with exactly the stored float16 values; a bfloat16 model
    rounds them once."""
    folder = make_model_folder(tmp_path / "m", TINY_A, seed=4)
    with SafetensorsFile(folder / "model.safetensors") as file:
        tensors = {name: file.read(name) for name in file.tensors}
    generator = torch.Generator().manual_seed(0)
    halves = {
        name: (torch.randn(t.shape, generator=generator) * 0.02 + (1.0 if name.endswith("norm.weight") else 0.0)).to(torch.float16)
        for name, t in tensors.items()
    }
    write_safetensors(folder / "model.safetensors", halves)
    model = load_model(folder, "float32", "cpu")
    down = model.blocks[1].feed_forward.w_down
    assert down.dtype == torch.float32 and torch.equal(down, halves["model.layers.1.mlp.down_proj.weight"].float())
    assert torch.equal(model.embedding.table, halves["model.embed_tokens.weight"].float())
    assert torch.equal(model.final_norm.weight, halves["model.norm.weight"].float())
    # float16 keeps three more mantissa bits than bfloat16: most of these values would change.
    assert not torch.equal(down, down.to(torch.bfloat16).float())
    rounded = load_model(folder, "bfloat16", "cpu")
    assert torch.equal(rounded.blocks[1].feed_forward.w_down, halves["model.layers.1.mlp.down_proj.weight"].to(torch.bfloat16))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_folder(tmp_path / "m", TINY_B, seed=1)
    with SafetensorsFile(folder / "model.safetensors") as file:
        tensors = {name: file.read(name) for name in file.tensors}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.2.self_attn.k_proj.bias"] = torch.zeros(33, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as caught:
        load_model(folder, "float32", "cpu")
    error = caught.value
    assert error.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"] or sorted(error.missing) == [
        "lm_head.weight",
        "model.layers.1.mlp.up_proj.weight",
    ]
    assert error.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert error.wrong_shape == [("model.layers.2.self_attn.k_proj.bias", (33,), (32,))]
    assert error.wrong_kind == [("model.norm.weight", "int32")]
    text = str(error)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [33], expected [32]"):
        assert needle in text


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError, match="not a model folder"):
        load_model(tmp_path / "nothing", "float32", "cpu")
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="no safetensors"):
        load_model(tmp_path, "float32", "cpu")
    with pytest.raises(ValueError, match="unknown dtype"):
        load_model(tmp_path, "float16", "cpu")


def test_run_order_is_data():
    from llm_inference_b200.parts import LayerCall

    entry, config = parse_config(TINY_B)
    recipe = entry.recipe(config)
    # Layer 1 runs twice (second time into a cache entry of its own) and layer 2 reads layer
    # 1's keys and values instead of writing any.
    recipe.schedule = [LayerCall(0), LayerCall(1), LayerCall(1, cache=3), LayerCall(2, cache=1, writes=False)]
    model = Model(recipe)
    specs = model.cache_specs()
    assert sorted(specs) == [0, 1, 3] and specs[0].window == 0 and specs[3].window == 24
    recipe.schedule = [LayerCall(0), LayerCall(2, cache=1, writes=False)]
    with pytest.raises(ValueError, match="nobody writes"):
        Model(recipe).cache_specs()


def test_safetensors_round_trip_and_malformed_files(tmp_path):
    """Whatever the writer writes the reader returns bit for bit (odd sizes, empty tensors,
    every stored dtype); a damaged container is refused with one kind of error that names
    the file."""
    import struct

    import numpy as np
    import torch

    from llm_inference_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

    rng = np.random.default_rng(3)
    tensors = {
        "a.weight": torch.from_numpy(rng.standard_normal((3, 5)).astype(np.float32)),
        "b.odd": torch.from_numpy(rng.standard_normal(7).astype(np.float32)).to(torch.bfloat16),
        "c.half": torch.from_numpy(rng.standard_normal((2, 1, 3)).astype(np.float16)),
        "d.table": torch.from_numpy(rng.integers(-5, 5, (4, 2))).to(torch.int64),
        "e.empty": torch.empty(0, 4),
        "f.scalar": torch.tensor(2.5),
        "g.bytes": torch.arange(11, dtype=torch.uint8),
    }
    path = tmp_path / "model.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt"})
    with SafetensorsFile(path) as file:
        assert file.metadata == {"format": "pt"} and set(file.tensors) == set(tensors)
        for name, tensor in tensors.items():
            got = file.read(name)
            assert got.dtype == tensor.dtype and got.shape == tensor.shape
            assert got.reshape(-1).view(torch.uint8).tolist() == tensor.contiguous().reshape(-1).view(torch.uint8).tolist()

    def container(header: bytes, data: bytes = b"") -> None:
        path.write_bytes(struct.pack("<Q", len(header)) + header + data)

    damaged = {
        "too short": lambda: path.write_bytes(b"\x01\x02"),
        "header length exceeds": lambda: path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}"),
        "not JSON": lambda: container(b"{ nope"),
        "not a JSON object": lambda: container(b"[1, 2]"),
        "is not an object": lambda: container(json.dumps({"w": 3}).encode()),
        "unsupported dtype": lambda: container(json.dumps({"w": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}).encode(), b"\0"),
        "no usable shape": lambda: container(json.dumps({"w": {"dtype": "F32", "data_offsets": [0, 4]}}).encode(), b"\0" * 4),
        "negative size": lambda: container(json.dumps({"w": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}).encode(), b"\0" * 4),
        "bad byte range": lambda: container(json.dumps({"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode(), b"\0" * 8),
        "runs past the file": lambda: container(json.dumps({"w": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode(), b"\0" * 4),
    }
    for message, damage in damaged.items():
        damage()
        with pytest.raises(SafetensorsError, match=message) as caught:
            SafetensorsFile(path)
        assert str(path) in str(caught.value)
