"""Typed model configurations read from a checkpoint's ``config.json``.

``ModelConfig`` is the small base every architecture's configuration derives
from; ``Qwen2Config`` is the one architecture this engine runs. Every size and
constant the model needs comes from these fields: nothing is defaulted in model
code. Key names and the required/optional split follow the reference's reader
(python/instinct/format.py:77-169) and its validation limits
(src/model_file.cpp:58-92, python/instinct/model_file.py:300-360).
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that is missing keys or describes an impossible model."""


_MISSING = object()


def _take(raw: dict[str, Any], key: str, kind: type, default: Any = _MISSING) -> Any:
    value = raw.get(key, None)
    if value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json is missing required key '{key}'")
        return default
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"config.json key '{key}' must be an integer, got {value!r}")
        return int(value)
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json key '{key}' must be a number, got {value!r}")
        return float(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config.json key '{key}' must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json key '{key}' must be a string, got {value!r}")
        return value
    raise TypeError(kind)


@dataclass(frozen=True)
class ModelConfig:
    """Fields every decoder-only architecture has."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...]

    # Limits the reference enforces on any model file (src/model_file.cpp:58-64).
    MAX_VOCAB: ClassVar[int] = 1_000_000
    MAX_HIDDEN: ClassVar[int] = 65_536
    MAX_INTERMEDIATE: ClassVar[int] = 262_144
    MAX_LAYERS: ClassVar[int] = 1_024
    MAX_POSITIONS: ClassVar[int] = 16_777_216

    def validate(self) -> None:
        def positive(name: str, limit: int) -> None:
            value = getattr(self, name)
            if not 0 < value <= limit:
                raise ConfigError(f"{name}={value} is outside (0, {limit}]")

        positive("vocab_size", self.MAX_VOCAB)
        positive("hidden_size", self.MAX_HIDDEN)
        positive("num_hidden_layers", self.MAX_LAYERS)
        positive("max_position_embeddings", self.MAX_POSITIONS)
        for eos in self.eos_token_ids:
            if not 0 <= eos < self.vocab_size:
                raise ConfigError(f"eos_token_id {eos} is outside the vocabulary")

    def to_json_dict(self) -> dict[str, Any]:
        raise NotImplementedError

    def save(self, folder: str | Path) -> None:
        path = Path(folder) / "config.json"
        path.write_text(json.dumps(self.to_json_dict(), indent=2, sort_keys=True) + "\n")


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """Qwen2 / Qwen2.5 dense decoder (python/instinct/backends/dense.py).

    ``use_sliding_window`` / ``max_window_layers`` / ``sliding_window`` choose the
    layers whose attention sees only the last ``sliding_window`` positions (the
    query's own included): when the flag is true these are the layers with index
    ``>= max_window_layers``. ``layer_types`` (``"full_attention"`` /
    ``"sliding_attention"`` per layer) overrides that rule when present.
    """

    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rope_theta: float = 0.0
    rms_norm_eps: float = 0.0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    layer_types: tuple[str, ...] = field(default_factory=tuple)

    MODEL_TYPE: ClassVar[str] = "qwen2"
    ARCHITECTURE: ClassVar[str] = "Qwen2ForCausalLM"

    @classmethod
    def from_json_dict(cls, raw: dict[str, Any]) -> "Qwen2Config":
        model_type = raw.get("model_type")
        if model_type is not None and model_type != cls.MODEL_TYPE:
            raise ConfigError(f"model_type {model_type!r} is not {cls.MODEL_TYPE!r}")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        # Newer checkpoints keep RoPE fields in ``rope_parameters``
        # (python/instinct/format.py:88-101).
        rope_theta = raw.get("rope_theta")
        if rope_theta is None:
            parameters = raw.get("rope_parameters")
            rope_theta = parameters.get("rope_theta") if isinstance(parameters, dict) else None
        if rope_theta is None:
            raise ConfigError("config.json is missing required key 'rope_theta'")
        # Scaled variants may sit under either key; both are refused rather than run unscaled.
        for key in ("rope_scaling", "rope_parameters"):
            scaling = raw.get(key)
            if scaling in (None, {}):
                continue
            if not isinstance(scaling, dict):
                raise ConfigError(f"config.json key '{key}' must be an object, got {scaling!r}")
            if (scaling.get("rope_type") or scaling.get("type")) not in (None, "default"):
                raise ConfigError(f"{key} {scaling!r} is not supported (only plain RoPE)")
        hidden = _take(raw, "hidden_size", int)
        heads = _take(raw, "num_attention_heads", int)
        head_dim = _take(raw, "head_dim", int, 0)
        if not head_dim:
            if heads <= 0 or hidden % heads:
                raise ConfigError(
                    f"hidden_size={hidden} is not a multiple of num_attention_heads={heads}"
                )
            head_dim = hidden // heads
        layer_types = raw.get("layer_types") or ()
        config = cls(
            architecture=(raw.get("architectures") or [cls.ARCHITECTURE])[0],
            vocab_size=_take(raw, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_take(raw, "num_hidden_layers", int),
            max_position_embeddings=_take(raw, "max_position_embeddings", int),
            eos_token_ids=eos_ids,
            intermediate_size=_take(raw, "intermediate_size", int),
            num_attention_heads=heads,
            num_key_value_heads=_take(raw, "num_key_value_heads", int),
            head_dim=head_dim,
            rope_theta=float(rope_theta),
            rms_norm_eps=_take(raw, "rms_norm_eps", float),
            tie_word_embeddings=_take(raw, "tie_word_embeddings", bool, False),
            hidden_act=_take(raw, "hidden_act", str, "silu"),
            use_sliding_window=_take(raw, "use_sliding_window", bool, False),
            sliding_window=_take(raw, "sliding_window", int, 0),
            max_window_layers=_take(raw, "max_window_layers", int, 0),
            layer_types=tuple(str(t) for t in layer_types),
        )
        config.validate()
        return config

    def validate(self) -> None:
        super().validate()
        if not 0 < self.intermediate_size <= self.MAX_INTERMEDIATE:
            raise ConfigError(f"intermediate_size={self.intermediate_size} is out of range")
        if self.num_attention_heads <= 0 or self.num_key_value_heads <= 0:
            raise ConfigError("head counts must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be positive and even")
        if not (math.isfinite(self.rope_theta) and self.rope_theta > 0):
            raise ConfigError(f"rope_theta={self.rope_theta} must be finite and positive")
        if not (math.isfinite(self.rms_norm_eps) and self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps={self.rms_norm_eps} must be finite and positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError("layer_types must name every layer")
            unknown = set(self.layer_types) - {"full_attention", "sliding_attention"}
            if unknown:
                raise ConfigError(f"unknown layer types {sorted(unknown)}")
        if any(self.layer_is_windowed(i) for i in range(self.num_hidden_layers)):
            if self.sliding_window <= 0:
                raise ConfigError("sliding-window layers need a positive sliding_window")
        if self.sliding_window < 0 or self.max_window_layers < 0:
            raise ConfigError("sliding_window and max_window_layers cannot be negative")

    def layer_is_windowed(self, layer: int) -> bool:
        if self.layer_types:
            return self.layer_types[layer] == "sliding_attention"
        return self.use_sliding_window and layer >= self.max_window_layers

    def layer_window(self, layer: int) -> int:
        """Window of ``layer`` in positions (the query's own included), 0 = all keys."""
        return self.sliding_window if self.layer_is_windowed(layer) else 0

    def to_json_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.MODEL_TYPE,
        }
        skip = {"architecture", "eos_token_ids", "layer_types"}
        for f in fields(self):
            if f.name not in skip:
                out[f.name] = getattr(self, f.name)
        if self.layer_types:
            out["layer_types"] = list(self.layer_types)
        if len(self.eos_token_ids) == 1:
            out["eos_token_id"] = self.eos_token_ids[0]
        elif self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def read_config_json(folder: str | Path) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {folder}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw
