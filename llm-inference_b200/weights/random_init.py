"""Seeded random weights, and a model folder written from a configuration and a seed.

Linear, embedding and bias tensors are N(0, std); norm scales are 1 + N(0, std).
Each tensor's stream depends only on (seed, tensor name), so any subset of a model
can be drawn alone. The reference draws test weights the same way, tensor by tensor
from one seeded generator (tests/test_mlx_engine.py:44-90).
"""

from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Iterable

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors

DEFAULT_STD = 0.02


def _stream_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 62) - 1)


def random_tensor(
    spec: TensorSpec,
    seed: int,
    *,
    std: float = DEFAULT_STD,
    dtype: torch.dtype = torch.bfloat16,
    device: torch.device | str = "cpu",
) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed(_stream_seed(seed, spec.name))
    if spec.integer:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    values = torch.empty(spec.shape, dtype=torch.float32, device=device)
    values.normal_(0.0, std, generator=generator)
    if spec.init == "one_plus_normal":
        values += 1.0
    elif spec.init != "normal":
        raise ValueError(f"unknown init {spec.init!r} for tensor '{spec.name}'")
    return values.to(dtype)


def random_weights(
    specs: Iterable[TensorSpec],
    seed: int,
    *,
    std: float = DEFAULT_STD,
    dtype: torch.dtype = torch.bfloat16,
    device: torch.device | str = "cpu",
    include_optional: bool = False,
) -> dict[str, torch.Tensor]:
    return {
        spec.name: random_tensor(spec, seed, std=std, dtype=dtype, device=device)
        for spec in specs
        if include_optional or not spec.optional
    }


def write_model_folder(
    folder: str | Path,
    config,
    seed: int,
    *,
    std: float = DEFAULT_STD,
    dtype: torch.dtype = torch.bfloat16,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded weights."""
    from ..config.registry import resolve_architecture

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_json_dict()
    recipe = resolve_architecture(raw).recipe(config)
    tensors = random_weights(recipe.tensor_specs(), seed, std=std, dtype=dtype)
    config.save(folder)
    write_safetensors(
        folder / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)}
    )
    return folder
