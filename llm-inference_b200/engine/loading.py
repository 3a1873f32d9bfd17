"""From a model folder (or a configuration and a seed) to a model with weights on the device."""

from __future__ import annotations

from pathlib import Path

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.model_config import ModelConfig, read_config_json
from ..config.registry import parse_config, resolve_architecture
from ..parts.model import Model
from ..weights.loader import load_weights
from ..weights.random_init import random_weights

DTYPES = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
    "f32": torch.float32,
}


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; use 'bfloat16' or 'float32'") from None


def load_model(model_path: str | Path, dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda:0") -> Model:
    """Build the model that ``config.json`` names and load its safetensors weights."""
    compute_dtype = parse_dtype(dtype)
    folder = Path(model_path)
    if not folder.is_dir():
        raise FileNotFoundError(f"{folder} is not a model folder (config.json plus *.safetensors)")
    entry, config = parse_config(read_config_json(folder))
    model = Model(entry.recipe(config))
    tensors = load_weights(folder, model.tensor_specs(), device="cpu")
    model.load(tensors, compute_dtype, torch.device(device))
    return model


def random_model(
    config: ModelConfig,
    seed: int,
    dtype: str | torch.dtype = "bfloat16",
    device: str | torch.device = "cuda:0",
    *,
    std: float = 0.02,
) -> Model:
    """A model with seeded random weights drawn straight on the device (nothing is written)."""
    entry = resolve_architecture(config.to_json_dict())
    model = Model(entry.recipe(config))
    dt = parse_dtype(dtype)
    tensors = random_weights(model.tensor_specs(), seed, std=std, dtype=torch.bfloat16, device=device)
    model.load(tensors, dt, torch.device(device))
    return model
