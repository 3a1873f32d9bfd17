"""Weights by tensor name, checked against what the model's parts expect.

Each part of a model lists the tensors it needs as :class:`TensorSpec`; the loader
reads exactly those names from a folder's ``*.safetensors`` and raises one
:class:`WeightsError` naming every missing tensor, every unexpected tensor and every
wrong shape (the reference checks names and shapes tensor by tensor:
python/instinct/model_contract.py:10-78, src/qwen_validation.cpp:11-46).

The loader changes no float's value: a tensor stored as float16, bfloat16 or float32 is handed
over in that format (64-bit floats become float32, integer tables int32), and the owning
part makes the one conversion to the dtype it computes in when it packs its weights. A
float32 engine therefore computes with exactly the stored float16 values, as the reference
widens its float16 tensors straight to the compute type
(python/instinct/backends/dense.py:36-48, storage format python/instinct/format.py:204-207);
for a bfloat16 engine rounding float16 to bfloat16 is the only possible choice, and it
happens once, in the part.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Iterable

import torch

from .safetensors_io import SafetensorsFile


class WeightsError(ValueError):
    def __init__(
        self,
        folder: str,
        missing: list[str],
        unexpected: list[str],
        wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
        wrong_kind: list[tuple[str, str]] = (),
    ) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = [f"weights in {folder} do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(
                f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected)
            )
        if self.wrong_shape:
            lines.append(
                f"  wrong shapes ({len(self.wrong_shape)}): "
                + ", ".join(
                    f"{name} is {list(found)}, expected {list(expected)}"
                    for name, found, expected in self.wrong_shape
                )
            )
        if self.wrong_kind:
            lines.append(
                f"  wrong dtypes ({len(self.wrong_kind)}): "
                + ", ".join(f"{name} is {found}" for name, found in self.wrong_kind)
            )
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs: its checkpoint name, shape and how to draw it at random."""

    name: str
    shape: tuple[int, ...]
    # "normal": N(0, std); "one_plus_normal": 1 + N(0, std) (norm scales).
    init: str = "normal"
    integer: bool = False
    # An optional tensor may be absent (a tied output head, for instance).
    optional: bool = False


def checkpoint_files(folder: str | Path) -> list[Path]:
    files = sorted(Path(folder).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors in {folder}")
    return files


def _stored_to_kept(tensor: torch.Tensor, spec: TensorSpec) -> torch.Tensor:
    if spec.integer:
        return tensor.to(torch.int32)
    if tensor.dtype in (torch.float16, torch.bfloat16, torch.float32):
        return tensor
    return tensor.to(torch.float32)


def load_weights(
    folder: str | Path, specs: Iterable[TensorSpec], device: torch.device | str = "cpu"
) -> dict[str, torch.Tensor]:
    """Read the tensors named by ``specs``; raise one error for every mismatch."""
    wanted = {spec.name: spec for spec in specs}
    files = [SafetensorsFile(path) for path in checkpoint_files(folder)]
    try:
        where: dict[str, tuple[SafetensorsFile, str]] = {}
        for file in files:
            for stored in file.tensors:
                where[stored.removeprefix("language_model.")] = (file, stored)
        missing = [n for n, s in wanted.items() if n not in where and not s.optional]
        unexpected = sorted(n for n in where if n not in wanted)
        wrong_shape = []
        wrong_kind = []
        for name, spec in wanted.items():
            if name not in where:
                continue
            file, stored = where[name]
            info = file.tensors[stored]
            if info.shape != tuple(spec.shape):
                wrong_shape.append((name, info.shape, tuple(spec.shape)))
            if info.dtype.is_floating_point == spec.integer:
                wrong_kind.append((name, str(info.dtype).removeprefix("torch.")))
        if missing or unexpected or wrong_shape or wrong_kind:
            raise WeightsError(str(folder), missing, unexpected, wrong_shape, wrong_kind)
        out = {}
        for name, spec in wanted.items():
            if name in where:
                file, stored = where[name]
                out[name] = _stored_to_kept(file.read(stored), spec).to(device)
        return out
    finally:
        for file in files:
            file.close()
