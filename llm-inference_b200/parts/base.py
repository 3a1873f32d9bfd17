"""Interfaces of the parts a model is put together from, and the table that names them.

A model is data: a :class:`ModelRecipe` lists, layer by layer, which mixer, feed-forward and
norm to build and with which sizes and constants, and in which order the layers run. Parts
never see a model configuration; they get their parameters as keyword arguments, say which
tensors they need and what cache they want, and compute on a :class:`StepContext`.

Kinds of part and what each must provide:

``norm``          ``forward(ctx, x, delta, rows=None) -> Tensor``: adds the pending branch
                  output ``delta`` into the 32-bit residual stream ``x`` and returns the
                  normalised rows in the compute dtype (only ``rows`` if given, without
                  touching ``x``).
``position``      owned by an attention mixer:
                  ``apply(ctx, cache, qkv, bias, q_out, q_heads, kv_heads, head_dim)`` adds the
                  projection bias, encodes each token's position into its queries and keys,
                  writes keys and values to the token's page and the queries to ``q_out``; the
                  mixer never looks inside (the rotary part does it in one fused kernel).
``mixer``         ``cache_spec() -> KVCacheSpec | StateSpec | None`` and
                  ``forward(ctx, cache, h) -> Tensor`` where ``cache`` is the
                  :class:`CacheView` of the layer call.
``feed_forward``  ``forward(ctx, h) -> Tensor``.
``embedding``     ``forward(ctx) -> Tensor`` (the 32-bit residual stream of the new tokens).
``head``          ``forward(ctx, h) -> Tensor`` (32-bit logits of the given rows).
``block``         ``forward(ctx, cache, x, delta) -> Tensor``: one layer's arrangement of the
                  parts above; returns the branch output still to be added to ``x``.

Every part also has ``tensor_specs() -> list[TensorSpec]`` and ``load(tensors, dtype, device)``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class KVCacheSpec:
    """Paged keys and values: ``window`` 0 keeps every position, else the last ``window``."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state: one array of each shape per request slot."""

    shapes: tuple[tuple[int, ...], ...]
    dtypes: tuple[torch.dtype, ...]


@dataclass(frozen=True)
class PartSpec:
    """Which registered part to build, and the parameters it is built with."""

    name: str
    params: dict[str, Any] = field(default_factory=dict)


class Part:
    """Base of every part: owns its weights, knows their checkpoint names and shapes."""

    graph_safe = True  # may be captured in a CUDA graph (no host reads, no allocation)

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        del tensors, dtype, device

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (each tensor counted once)."""
        return 0


_PARTS: dict[tuple[str, str], Callable[..., Part]] = {}
KINDS = ("norm", "position", "mixer", "feed_forward", "embedding", "head", "block")


def register_part(kind: str, name: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if kind not in KINDS:
        raise ValueError(f"unknown kind of part '{kind}' (kinds: {', '.join(KINDS)})")
    if (kind, name) in _PARTS and not replace:
        raise ValueError(f"{kind} '{name}' is already registered")
    _PARTS[(kind, name)] = factory


def build_part(kind: str, spec: PartSpec, **extra: Any) -> Part:
    try:
        factory = _PARTS[(kind, spec.name)]
    except KeyError:
        known = sorted(n for k, n in _PARTS if k == kind)
        raise ValueError(f"no {kind} named '{spec.name}' is registered (known: {known})") from None
    return factory(**spec.params, **extra)


def registered_parts(kind: str) -> tuple[str, ...]:
    return tuple(sorted(n for k, n in _PARTS if k == kind))
