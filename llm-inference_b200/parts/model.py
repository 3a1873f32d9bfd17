"""A model as data (:class:`ModelRecipe`) and the object built from it (:class:`Model`)."""

from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any

import torch

from ..weights.loader import TensorSpec
from .base import KVCacheSpec, PartSpec, StateSpec, build_part
from .context import CacheView, StepContext


@contextmanager
def _nvtx_range(name: str):
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


@contextmanager
def _no_range(name: str):
    yield


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run ``layer`` against cache entry ``cache``.

    By default a layer owns the cache entry with its own index. Naming another entry with
    ``writes=False`` lets the layer read what that entry's owner wrote this step; naming a
    layer twice runs it twice (give the second call a cache entry of its own)."""

    layer: int
    cache: int | None = None
    writes: bool = True

    @property
    def cache_id(self) -> int:
        return self.layer if self.cache is None else self.cache


@dataclass
class ModelRecipe:
    """Everything needed to build a model; produced from a configuration by the
    architecture's recipe function."""

    config: Any
    embedding: PartSpec
    layers: list[PartSpec]  # one block spec per layer
    final_norm: PartSpec
    head: PartSpec
    schedule: list[LayerCall] = field(default_factory=list)

    def __post_init__(self) -> None:
        if not self.schedule:
            self.schedule = [LayerCall(i) for i in range(len(self.layers))]

    def build_parts(self) -> "Model":
        return Model(self)

    def tensor_specs(self) -> list[TensorSpec]:
        return Model(self).tensor_specs()


class Model:
    def __init__(self, recipe: ModelRecipe) -> None:
        self.recipe = recipe
        self.config = recipe.config
        self.embedding = build_part("embedding", recipe.embedding)
        self.blocks = [build_part("block", spec) for spec in recipe.layers]
        self.final_norm = build_part("norm", recipe.final_norm)
        self.head = build_part("head", recipe.head)
        self.schedule = list(recipe.schedule)
        for call in self.schedule:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"the run order names layer {call.layer}, which does not exist")
        self.dtype: torch.dtype | None = None
        self.device: torch.device | None = None
        self.graph_safe = all(
            p.graph_safe for p in (self.embedding, *self.blocks, self.final_norm, self.head)
        )

    # -- weights ---------------------------------------------------------------------------

    def tensor_specs(self) -> list[TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            for spec in part.tensor_specs():
                if spec.name in specs and specs[spec.name].shape != spec.shape:
                    raise ValueError(f"two parts want tensor '{spec.name}' with different shapes")
                # A tensor one part requires stays required even if another calls it optional.
                if spec.name not in specs or specs[spec.name].optional:
                    specs[spec.name] = spec
        return list(specs.values())

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device | str) -> None:
        device = torch.device(device)
        self.dtype, self.device = dtype, device
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            part.load(tensors, dtype, device)
        if hasattr(self.head, "share"):
            self.head.share(self.embedding)

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads: every layer call's weights, the last norm, the head."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes() + self.embedding.weight_bytes()
        return total + sum(self.blocks[call.layer].weight_bytes() for call in self.schedule)

    # -- cache requirements ----------------------------------------------------------------

    def cache_specs(self) -> dict[int, KVCacheSpec | StateSpec]:
        """Cache entry id -> what its owner (the call that writes it) needs."""
        specs: dict[int, KVCacheSpec | StateSpec] = {}
        for call in self.schedule:
            spec = self.blocks[call.layer].cache_spec()
            if spec is None:
                continue
            if call.writes:
                if call.cache_id in specs and specs[call.cache_id] != spec:
                    raise ValueError(f"cache entry {call.cache_id} is written with two different shapes")
                specs[call.cache_id] = spec
        for call in self.schedule:
            spec = self.blocks[call.layer].cache_spec()
            if spec is not None and not call.writes and call.cache_id not in specs:
                raise ValueError(f"layer {call.layer} reads cache entry {call.cache_id}, which nobody writes")
        return specs

    # -- the forward pass of one step --------------------------------------------------------

    def forward(self, ctx: StepContext, cache_views) -> torch.Tensor:
        """Run the step's tokens through every layer call; return 32-bit logits of
        ``ctx.logit_rows`` as ``[wanted, vocab]``. ``cache_views(call)`` yields the call's
        :class:`CacheView`."""
        # With options["nvtx"] every layer call and the head get a named range, as the reference
        # marks them (cuda/qwen_model.cu:106,138,169); the ranges are host-side marks around the
        # launches and change nothing on the device.
        mark = _nvtx_range if ctx.options.get("nvtx") else _no_range
        # A step of single tokens of a model made of the stock parts can run as one resident
        # kernel (parts/resident.py) instead of the chain of kernels below.
        resident = ctx.options.get("resident")
        if resident is not None and resident.takes(ctx):
            with mark("resident step"):
                return resident.run(ctx, cache_views)
        x = self.embedding.forward(ctx)
        delta = None
        for index, call in enumerate(self.schedule):
            block = self.blocks[call.layer]
            view: CacheView | None = cache_views(call) if block.cache_spec() is not None else None
            with mark(f"layer {call.layer}"):
                if getattr(block, "takes_next_norm", False):
                    # The norm that reads this block's output: a block that adds its last branch
                    # into the stream by itself folds that norm's scale into what it hands on.
                    following = self.schedule[index + 1].layer if index + 1 < len(self.schedule) else None
                    next_norm = getattr(self.blocks[following], "mixer_norm", None) if following is not None else self.final_norm
                    delta = block.forward(ctx, view, x, delta, next_norm=next_norm)
                else:
                    delta = block.forward(ctx, view, x, delta)
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.head.vocab_size), dtype=torch.float32, device=ctx.device)
        with mark("head"):
            if not isinstance(delta, torch.Tensor) and delta is not None and not getattr(self.final_norm, "foldable", False):
                delta = None  # the stream is current; this norm knows nothing of the folded form
            h = self.final_norm.forward(ctx, x, delta, rows=ctx.logit_rows, out_name="normed_rows")
            return self.head.forward(ctx, h)
