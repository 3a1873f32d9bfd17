"""How one layer arranges its parts."""

from __future__ import annotations

import torch

from .base import Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class PreNormResidualBlock(Part):
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))``
    (python/instinct/backends/dense.py:89,104,122-129).

    The block receives the previous branch output still to be added (``delta``) so that each
    add runs inside the norm kernel that follows it, and returns its own last branch output
    the same way."""

    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec, feed_forward_norm: PartSpec) -> None:
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer = build_part("mixer", mixer)
        self.feed_forward_norm = build_part("norm", feed_forward_norm)
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.parts = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)
        self.graph_safe = all(p.graph_safe for p in self.parts)

    def tensor_specs(self):
        return [spec for part in self.parts for spec in part.tensor_specs()]

    def load(self, tensors, dtype, device) -> None:
        for part in self.parts:
            part.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(part.weight_bytes() for part in self.parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta: torch.Tensor | None) -> torch.Tensor:
        h = self.mixer_norm.forward(ctx, x, delta)
        # The mixer's and the feed-forward's outputs share one scratch buffer: the second norm
        # has consumed the former before the feed-forward's last product writes the latter.
        a = self.mixer.forward(ctx, cache, h)
        h = self.feed_forward_norm.forward(ctx, x, a)
        return self.feed_forward.forward(ctx, h)


register_part("block", "pre_norm_residual", PreNormResidualBlock)
