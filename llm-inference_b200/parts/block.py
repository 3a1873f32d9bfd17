"""How one layer arranges its parts."""

from __future__ import annotations

import torch

from . import ops
from .base import Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class PreNormResidualBlock(Part):
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))``
    (python/instinct/backends/dense.py:89,104,122-129).

    The block receives the previous branch output still to be added (``delta``) so that each
    add runs inside the norm kernel that follows it, and returns its own last branch output
    the same way.

    Where the parts allow it (``takes_sink`` / ``takes_folded`` on the mixer and the
    feed-forward, ``foldable`` on the norms) and the step is short, a branch adds its output
    into the stream in its last product's epilogue and what travels on is
    :class:`ops.FoldedRows`: the norm that follows launches nothing. ``next_norm`` is the norm
    that will read this block's output (the next block's first norm, or the model's last)."""

    takes_next_norm = True

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

    def forward(self, ctx: StepContext, cache: CacheView | None, x: torch.Tensor, delta, next_norm: Part | None = None):
        mixer, ff = self.mixer, self.feed_forward
        h = self._norm(self.mixer_norm, ctx, x, delta, getattr(mixer, "takes_folded", False))
        # The mixer's and the feed-forward's outputs share one scratch buffer: the second norm
        # has consumed the former before the feed-forward's last product writes the latter.
        if getattr(mixer, "takes_sink", False) and getattr(self.feed_forward_norm, "foldable", False):
            a = mixer.forward(ctx, cache, h, sink=ops.ResidualSink(x, self.feed_forward_norm))
        else:
            a = mixer.forward(ctx, cache, h)
        h = self._norm(self.feed_forward_norm, ctx, x, a, getattr(ff, "takes_folded", False))
        if next_norm is not None and getattr(ff, "takes_sink", False) and getattr(next_norm, "foldable", False):
            return ff.forward(ctx, h, sink=ops.ResidualSink(x, next_norm))
        return ff.forward(ctx, h)

    @staticmethod
    def _norm(norm: Part, ctx: StepContext, x: torch.Tensor, delta, folded_ok: bool):
        if isinstance(delta, ops.FoldedRows):
            if getattr(norm, "foldable", False):
                return norm.forward(ctx, x, delta, folded_ok=folded_ok)
            return norm.forward(ctx, x, None)  # a norm that knows nothing of the folded form: the stream is current
        return norm.forward(ctx, x, delta)


register_part("block", "pre_norm_residual", PreNormResidualBlock)
