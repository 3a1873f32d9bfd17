"""Normalisation parts."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, register_part
from .context import StepContext


class RMSNorm(Part):
    """``y = v * rsqrt(mean(v^2) + eps) * weight`` with ``v = x + delta``, all in 32-bit
    (python/instinct/backends/portable.py:144-149). The add into the residual stream is
    part of the same kernel.

    In short bfloat16 steps the norm can disappear into the matrix products around it: the
    product before it adds its own output into the stream and hands over
    :class:`ops.FoldedRows` instead of a branch output; if the consumer says it takes that
    form (``folded_ok``) the norm passes it on and launches nothing."""

    foldable = True  # y = x * rsqrt(mean(x^2) + eps) * weight, nothing else: what the products' epilogues assume

    def __init__(self, *, name: str, hidden_size: int, eps: float) -> None:
        self.name, self.hidden_size, self.eps = name, hidden_size, float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + ".weight", (self.hidden_size,), init="one_plus_normal")]

    def load(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name + ".weight"].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * 4

    def forward(
        self,
        ctx: StepContext,
        x: torch.Tensor,
        delta: torch.Tensor | None,
        rows: torch.Tensor | None = None,
        out_name: str = "normed",
        folded_ok: bool = False,
    ) -> torch.Tensor:
        if isinstance(delta, ops.FoldedRows):
            # The stream is already up to date. Pass the folded form on if it was made for this
            # norm and the consumer takes it; otherwise normalise the stream here.
            if folded_ok and rows is None and delta.norm is self:
                return delta
            delta = None
        count = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer(out_name, (count, self.hidden_size), per_token=rows is None)
        return ops.rmsnorm(ctx, x, delta, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)
