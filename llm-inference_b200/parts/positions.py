"""Position encodings."""

from __future__ import annotations

import numpy as np
import torch

from . import ops
from .base import Part, register_part
from .context import CacheView, StepContext


class RotaryEncoding(Part):
    """Rotary position encoding over the first ``rotary_dims`` dims of each head, pairing
    dim i with i + rotary_dims / 2; inverse frequencies ``theta ** (-2 i / rotary_dims)`` are
    tabulated once in 32-bit and the kernel multiplies them by the position
    (python/instinct/backends/portable.py:115-132)."""

    def __init__(self, *, head_dim: int, theta: float, rotary_dims: int | None = None) -> None:
        self.head_dim = head_dim
        self.rotary_dims = head_dim if rotary_dims is None else rotary_dims
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= head_dim:
            raise ValueError(f"rotary_dims={self.rotary_dims} must be even and at most head_dim={head_dim}")
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def table(self) -> np.ndarray:
        half = self.rotary_dims // 2
        exponent = -(np.arange(half, dtype=np.float32) * np.float32(2.0) / np.float32(self.rotary_dims))
        return np.power(np.float32(self.theta), exponent, dtype=np.float32)

    def load(self, tensors, dtype, device) -> None:
        self.inv_freq = torch.from_numpy(self.table()).to(device)

    def apply(
        self,
        ctx: StepContext,
        cache: CacheView,
        qkv: torch.Tensor,
        bias: torch.Tensor | None,
        q_out: torch.Tensor,
        q_heads: int,
        kv_heads: int,
        head_dim: int,
    ) -> torch.Tensor:
        """The position part's one duty towards an attention mixer: take the step's projected
        rows ``qkv`` (``[tokens, (q_heads + 2 kv_heads) * head_dim]``, bias not yet added), add
        the bias, encode each token's position into its queries and keys, store keys and values
        in the token's page of ``cache`` (unless ``cache.writes`` is false) and the queries
        densely in ``q_out``. Here all of it is one kernel."""
        return ops.rope_kv_write(ctx, cache, qkv, bias, self.inv_freq, q_out, q_heads, kv_heads, head_dim)


register_part("position", "rotary", RotaryEncoding)
