"""Chooses the attention kernel for a step.

In bfloat16, with a head size and page size the tensor-core kernels take, the step's
single-token requests (which lead the batch) go to a split-key decode kernel (mma.sync; keys
and values by TMA when head_dim is 128 and pages hold 64 rows or more, by cp.async otherwise) and
the prompt portions to the tcgen05 / TMEM kernel (head_dim 128, pages of at least 16 rows) or
else to the mma.sync prefill form. Everything else - float32, other head sizes, pages whose
size is no power of two - runs the plain kernel, which takes every shape.
``options["attention"]``: ``"auto"``, ``"plain"``, ``"flash"`` (mma.sync only) or
``"tcgen05"`` (refuse shapes the tcgen05 kernel does not take).
"""

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
    choice = ctx.options.get("attention", "auto")
    tuned = (
        choice != "plain"
        and q.dtype == torch.bfloat16
        and ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, cache.page_size, decode=False)
    )
    if not tuned:
        if choice in ("flash", "tcgen05"):
            raise ops.KernelError("the tensor-core attention kernels do not take this shape or dtype")
        ops.paged_attention_plain(ctx, cache, q, out, q_heads, kv_heads, head_dim, scale)
        return
    decode_seqs = ctx.num_decode_seqs
    if decode_seqs and not ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, cache.page_size, decode=True):
        decode_seqs = 0  # more than 16 query heads per kv head: the prefill form handles one-token runs too
    if decode_seqs:
        reach = ctx.max_kv_len if not cache.window else min(ctx.max_kv_len, cache.window + 64)
        tma = ops.decode_uses_tma(ctx, decode_seqs, q_heads, kv_heads, head_dim, cache.page_size)
        splits = int(ctx.options.get("decode_splits", 0)) or ops.decode_splits(decode_seqs, kv_heads, reach, tma, ops.sm_count(ctx))
        ops.paged_flash_attention(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=0, num_seqs=decode_seqs, decode=True, max_q_len=1, splits=splits,
        )
    if ctx.num_seqs > decode_seqs and choice in ("auto", "tcgen05") and ops.prefill_tcgen05_supported(
        ctx, q_heads, kv_heads, head_dim, cache.page_size, ctx.max_kv_len
    ):
        ops.paged_prefill_attention_tcgen05(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=decode_seqs, num_seqs=ctx.num_seqs - decode_seqs, max_q_len=ctx.max_q_len,
        )
    elif ctx.num_seqs > decode_seqs:
        if choice == "tcgen05":
            raise ops.KernelError("the tcgen05 attention kernel does not take this shape")
        ops.paged_flash_attention(
            ctx, cache, q, out, q_heads, kv_heads, head_dim, scale,
            first_seq=decode_seqs, num_seqs=ctx.num_seqs - decode_seqs, decode=False, max_q_len=ctx.max_q_len,
        )
