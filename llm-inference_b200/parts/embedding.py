"""Token embedding and the output head."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, register_part
from .context import StepContext


class TokenEmbedding(Part):
    """``x[t] = table[token[t]]`` widened to the 32-bit residual stream
    (python/instinct/backends/dense.py:82)."""

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int) -> None:
        self.name, self.vocab_size, self.hidden_size = name, vocab_size, hidden_size
        self.table: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + ".weight", (self.vocab_size, self.hidden_size))]

    def load(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name + ".weight"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return 0  # a step reads only its tokens' rows

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.buffer("residual", (ctx.num_tokens, self.hidden_size), torch.float32)
        return ops.embedding_gather(ctx, self.table, x)


class OutputHead(Part):
    """``logits = h W^T`` in 32-bit. With ``tied_to`` the matrix is the embedding table and
    the checkpoint need not hold a tensor of its own (python/instinct/export.py:38-41)."""

    def __init__(self, *, name: str, vocab_size: int, hidden_size: int, tied_to: str | None = None) -> None:
        self.name, self.vocab_size, self.hidden_size, self.tied_to = name, vocab_size, hidden_size, tied_to
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name + ".weight", (self.vocab_size, self.hidden_size), optional=self.tied_to is not None)]

    def load(self, tensors, dtype, device) -> None:
        own = tensors.get(self.name + ".weight")
        if own is None:
            own = tensors[self.tied_to + ".weight"]
        self.weight = own.to(device=device, dtype=dtype).contiguous()

    def share(self, embedding: TokenEmbedding) -> None:
        """Use the embedding's device tensor when both hold the same values."""
        if self.tied_to is not None and self.weight is not None and embedding.table is not None:
            if self.weight.shape == embedding.table.shape and torch.equal(self.weight, embedding.table):
                self.weight = embedding.table

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        logits = ctx.buffer("logits", (h.shape[0], self.vocab_size), torch.float32, per_token=False)
        return ops.linear(ctx, h, self.weight, logits)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", OutputHead)
