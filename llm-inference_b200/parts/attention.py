"""The attention mixer: projections, rotary encoding, cache write and attention over the cache."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import KVCacheSpec, Part, PartSpec, build_part, register_part
from .context import CacheView, StepContext


class GroupedQueryAttention(Part):
    """Causal grouped-query attention over a paged cache.

    ``q = h Wq^T + bq`` and likewise k, v; q and k are rotated at the token's position; k and
    v go to the token's page; each query head attends, through ``softmax(q k^T * scale)``,
    to the keys of its kv head at positions no later than its own and, with a window, no
    earlier than ``position - window + 1``; the heads' outputs go through ``Wo`` without bias
    (python/instinct/backends/dense.py:88-104). The three input projections are stored as one
    ``[(q_heads + 2 kv_heads) * head_dim, hidden]`` matrix so they are one matrix product.
    """

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        q_heads: int,
        kv_heads: int,
        head_dim: int,
        position: PartSpec,
        qkv_bias: bool = True,
        window: int = 0,
        scale: float | None = None,
    ) -> None:
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads cannot share {kv_heads} kv heads")
        if head_dim % 16:
            raise ValueError(f"head_dim={head_dim} must be a multiple of 16 for the attention kernels")
        self.prefix = prefix
        self.hidden_size, self.q_heads, self.kv_heads, self.head_dim = hidden_size, q_heads, kv_heads, head_dim
        self.qkv_bias, self.window = qkv_bias, int(window)
        self.scale = float(scale) if scale is not None else head_dim**-0.5
        self.position = build_part("position", position)
        self.graph_safe = self.position.graph_safe
        self.w_qkv = self.b_qkv = self.w_o = None

    def cache_spec(self) -> KVCacheSpec:
        return KVCacheSpec(self.kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, h = self.prefix, self.head_dim, self.hidden_size
        specs = []
        for name, heads in (("q_proj", self.q_heads), ("k_proj", self.kv_heads), ("v_proj", self.kv_heads)):
            specs.append(TensorSpec(f"{p}{name}.weight", (heads * d, h)))
            if self.qkv_bias:
                specs.append(TensorSpec(f"{p}{name}.bias", (heads * d,)))
        specs.append(TensorSpec(f"{p}o_proj.weight", (h, self.q_heads * d)))
        return specs + self.position.tensor_specs()

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        names = ("q_proj", "k_proj", "v_proj")
        self.w_qkv = torch.cat([tensors[f"{p}{n}.weight"].to(device=device, dtype=dtype) for n in names]).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat(
                [tensors[f"{p}{n}.bias"].to(device=device, dtype=torch.float32) for n in names]
            ).contiguous()
        self.w_o = tensors[f"{p}o_proj.weight"].to(device=device, dtype=dtype).contiguous()
        self.position.load(tensors, dtype, device)

    def weight_bytes(self) -> int:
        total = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        return total + (self.b_qkv.numel() * 4 if self.b_qkv is not None else 0)

    takes_folded = True  # `h` may be ops.FoldedRows: the q/k/v product applies the norm's 1 / rms
    takes_sink = True  # with a sink the output product adds into the residual stream itself

    def forward(self, ctx: StepContext, cache: CacheView, h, sink: ops.ResidualSink | None = None):
        t = ctx.num_tokens
        width = (self.q_heads + 2 * self.kv_heads) * self.head_dim
        qkv = ops.linear(ctx, h, self.w_qkv, ctx.buffer("qkv", (t, width)))
        q = ctx.buffer("q", (t, self.q_heads * self.head_dim))
        # Bias, position encoding and the cache write are the position part's: the mixer does not
        # know how positions are encoded.
        self.position.apply(ctx, cache, qkv, self.b_qkv, q, self.q_heads, self.kv_heads, self.head_dim)
        attn = ctx.buffer("attn", (t, self.q_heads * self.head_dim))
        self.attend(ctx, cache, q, attn)
        if sink is not None:
            folded = ops.linear_into_residual(ctx, attn, self.w_o, sink)
            if folded is not None:
                return folded
        return ops.linear(ctx, attn, self.w_o, ctx.buffer("branch", (t, self.hidden_size)))

    def attend(self, ctx: StepContext, cache: CacheView, q: torch.Tensor, out: torch.Tensor) -> None:
        from . import attention_dispatch

        attention_dispatch.attend(ctx, cache, q, out, self.q_heads, self.kv_heads, self.head_dim, self.scale)


register_part("mixer", "gqa_attention", GroupedQueryAttention)
