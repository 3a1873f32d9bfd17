"""Feed-forward parts."""

from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from . import ops
from .base import Part, register_part
from .context import StepContext


class SwiGLU(Part):
    """``down(silu(gate(h)) * up(h))`` without biases (python/instinct/backends/dense.py:124-128).
    The gate and up matrices are stored as one ``[2 * intermediate, hidden]`` matrix with their
    rows interleaved (row 2j is gate_j, row 2j + 1 is up_j), so one matrix product yields each
    gate next to its up value and the activation can run in that product's epilogue."""

    def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int) -> None:
        self.prefix, self.hidden_size, self.intermediate_size = prefix, hidden_size, intermediate_size
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> list[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(f"{p}gate_proj.weight", (i, h)),
            TensorSpec(f"{p}up_proj.weight", (i, h)),
            TensorSpec(f"{p}down_proj.weight", (h, i)),
        ]

    def load(self, tensors, dtype, device) -> None:
        p = self.prefix
        gate, up = (tensors[f"{p}{n}.weight"].to(device=device, dtype=dtype) for n in ("gate_proj", "up_proj"))
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size).contiguous()
        self.w_down = tensors[f"{p}down_proj.weight"].to(device=device, dtype=dtype).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    takes_folded = True  # `h` may be ops.FoldedRows: the gate/up product applies the norm's 1 / rms
    takes_sink = True  # with a sink the down product adds into the residual stream itself

    def forward(self, ctx: StepContext, h, sink: ops.ResidualSink | None = None):
        t, i = ctx.num_tokens, self.intermediate_size
        act = ctx.buffer("act", (t, i))
        if not ops.linear_swiglu(ctx, h, self.w_gate_up, act):
            gate_up = ops.linear(ctx, h, self.w_gate_up, ctx.buffer("gate_up", (t, 2 * i)))
            ops.silu_mul(ctx, gate_up, act)
        if sink is not None:
            folded = ops.linear_into_residual(ctx, act, self.w_down, sink)
            if folded is not None:
                return folded
        return ops.linear(ctx, act, self.w_down, ctx.buffer("branch", (t, self.hidden_size)))


register_part("feed_forward", "swiglu", SwiGLU)
