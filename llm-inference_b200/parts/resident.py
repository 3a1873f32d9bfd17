"""A whole decode step as one resident kernel (``csrc/kernels/resident_decode.cu``).

A model that is put together from the stock parts in the stock arrangement (token embedding;
blocks of RMSNorm, grouped-query attention with rotary encoding over heads of 128, RMSNorm,
SwiGLU; last RMSNorm; linear head), in bfloat16, can run a step in which every request feeds
one token, up to 16 of them, as a single kernel launch instead of some nine launches per
layer. This module decides whether a model qualifies, turns its parts into the kernel's list
of phases once per batch-size bucket, and launches the step. Everything else (prompt
portions, larger batches, other parts, float32) keeps the chain of kernels in ``Model.forward``;
both paths compute the same formulas and are tested against the same plain implementation.

It is an option (``decode_kernel="resident"``), not the default: measured on a B200 at the
Qwen2.5-1.5B sizes with 8 requests of 2,048 keys it takes 2.77 ms per step where the chain of
kernels takes 1.24 ms. Every phase costs its slowest block some ten dependent trips to L2
(barrier, operand fetch, partial sums through scratch, arrival counter, the last arriver's
reduction, epilogue), about 14 to 20 microseconds, whatever the phase streams; the chain's
kernels pay the like of it once per kernel but overlap their neighbours.
"""

from __future__ import annotations

import struct
from ctypes import byref, c_float, c_int, c_int64, c_longlong, c_void_p

import numpy as np
import torch

from ..csrc.library import KernelError, ptr
from .attention import GroupedQueryAttention
from .block import PreNormResidualBlock
from .context import StepContext
from .embedding import OutputHead, TokenEmbedding
from .feed_forward import SwiGLU
from .norms import RMSNorm
from .positions import RotaryEncoding

PH_EMBED, PH_GEMM, PH_ATTN = 0, 1, 2
X_NORM, X_ACT, X_MERGE = 0, 1, 2
E_QKV_ROPE, E_RESIDUAL, E_SWIGLU, E_LOGITS = 0, 1, 2, 3
MAX_SPLITS = 16


def _float_bits(value: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(value)))[0]


class ResidentDecoder:
    """The resident-kernel path of one model over one cache."""

    def __init__(self, model, cache, lib) -> None:
        self.model, self.cache, self.lib = model, cache, lib
        api = lib.lib
        api.b200_resident_supported.argtypes = [c_int] * 8
        api.b200_resident_supported.restype = c_int
        api.b200_resident_scratch.argtypes = [c_int, c_int, c_void_p, c_void_p]
        api.b200_resident_scratch.restype = None
        for name in ("b200_resident_phase_bytes", "b200_resident_phase_fields", "b200_resident_max_tokens", "b200_resident_blocks"):
            getattr(api, name).restype = c_int
        lib.bind("b200_resident_build", [c_void_p, c_int, c_void_p, c_void_p])
        lib.bind(
            "b200_resident_decode",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float] + [c_void_p] * 16,
        )
        self.blocks = int(api.b200_resident_blocks())
        self.max_tokens = int(api.b200_resident_max_tokens())
        self.phase_bytes = int(api.b200_resident_phase_bytes())
        self.phase_fields = int(api.b200_resident_phase_fields())
        first = model.blocks[0].mixer
        self.hidden = first.hidden_size
        self.q_heads, self.kv_heads, self.scale = first.q_heads, first.kv_heads, first.scale
        self.intermediate = model.blocks[0].feed_forward.intermediate_size
        self.vocab = model.head.vocab_size
        self._plans: dict[tuple, torch.Tensor] = {}
        self._phases = 2 + 5 * len(model.schedule)  # embedding, five per layer call, output head

    # -- whether a model qualifies --------------------------------------------------------------------

    @classmethod
    def for_model(cls, model, cache, lib) -> "ResidentDecoder | None":
        """The resident path for this model, or None if any part, size or dtype is not one the
        kernel was written for."""
        if model.dtype != torch.bfloat16 or cache.state_specs or not cache.groups:
            return None
        if type(model.embedding) is not TokenEmbedding or type(model.head) is not OutputHead or type(model.final_norm) is not RMSNorm:
            return None
        if not model.blocks or model.embedding.table.dtype != torch.bfloat16:
            return None
        seen_entries = set()
        for call in model.schedule:
            if not call.writes or call.cache_id in seen_entries:
                return None  # a call that only reads another call's cache
            seen_entries.add(call.cache_id)
        first = model.blocks[0]
        for block in model.blocks:
            if type(block) is not PreNormResidualBlock:
                return None
            mixer, ff = block.mixer, block.feed_forward
            if type(mixer) is not GroupedQueryAttention or type(ff) is not SwiGLU:
                return None
            if type(block.mixer_norm) is not RMSNorm or type(block.feed_forward_norm) is not RMSNorm:
                return None
            position = mixer.position
            if not isinstance(position, RotaryEncoding) or type(position).apply is not RotaryEncoding.apply:
                return None
            if position.rotary_dims != mixer.head_dim or mixer.head_dim != 128:
                return None
            same = (
                mixer.hidden_size == first.mixer.hidden_size and mixer.q_heads == first.mixer.q_heads
                and mixer.kv_heads == first.mixer.kv_heads and mixer.scale == first.mixer.scale
                and ff.intermediate_size == first.feed_forward.intermediate_size
                and torch.equal(position.inv_freq, first.mixer.position.inv_freq)
            )
            if not same:
                return None
        decoder = cls(model, cache, lib)
        ok = lib.lib.b200_resident_supported(
            decoder.hidden, decoder.intermediate, decoder.q_heads, decoder.kv_heads, 128, decoder.vocab,
            cache.page_size, decoder.blocks,
        )
        return decoder if ok else None

    def takes(self, ctx: StepContext) -> bool:
        """Whether this step can run as the resident kernel: single tokens only, few enough."""
        options = ctx.options
        return (
            ctx.num_tokens == ctx.num_seqs == ctx.num_decode_seqs
            and 0 < ctx.num_tokens <= self.max_tokens
            and options.get("decode_kernel", "chain") == "resident"
            # A caller that forces one of the chain's kernels gets the chain.
            and all(options.get(name, "auto") == "auto" for name in ("attention", "gemm", "decode_loader"))
            and not options.get("decode_splits")
        )

    # -- the plan: the model's parts as the kernel's phases ------------------------------------------

    def _plan(self, ctx: StepContext, cache_views, buffers: dict[str, torch.Tensor]) -> torch.Tensor:
        model = self.model
        views = [cache_views(call) for call in model.schedule]
        # Everything a plan holds an address of: the step's scratch (moves only when the workspace
        # grows) and the block tables (their place in the metadata buffer depends on the step's shape).
        key = (ctx.num_tokens, ctx.workspace.generation, tuple(view.block_table.data_ptr() for view in views))
        plan = self._plans.get(key)
        if plan is not None:
            return plan
        rows: list[list[int]] = []

        def phase(kind, xkind=0, ekind=0, n=0, k=0, w=None, norm=None, eps=0.0, bias=None, keys=None, values=None,
                  table=None, arena_rows=0, window=0, out=None, pages=0, operand=None):
            address = lambda t: 0 if t is None else t.data_ptr()
            rows.append([
                kind, xkind, ekind, n, k, address(w), address(norm), _float_bits(eps), address(bias), address(keys),
                address(values), address(table), arena_rows, window, address(out), pages, address(operand), 0,
            ])

        # Every product that follows a norm takes `xn` as its operand: the residual stream times that
        # norm's scale, written by whoever produced the stream (the embedding, or the product whose
        # epilogue added into it), which therefore carries the scale of the norm that FOLLOWS it; the
        # token's 1 / rms is applied in the consuming product's epilogue.
        xn, act = buffers["xn"], buffers["act"]
        calls = list(zip(model.schedule, views))
        norms_after = [model.blocks[call.layer].mixer_norm for call, _ in calls[1:]] + [model.final_norm]
        phase(PH_EMBED, norm=model.blocks[calls[0][0].layer].mixer_norm.weight, out=model.embedding.table)
        for (call, view), next_norm in zip(calls, norms_after):
            block = model.blocks[call.layer]
            mixer, ff = block.mixer, block.feed_forward
            arena_rows = view.keys.shape[0] * view.keys.shape[1] * view.keys.shape[2]
            if not (view.keys.is_contiguous() and view.values.is_contiguous() and view.block_table.is_contiguous()):
                raise KernelError("resident decode: the cache arenas and block tables must be contiguous")
            phase(PH_GEMM, X_NORM, E_QKV_ROPE, mixer.w_qkv.shape[0], self.hidden, mixer.w_qkv, eps=block.mixer_norm.eps,
                  bias=mixer.b_qkv, keys=view.keys, values=view.values, table=view.block_table, pages=view.num_pages,
                  operand=xn)
            phase(PH_ATTN, keys=view.keys, values=view.values, table=view.block_table, arena_rows=arena_rows,
                  window=view.window, pages=view.num_pages)
            phase(PH_GEMM, X_MERGE, E_RESIDUAL, self.hidden, mixer.w_o.shape[1], mixer.w_o, norm=block.feed_forward_norm.weight)
            phase(PH_GEMM, X_NORM, E_SWIGLU, ff.w_gate_up.shape[0], self.hidden, ff.w_gate_up,
                  eps=block.feed_forward_norm.eps, out=act, operand=xn)
            phase(PH_GEMM, X_ACT, E_RESIDUAL, self.hidden, self.intermediate, ff.w_down, norm=next_norm.weight, operand=act)
        phase(PH_GEMM, X_NORM, E_LOGITS, self.vocab, self.hidden, model.head.weight, eps=model.final_norm.eps,
              out=buffers["logits"], operand=xn)
        fields = np.asarray(rows, dtype=np.int64)
        assert fields.shape[1] == self.phase_fields
        plan = torch.empty(len(rows) * self.phase_bytes, dtype=torch.uint8, device=ctx.device)
        self.lib.call("b200_resident_build", c_void_p(fields.ctypes.data), c_int(len(rows)), ptr(plan), ctx.stream)
        if len(self._plans) > 64:
            self._plans.clear()
        self._plans[key] = plan
        return plan

    # -- one step ---------------------------------------------------------------------------------------

    def run(self, ctx: StepContext, cache_views) -> torch.Tensor:
        """Runs the step; returns 32-bit logits of ``ctx.logit_rows``."""
        t = ctx.num_tokens
        splits = max(1, min(MAX_SPLITS, self.blocks // (t * self.kv_heads)))
        rows = self.max_tokens
        floats, counters = c_longlong(0), c_int(0)
        largest = max(self.vocab, 2 * self.intermediate, (self.q_heads + 2 * self.kv_heads) * 128, self.hidden)
        self.lib.lib.b200_resident_scratch(largest, self.blocks, byref(floats), byref(counters))
        f32, bf16 = torch.float32, torch.bfloat16
        buffers = {
            "x": ctx.buffer("resident_x", (rows, self.hidden), f32, per_token=False),
            "xn": ctx.buffer("resident_xn", (rows, self.hidden), bf16, per_token=False),
            "ss": ctx.buffer("resident_ss", (self.hidden // 32, rows), f32, per_token=False),
            "q": ctx.buffer("resident_q", (rows, self.q_heads * 128), bf16, per_token=False),
            "part_o": ctx.buffer("resident_part_o", (rows * self.q_heads * MAX_SPLITS, 128), f32, per_token=False),
            "part_ml": ctx.buffer("resident_part_ml", (rows * self.q_heads * MAX_SPLITS, 2), f32, per_token=False),
            "act": ctx.buffer("resident_act", (rows, self.intermediate), bf16, per_token=False),
            "scratch": ctx.buffer("resident_scratch", (floats.value,), f32, per_token=False),
            "logits": ctx.buffer("resident_logits", (rows, self.vocab), f32, per_token=False),
        }
        counter_buf = ctx.workspace.zeros("resident_counters", max(counters.value, 4096), torch.int32)
        bar = ctx.workspace.zeros("resident_barrier", 64, torch.int32)
        plan = self._plan(ctx, cache_views, buffers)
        first = self.model.blocks[0].mixer
        self.lib.call(
            "b200_resident_decode", ptr(plan), c_int(self._phases), c_int(t), c_int(self.hidden), c_int(self.q_heads),
            c_int(self.kv_heads), c_int(self.cache.page_size), c_int(self.cache.max_pages_per_request), c_int(self.vocab),
            c_int(splits), c_float(self.scale), ptr(first.position.inv_freq), ptr(ctx.token_ids), ptr(ctx.positions),
            ptr(ctx.seq_kv_len), ptr(buffers["x"]), ptr(buffers["xn"]), ptr(buffers["ss"]), ptr(buffers["q"]), ptr(buffers["part_o"]),
            ptr(buffers["part_ml"]), ptr(buffers["scratch"]), ptr(counter_buf), ptr(bar), ptr(ctx.err),
            ptr(ctx.options.get("resident_trace")), ctx.stream,
        )
        logits = buffers["logits"]
        wanted = ctx.host.logit_rows
        if wanted.shape[0] == t and bool((wanted == np.arange(t, dtype=wanted.dtype)).all()):
            return logits[:t]
        return logits.index_select(0, ctx.logit_rows.long())
