"""Tensor-level calls into the kernel library (and the library matrix product).

Each function checks shapes and strides, then launches on the current CUDA stream. Matrix
products in bfloat16 go to the vendor library through ``torch.mm``, as the reference sends
its linear layers to cuBLASLt (cuda/execution_context.cu:95-110); in float32 they use this
engine's own FMA kernel so that nothing runs in a reduced-precision matrix mode.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_int64
from dataclasses import dataclass
from typing import Any

import torch

from ..csrc.library import KernelError, dtype_code, ptr
from .context import CacheView, StepContext


@dataclass
class FoldedRows:
    """A normalised residual stream that nobody has materialised: ``xn`` is the stream times the
    norm's scale (bfloat16) and ``ss`` holds ``parts`` rows of partial sums of squares from which
    a consuming matrix product takes each token's 1 / rms and applies it to its outputs (the
    factor commutes with the product). ``x`` is the stream itself, already up to date, and
    ``norm`` the norm part whose scale went into ``xn``; whoever cannot take the folded form
    runs that norm on ``x`` instead (``materialise``)."""

    xn: torch.Tensor
    ss: torch.Tensor
    parts: int
    x: torch.Tensor
    norm: Any

    def materialise(self, ctx: StepContext) -> torch.Tensor:
        return self.norm.forward(ctx, self.x, None)


@dataclass
class ResidualSink:
    """What a mixer or feed-forward needs to add its output into the residual stream by itself: the
    stream and the norm part that follows (its scale is folded into the next operand)."""

    x: torch.Tensor
    norm: Any


def fold_enabled(ctx: StepContext) -> bool:
    """With ``options["fold_norms"]`` norms are folded into the products around them in bfloat16
    steps of up to 16 tokens, where the engine's own weight-streaming products run. Off by
    default: measured on one B200 in alternation (Qwen2.5-1.5B sizes, 8 requests of 2,048 keys)
    the step has 200 launches instead of 255 and takes 1.293 ms instead of 1.284 ms; with the
    folded products' extra work (partial sums of squares, 1 / rms) left out altogether it takes
    1.263 ms, so 1.6 % is all there is to gain: the norm kernels are hidden behind the products
    that follow them, which fetch their weights while the norm runs."""
    return (
        ctx.dtype == torch.bfloat16 and 0 < ctx.num_tokens <= 16 and bool(ctx.options.get("fold_norms", False))
        and ctx.options.get("gemm", "auto") != "library"
    )


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


_MM_OUT_DTYPE: bool | None = None


def _mm_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """bf16 x bf16 -> fp32 through the library, accumulating and storing in 32-bit."""
    global _MM_OUT_DTYPE
    if _MM_OUT_DTYPE is None:
        try:
            a = torch.zeros(8, 16, dtype=torch.bfloat16, device=x.device)
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _MM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    if _MM_OUT_DTYPE:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    else:
        out.copy_(torch.mm(x, weight.t()))


def linear(
    ctx: StepContext,
    x: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    bias: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out = x @ weight.T (+ bias)``; ``weight`` is ``[out_features, in_features]``. ``x`` may be
    :class:`FoldedRows` (bias-free products only): the product then applies the norm's 1 / rms."""
    if isinstance(x, FoldedRows):
        folded = x
        m, k = folded.xn.shape
        kernel = None
        if bias is None and fold_enabled(ctx) and weight.shape[1] == k and tuple(out.shape) == (m, weight.shape[0]):
            epilogue = 1 if out.dtype == torch.float32 else 0
            kernel = _small_gemm_kernel(ctx, m, weight.shape[0], k, epilogue)
        if kernel is None:
            return linear(ctx, folded.materialise(ctx), weight, out, bias)
        _small_gemm(ctx, kernel, folded.xn, weight, out, epilogue, scale=folded)
        return out
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or tuple(out.shape) != (m, n):  # the message is built only when needed: this runs per product
        _need(weight.shape[1] == k, f"linear: x is [{m},{k}] but weight is {list(weight.shape)}")
        _need(False, f"linear: out is {list(out.shape)}, expected [{m},{n}]")
    _need(x.is_contiguous() and weight.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
    if m == 0:
        return out
    if x.dtype == torch.float32:
        _need(weight.dtype == torch.float32 and out.dtype == torch.float32, "linear: float32 path needs float32 operands")
        _need(bias is None or bias.dtype == torch.float32, "linear: bias must be float32")
        ctx.lib.call(
            "b200_gemm_f32", ptr(x), ptr(weight), ptr(bias), ptr(out), c_int(m), c_int(n), c_int(k),
            c_int(k), c_int(k), c_int(n), ctx.stream,
        )
        return out
    _need(x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16, "linear: bfloat16 path needs bfloat16 operands")
    if bias is None:
        epilogue = 1 if out.dtype == torch.float32 else 0
        kernel = _small_gemm_kernel(ctx, m, n, k, epilogue)
        if kernel is not None:
            _small_gemm(ctx, kernel, x, weight, out, epilogue)
            return out
    if out.dtype == torch.float32:
        _need(bias is None, "linear: no bias on the 32-bit output path")
        _mm_f32_out(x, weight, out)
    elif bias is not None:
        torch.addmm(bias, x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out=out)
    return out


def _small_gemm_kernel(ctx: StepContext, m: int, n: int, k: int, epilogue: int) -> str | None:
    """Which of this engine's own weight-streaming products takes the shape, if any.

    ``options["gemm"]``: ``"auto"`` (tcgen05 kernel, else the mma.sync one), ``"tcgen05"``,
    ``"skinny"``, or ``"library"`` (always the vendor library)."""
    choice = ctx.options.get("gemm", "auto")
    if choice == "library":
        return None
    key = (m, n, k, epilogue, choice)
    if key not in _GEMM_CHOICES:
        if len(_GEMM_CHOICES) > 4096:
            _GEMM_CHOICES.clear()
        _GEMM_CHOICES[key] = _choose_small_gemm(ctx, m, n, k, epilogue, choice)
    return _GEMM_CHOICES[key]


_GEMM_CHOICES: dict[tuple, str | None] = {}  # the rule below is a pure function of its key


def _choose_small_gemm(ctx: StepContext, m: int, n: int, k: int, epilogue: int, choice: str) -> str | None:
    stream = bool(ctx.lib.lib.b200_stream_gemm_supported(m, n, k, epilogue))
    skinny = bool(ctx.lib.lib.b200_skinny_gemm_supported(m, n, k, epilogue))
    if choice == "tcgen05":
        return "stream" if stream else None
    if choice == "skinny":
        return "skinny" if skinny else None
    # auto, from measurements on a B200 (graph-timed, weights from HBM, 1.5B shape): for up to
    # 16 rows the mma.sync kernel wins on small matrices, whose time is all launch and ramp
    # (3.0 vs 5.1 us for the 6 MB q/k/v product), and the tcgen05 kernel on large ones (down
    # 11.4 vs 14.1 us, output head 74 vs 107 us; vendor library 16.8 and 78 us). With more
    # rows the vendor library's tiles are faster on products with a short inner dimension
    # (64 rows, q/k/v: 4.6 vs 7.7 us; output head 84 vs 89 us), and it keeps those; products with
    # a long one (down: K = 8960 or 18944), which the tcgen05 kernel splits over a cluster,
    # stay here up to 64 rows (32 rows 10.2 vs 13.1 us, 64 rows 11.8 vs 13.2 us; at 128 rows
    # 15.5 vs 13.3 us the library wins again).
    # Inside a decode step the comparison shifts towards the engine's own kernels, which overlap
    # their neighbours (programmatic dependent launch) where the library's do not: with all
    # products on the tcgen05 kernel a step of 32 requests takes 1.85 ms against 1.90 ms, one of
    # 64 requests 2.57 ms against 2.25 ms. So up to 32 rows everything stays here.
    # At the 7B and 14B shapes the same rule holds: steps of 32 requests 3.76 against 4.07 ms
    # (7B) and 8.06 against 8.30 ms (14B) with the library for every product above 16 rows;
    # at 64 rows only the down products (K of 8960 and more) are worth keeping (14B: 11.66 ms
    # against 11.93 ms with q/k/v and o, K = 5120, kept too).
    if m > 16:
        return "stream" if stream and (m <= 32 or (m <= 64 and k >= 8192)) else None
    weight_bytes = 2 * n * k
    if skinny and weight_bytes < (16 << 20):
        return "skinny"
    return "stream" if stream else ("skinny" if skinny else None)


def linear_swiglu(ctx: StepContext, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """``out = silu(gate) * up`` of ``x @ weight.T`` with interleaved gate/up rows, in one
    kernel. Returns False (doing nothing) when no fused kernel takes the shape."""
    folded = x if isinstance(x, FoldedRows) else None
    if folded is not None:
        x = folded.xn
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype != torch.bfloat16 or m == 0:
        return False
    kernel = _small_gemm_kernel(ctx, m, n, k, 2)
    if kernel is None or (folded is not None and not fold_enabled(ctx)):
        return False
    _need(tuple(out.shape) == (m, n // 2) and out.is_contiguous() and x.is_contiguous(), "linear_swiglu: bad operands")
    _small_gemm(ctx, kernel, x, weight, out, 2, scale=folded)
    return True


def linear_into_residual(ctx: StepContext, a: torch.Tensor, weight: torch.Tensor, sink: ResidualSink) -> FoldedRows | None:
    """``sink.x += a @ weight.T`` inside the product's epilogue, which also writes the stream times
    the scale of the norm that follows and its partial sums of squares: returns them as
    :class:`FoldedRows`, or None (doing nothing) when the step, the norm or the shape does not
    allow it and the caller has to produce the branch output as a tensor."""
    m, k = a.shape
    n = weight.shape[0]
    norm = sink.norm
    weight_of_norm = getattr(norm, "weight", None)
    if not fold_enabled(ctx) or not getattr(norm, "foldable", False) or weight_of_norm is None:
        return None
    if a.dtype != torch.bfloat16 or tuple(sink.x.shape) != (m, n) or sink.x.dtype != torch.float32:
        return None
    kernel = _small_gemm_kernel(ctx, m, n, k, 0)
    if kernel is None:
        return None
    parts = int(getattr(ctx.lib.lib, f"b200_{kernel}_gemm_fold_parts")(*((m, n, k) if kernel == "stream" else (n, k))))
    xn = ctx.buffer("fold_xn", (m, n), torch.bfloat16)
    ss = ctx.buffer(f"fold_ss_{n}_{k}", (parts, 16), torch.float32, per_token=False)
    _small_gemm(ctx, kernel, a, weight, None, 0, sink=(sink.x, weight_of_norm, xn, ss))
    return FoldedRows(xn=xn, ss=ss, parts=parts, x=sink.x, norm=norm)


_SKINNY_SCRATCH: dict[tuple[int, int, int], tuple[int, int]] = {}  # (m, n, k) -> (floats, counters)


def _small_gemm(
    ctx: StepContext, kernel: str, x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None, epilogue: int,
    scale: FoldedRows | None = None, sink: tuple | None = None,
) -> None:
    """Launch a weight-streaming product. The mma.sync kernel keeps the partial sums of blocks
    that share rows of the weight matrix, and their arrival counters, in the step's workspace;
    the tcgen05 kernel reduces inside its clusters and needs none. ``scale``: the operand is a
    folded norm's ``xn`` and the outputs take the tokens' 1 / rms; ``sink``: (stream, next norm's
    scale, xn, ss) for the residual epilogue (see NormFold in csrc/kernels/common.cuh)."""
    from ctypes import byref

    m, k = x.shape
    n = weight.shape[0]
    head = [ptr(weight), ptr(x), ptr(out), c_int(m), c_int(n), c_int(k), c_int(epilogue)]
    folding = scale is not None or sink is not None
    if folding:
        width = k if scale is not None else 0
        eps = float(scale.norm.eps) if scale is not None else 0.0
        fold = [
            ptr(scale.ss if scale is not None else None), c_int(scale.parts if scale is not None else 0), c_int(width),
            c_float(eps),
        ] + ([ptr(t) for t in sink] if sink is not None else [ptr(None)] * 4)
    else:
        fold = []
    suffix = "_fold" if folding else ""
    if kernel == "stream":
        ctx.lib.call("b200_stream_gemm" + suffix, *head, ptr(ctx.err), *fold, ctx.stream)
        return
    need = _SKINNY_SCRATCH.get((m, n, k))
    if need is None:
        floats, counters = c_int64(0), c_int(0)
        ctx.lib.lib.b200_skinny_gemm_scratch(m, n, k, byref(floats), byref(counters))
        need = _SKINNY_SCRATCH[(m, n, k)] = (floats.value, counters.value)
    floats, counters = need
    scratch = counter_buf = None
    if floats:
        scratch = ctx.buffer("gemm_partials", (floats,), torch.float32, per_token=False)
        counter_buf = ctx.workspace.zeros("gemm_counters", max(counters, 4096), torch.int32)
    ctx.lib.call(
        "b200_skinny_gemm" + suffix, *head, ptr(scratch), c_int64(floats), ptr(counter_buf),
        c_int(counter_buf.numel() if counter_buf is not None else 0), *fold, ctx.stream,
    )


def embedding_gather(ctx: StepContext, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    vocab, hidden = table.shape
    _need(tuple(out.shape) == (ctx.num_tokens, hidden) and out.dtype == torch.float32, "embedding: bad output")
    ctx.lib.call(
        "b200_embedding_gather", ptr(table), c_int(dtype_code(table.dtype)), ptr(ctx.token_ids), ptr(out),
        c_int(ctx.num_tokens), c_int(hidden), c_int(vocab), ptr(ctx.err), ctx.stream,
    )
    return out


def rmsnorm(
    ctx: StepContext,
    x: torch.Tensor,
    delta: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: torch.Tensor | None = None,
) -> torch.Tensor:
    hidden = x.shape[1]
    num_rows = x.shape[0] if rows is None else rows.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: the residual stream is contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (hidden,), "rmsnorm: weight must be float32 [hidden]")
    _need(tuple(out.shape) == (num_rows, hidden) and out.is_contiguous(), "rmsnorm: bad output shape")
    _need(delta is None or (delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous()), "rmsnorm: bad delta")
    ctx.lib.call(
        "b200_rmsnorm", ptr(x), ptr(delta), ptr(weight), ptr(out), ptr(rows), c_int(num_rows), c_int(hidden),
        c_float(eps), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def silu_mul(ctx: StepContext, gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    tokens, twice = gate_up.shape
    inter = twice // 2
    _need(twice == 2 * inter and tuple(out.shape) == (tokens, inter), "silu_mul: bad shapes")
    _need(gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype, "silu_mul: bad operands")
    ctx.lib.call(
        "b200_silu_mul", ptr(gate_up), ptr(out), c_int(tokens), c_int(inter), c_int(dtype_code(out.dtype)), ctx.stream,
    )
    return out


def rope_kv_write(
    ctx: StepContext,
    cache: CacheView,
    qkv: torch.Tensor,
    bias: torch.Tensor | None,
    inv_freq: torch.Tensor,
    q_out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
) -> torch.Tensor:
    tokens = qkv.shape[0]
    width = (q_heads + 2 * kv_heads) * head_dim
    rot = 2 * inv_freq.numel()
    _need(tuple(qkv.shape) == (tokens, width) and qkv.is_contiguous(), "rope_kv_write: bad qkv")
    _need(tuple(q_out.shape) == (tokens, q_heads * head_dim) and q_out.is_contiguous(), "rope_kv_write: bad q_out")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "rope_kv_write: bias must be float32 [width]")
    _need(inv_freq.dtype == torch.float32, "rope_kv_write: inverse frequencies must be float32")
    _need(cache.keys.dtype == qkv.dtype and cache.values.dtype == qkv.dtype, "rope_kv_write: cache dtype differs")
    ctx.lib.call(
        "b200_rope_kv_write", ptr(qkv), ptr(bias), ptr(inv_freq), ptr(ctx.positions), ptr(ctx.token_seq),
        ptr(getattr(ctx, "seq_kv_len", None)), ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages),
        ptr(cache.keys), ptr(cache.values), ptr(q_out), c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(rot),
        c_int(cache.page_size), c_int(1 if cache.writes else 0), c_int(dtype_code(qkv.dtype)), ptr(ctx.err), ctx.stream,
    )
    return q_out


def paged_attention_plain(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_token: int = 0,
    num_tokens: int | None = None,
) -> torch.Tensor:
    """Attention of rows ``first_token .. first_token + num_tokens`` of the step over the cache."""
    tokens = ctx.num_tokens - first_token if num_tokens is None else num_tokens
    if tokens <= 0:
        return out
    _need(q.is_contiguous() and out.is_contiguous() and q.dtype == out.dtype, "attention: bad operands")
    _need(cache.keys.dtype == q.dtype, "attention: cache dtype differs from the queries'")
    row_bytes = q_heads * head_dim * q.element_size()
    ctx.lib.call(
        "b200_paged_attention_plain",
        ptr(q) if first_token == 0 else _offset(q, first_token * row_bytes),
        ptr(cache.keys), ptr(cache.values),
        _offset(ctx.positions, first_token * 4), _offset(ctx.token_seq, first_token * 4),
        ptr(cache.block_table), c_int(cache.max_pages), c_int(cache.num_pages),
        ptr(out) if first_token == 0 else _offset(out, first_token * row_bytes),
        c_int(tokens), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size),
        c_int(cache.window), c_float(scale), c_int(dtype_code(q.dtype)), ptr(ctx.err), ctx.stream,
    )
    return out


NUM_SMS = 148  # a B200; only what `decode_splits` assumes when no device is asked (tests on the CPU)
DECODE_STAGES = 3  # pieces in flight per warp of the TMA decode kernel
MAX_DECODE_SPLITS = 64  # what the merge kernel takes in one round trip


def flash_attention_supported(ctx: StepContext, q_heads: int, kv_heads: int, head_dim: int, page_size: int, decode: bool) -> bool:
    return bool(ctx.lib.lib.b200_flash_attention_supported(q_heads, kv_heads, head_dim, page_size, 1 if decode else 0))


def decode_uses_tma(ctx: StepContext, num_seqs: int, q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether a decode step's attention runs the kernel whose warps load by TMA: whenever
    the shape suits it (head_dim 128, pages of 64 rows or more), unless
    ``options["decode_loader"]`` says ``"cp_async"``."""
    loader = ctx.options.get("decode_loader", "auto")
    if loader == "cp_async" or not ctx.lib.lib.b200_decode_attention_tma_supported(q_heads, kv_heads, head_dim, page_size):
        _need(loader != "tma", "the TMA decode kernel does not take this shape")
        return False
    return True


def sm_count(ctx: StepContext) -> int:
    """SMs of the device the step runs on (the library asks the device once)."""
    return int(ctx.lib.lib.b200_sm_count())


def decode_splits(num_seqs: int, kv_heads: int, max_kv_len: int, tma: bool = False, num_sms: int = NUM_SMS) -> int:
    """How many blocks cut each request's keys in a decode step: at least one 64-key tile
    each, and few enough that the merge of their partial results stays cheap. The cp.async
    kernel (three blocks per SM) wants about two waves of blocks. The TMA kernel (rings three
    deep, two blocks per SM) wants all its blocks resident at once: measured on a B200 at
    2,048 keys, 64 requests x 2 kv heads take 26 us in 2 splits and 35 us in 6, and 64 x 8
    take 82 us unsplit. Normally at most 16 splits (14 or fewer for 10 to 24 pairs of up to 4,096 keys, see below). Very few pairs with many keys go up to 64
    while every split keeps four tiles: one request of the 1.5B shape with 30,000 keys is 32
    blocks for 148 SMs in 16 splits (1.94 ms per step) and 128 blocks in 64 (1.35 ms); 8,192
    keys: 1.36 -> 1.15 ms. With 8 such requests 18 splits were no faster than 16 (2.26 vs
    2.17 ms): the wider merge costs what the two extra splits gain."""
    tiles = max(1, (max_kv_len + 63) // 64)
    pairs = max(1, num_seqs * kv_heads)
    want = (2 if tma else 6) * num_sms // pairs  # rounded down: one block too many would start another wave
    if want >= 32:
        most = max(16, min(MAX_DECODE_SPLITS, tiles // 4))
    elif tma and want >= 12 and tiles <= 64:
        # 10 to 24 pairs of up to 4,096 keys: the blocks share their SMs with the kernels around them in the chain, and
        # about 1.5 blocks per SM leave those room to move in early. Measured at 2,100-2,300 keys,
        # 1.5B shape, ms per step with 16 (or the 2-per-SM count) -> with this rule: batch 5 1.125 ->
        # 1.115, 6 1.131 -> 1.121, 7 1.137 -> 1.131, 8 1.153 -> 1.132 (1,200 keys 1.112 -> 1.090,
        # 3,800 keys 1.217 -> 1.199), 9 1.273 -> 1.268, 10 1.282 -> 1.264, 12 unchanged; 7B shape,
        # batch 4: 2.722 -> 2.686. With more pairs (batch 16: 9 splits, 32: 4, 64: 2) two per SM
        # stay the best, with fewer (batch 4: 16 or 20 splits) the blocks do not fill the SMs; with
        # more keys the attention wants the SMs for itself (batch 8, 8,192 keys: 1.353 ms with 16
        # splits, 1.378 with 13; 30,000 keys: 2.097 and 2.136).
        most = min(14, (3 * num_sms // 2) // pairs)
    else:
        most = 16
    return max(1, min(tiles, most, want))


def paged_flash_attention(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_seq: int,
    num_seqs: int,
    decode: bool,
    max_q_len: int,
    splits: int = 1,
) -> torch.Tensor:
    """Tensor-core attention for requests ``first_seq .. first_seq + num_seqs`` of the step."""
    if num_seqs <= 0:
        return out
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.keys.dtype == torch.bfloat16, "flash attention is bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous(), "flash attention: operands must be contiguous")
    _need(not decode or first_seq == 0, "flash attention: decoded tokens must lead the batch")
    scratch = None
    # The cp.async kernel merges its splits on chip by a thread-block cluster when there are
    # very few (request, kv head) pairs, otherwise through scratch by a second small kernel:
    # measured on a B200, the cluster form wins at batch 1 (1.48 vs 1.66 ms per step of the
    # 1.5B shape) and loses from batch 8 on (1.72 vs 1.65 ms), where clusters of 16 blocks are
    # slow to place. The TMA kernel always goes through scratch unless told otherwise: at
    # batch 1 both forms take 1.10 ms per step (the cp.async kernel 1.15), at batch 2 scratch
    # 1.10 and the cluster 1.12, from batch 4 on the cluster loses.
    use_tma = decode and decode_uses_tma(ctx, num_seqs, q_heads, kv_heads, head_dim, cache.page_size)
    merge = ctx.options.get("attention_merge", "auto")
    if merge == "auto":
        merge = "cluster" if num_seqs * kv_heads <= 4 and not use_tma else "scratch"
    if decode and splits > 1 and (splits > 16 or merge == "scratch"):
        scratch = ctx.buffer("attention_partials", (num_seqs * q_heads * splits * (head_dim + 2),), torch.float32, per_token=False)
    # Keys and values by TMA into per-warp rings where the shape allows; "cp_async" keeps the
    # block-wide cp.async tiles.
    if use_tma:
        ctx.lib.call(
            "b200_paged_decode_attention_tma", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
            ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(num_seqs), c_int(cache.max_pages),
            c_int(cache.num_pages), c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size),
            c_int(cache.window), c_float(scale), c_int(splits), c_int(int(ctx.options.get("decode_stages", DECODE_STAGES))),
            ptr(scratch), ptr(ctx.err), ctx.stream,
        )
        if scratch is not None:
            ctx.lib.calls += 1  # the merge kernel is a launch of its own
        return out
    ctx.lib.call(
        "b200_paged_flash_attention", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
        ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(first_seq), c_int(num_seqs),
        c_int(num_seqs if decode else ctx.num_tokens), c_int(max_q_len), c_int(cache.max_pages), c_int(cache.num_pages),
        c_int(q_heads), c_int(kv_heads), c_int(head_dim), c_int(cache.page_size), c_int(cache.window), c_float(scale),
        c_int(1 if decode else 0), c_int(splits), ptr(scratch), ptr(ctx.err), ctx.stream,
    )
    if scratch is not None:
        ctx.lib.calls += 1  # the merge kernel is a launch of its own
    return out


def prefill_tcgen05_supported(ctx: StepContext, q_heads: int, kv_heads: int, head_dim: int, page_size: int, max_kv_len: int) -> bool:
    return bool(ctx.lib.lib.b200_flash_prefill_tcgen05_supported(q_heads, kv_heads, head_dim, page_size, max_kv_len))


def paged_prefill_attention_tcgen05(
    ctx: StepContext,
    cache: CacheView,
    q: torch.Tensor,
    out: torch.Tensor,
    q_heads: int,
    kv_heads: int,
    head_dim: int,
    scale: float,
    *,
    first_seq: int,
    num_seqs: int,
    max_q_len: int,
) -> torch.Tensor:
    """Prompt-portion attention on tcgen05 / TMEM for requests ``first_seq ..`` of the step."""
    if num_seqs <= 0:
        return out
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and cache.keys.dtype == torch.bfloat16, "tcgen05 attention is bfloat16 only")
    _need(q.is_contiguous() and out.is_contiguous() and cache.keys.is_contiguous() and cache.values.is_contiguous(), "tcgen05 attention: operands must be contiguous")
    ctx.lib.call(
        "b200_flash_prefill_tcgen05", ptr(q), ptr(cache.keys), ptr(cache.values), ptr(out), ptr(cache.block_table),
        ptr(ctx.seq_q_start), ptr(ctx.seq_q_len), ptr(ctx.seq_kv_len), c_int(first_seq), c_int(num_seqs), c_int(max_q_len),
        c_int(ctx.max_kv_len), c_int(cache.max_pages), c_int(cache.num_pages), c_int(q_heads), c_int(kv_heads),
        c_int(head_dim), c_int(cache.page_size), c_int(cache.window), c_float(scale), ptr(ctx.err), ctx.stream,
    )
    return out


def _offset(tensor: torch.Tensor, nbytes: int) -> int:
    return tensor.data_ptr() + nbytes


def argmax_rows(lib, logits: torch.Tensor, out: torch.Tensor, row_index: torch.Tensor | None, rows: int, stream) -> None:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "argmax: logits must be float32 rows")
    lib.call(
        "b200_argmax_rows", ptr(logits), c_int(rows), c_int(logits.shape[1]), c_int64(logits.stride(0)),
        ptr(row_index), ptr(out), ptr(None), ptr(None), stream,
    )
