"""Each kernel alone against a plain PyTorch float32 (or float64) reference of the same op,
at sizes other than the engine's."""

from __future__ import annotations

import math
from ctypes import c_float, c_int, c_int64, c_void_p
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def lib():
    from llm_inference_b200.csrc.library import kernels

    return kernels()


def make_ctx(lib, token_ids=None, positions=None, token_seq=None, starts=None, runs=None):
    from llm_inference_b200.parts.context import Workspace

    dev = torch.device("cuda:0")
    n = len(positions) if positions is not None else len(token_ids)
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=dev) if v is not None else None
    workspace = Workspace(dev)
    ctx = SimpleNamespace(
        lib=lib,
        device=dev,
        dtype=torch.bfloat16,
        num_tokens=n,
        token_ids=as_dev(token_ids),
        positions=as_dev(positions),
        token_seq=as_dev(token_seq),
        err=torch.zeros(1, dtype=torch.int32, device=dev),
        stream=c_void_p(torch.cuda.current_stream().cuda_stream),
        workspace=workspace,
        options={},
        buffer=lambda name, shape, dtype=None, per_token=True: workspace.get(name, shape, dtype, per_token=per_token),
    )
    if runs is not None:
        q_start = np.concatenate([[0], np.cumsum(runs)[:-1]]).tolist()
        ctx.num_seqs = len(runs)
        ctx.seq_q_start = as_dev(q_start)
        ctx.seq_q_len = as_dev(list(runs))
        ctx.seq_kv_len = as_dev([s + r for s, r in zip(starts, runs)])
        ctx.max_q_len = max(runs)
        ctx.max_kv_len = max(s + r for s, r in zip(starts, runs))
        lead = 0
        while lead < len(runs) and runs[lead] == 1:
            lead += 1
        ctx.num_decode_seqs = lead
    return ctx


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gather(lib, dtype):
    from llm_inference_b200.parts import ops

    torch.manual_seed(0)
    table = torch.randn(1000, 200, device="cuda").to(dtype)
    ids = [0, 999, 5, 5, 123, 77, 998]
    ctx = make_ctx(lib, token_ids=ids)
    out = torch.empty(len(ids), 200, device="cuda")
    ops.embedding_gather(ctx, table, out)
    assert torch.equal(out, table[ids].float())
    assert int(ctx.err.item()) == 0
    # An id outside the table is reported, not read.
    ctx = make_ctx(lib, token_ids=[3, 1000])
    ops.embedding_gather(ctx, table, out[:2])
    assert int(ctx.err.item()) == 2 and torch.all(out[1] == 0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [1000, 96, 4104, 1001, 8200])  # 16-byte form, and rows it does not take
def test_rmsnorm_with_and_without_the_residual_add(lib, dtype, hidden):
    from llm_inference_b200.parts import ops

    torch.manual_seed(1)
    rows, eps = 37, 1e-5
    x = torch.randn(rows, hidden, device="cuda") * 3
    delta = torch.randn(rows, hidden, device="cuda").to(dtype)
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda")
    ctx = make_ctx(lib, positions=[0] * rows)

    def reference(v):
        v = v.double()
        return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * weight.double()

    out = torch.empty(rows, hidden, device="cuda", dtype=dtype)
    x0 = x.clone()
    ops.rmsnorm(ctx, x0, None, weight, eps, out)
    assert torch.equal(x0, x)
    torch.testing.assert_close(out.double(), reference(x), **tol(dtype))
    x1 = x.clone()
    ops.rmsnorm(ctx, x1, delta, weight, eps, out)
    torch.testing.assert_close(x1, x + delta.float(), atol=1e-6, rtol=1e-6)  # the sum stays 32-bit
    torch.testing.assert_close(out.double(), reference(x + delta.float()), **tol(dtype))
    # Only some rows, and the stream is left alone.
    picks = torch.tensor([36, 0, 5, 5], dtype=torch.int32, device="cuda")
    x2 = x.clone()
    some = torch.empty(4, hidden, device="cuda", dtype=dtype)
    ops.rmsnorm(ctx, x2, delta, weight, eps, some, picks)
    assert torch.equal(x2, x)
    torch.testing.assert_close(some.double(), reference(x + delta.float())[picks.long()], **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(37, 83, 129), (1, 311, 96), (130, 64, 64), (5, 7, 3), (64, 152, 1000)])
def test_gemm_f32_is_true_32_bit(lib, m, n, k):
    from llm_inference_b200.parts import ops

    torch.manual_seed(2)
    # Values that TF32 or bfloat16 products would visibly corrupt.
    a = torch.randn(m, k, device="cuda") * (1 + 1e-4 * torch.randn(m, k, device="cuda"))
    w = torch.randn(n, k, device="cuda")
    bias = torch.randn(n, device="cuda")
    ctx = make_ctx(lib, positions=[0] * m)
    out = torch.empty(m, n, device="cuda")
    ops.linear(ctx, a, w, out, bias)
    want = (a.double() @ w.double().T + bias.double())
    error = (out.double() - want).abs().max().item()
    assert error < 2e-5 * math.sqrt(k), error
    # A row's result does not depend on the other rows of the call.
    alone = torch.empty(1, n, device="cuda")
    ops.linear(ctx, a[m // 2 : m // 2 + 1].contiguous(), w, alone, bias)
    assert torch.equal(alone[0], out[m // 2])


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(lib, dtype):
    from llm_inference_b200.parts import ops

    torch.manual_seed(3)
    gate_up = (torch.randn(13, 2 * 272, device="cuda") * 4).to(dtype)
    out = torch.empty(13, 272, device="cuda", dtype=dtype)
    ops.silu_mul(make_ctx(lib, positions=[0] * 13), gate_up, out)
    g, u = gate_up[:, 0::2].double(), gate_up[:, 1::2].double()  # gate and up interleaved
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))
    odd = (torch.randn(3, 2 * 37, device="cuda") * 4).to(dtype)  # not a multiple of eight
    out = torch.empty(3, 37, device="cuda", dtype=dtype)
    ops.silu_mul(make_ctx(lib, positions=[0] * 3), odd, out)
    g, u = odd[:, 0::2].double(), odd[:, 1::2].double()
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize(
    "m,n,k",
    [(1, 2048, 1536), (8, 1536, 8960), (5, 311, 96), (16, 272, 96), (9, 100, 64), (13, 4608, 3584), (8, 50, 40),
     (2, 3000, 264), (16, 151936, 64), (3, 1536, 1536), (8, 3584, 18944),
     # clusters whose last row block is ragged (8 blocks x 16 members, 104 rows in the last), 7 and all 16 tokens
     (7, 1000, 4096), (16, 1000, 4096)],
)
@pytest.mark.parametrize("kernel", ["skinny", "tcgen05"])
def test_weight_streaming_gemm_matches_float64(lib, m, n, k, kernel):
    from llm_inference_b200.parts import ops

    torch.manual_seed(m * 7 + n)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    ctx = make_ctx(lib, positions=[0] * m)
    ctx.options["gemm"] = kernel
    assert ops._small_gemm_kernel(ctx, m, n, k, 0) == {"skinny": "skinny", "tcgen05": "stream"}[kernel]
    want = x.double() @ w.double().T
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
        ops.linear(ctx, x, w, out)
        kw = dict(atol=2e-2, rtol=2e-2) if out_dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(out.double(), want, **kw)
    # Against the library product of the same operands.
    ctx.options["gemm"] = "library"
    ref = torch.empty(m, n, device="cuda", dtype=torch.float32)
    ops.linear(ctx, x, w, ref)
    ctx.options["gemm"] = kernel
    torch.testing.assert_close(out, ref, atol=2e-4, rtol=2e-4)
    # A row's result does not depend on the other rows of the call.
    alone = torch.empty(1, n, device="cuda", dtype=torch.float32)
    ops.linear(ctx, x[m - 1 :].contiguous(), w, alone)
    assert torch.equal(alone[0], out[m - 1])
    if n % 2 == 0:
        act = torch.full((m, n // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
        assert ops.linear_swiglu(ctx, x, w, act)
        g, u = want[:, 0::2], want[:, 1::2]
        torch.testing.assert_close(act.double(), g / (1 + torch.exp(-g)) * u, atol=2e-2, rtol=2e-2)
    assert int(ctx.err.item()) == 0


@pytest.mark.parametrize("m,n,k", [(17, 1536, 1536), (64, 17920, 1536), (100, 272, 96), (256, 2048, 1536), (33, 1536, 8960),
                                   # clusters of 3 (slices of 44, 44 and 40 rows, four rows per load) and of 16 with a ragged last block
                                   (20, 10200, 1536), (40, 1000, 4096)])
def test_tcgen05_gemm_takes_up_to_256_rows(lib, m, n, k):
    from llm_inference_b200.parts import ops

    torch.manual_seed(m + n)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    ctx = make_ctx(lib, positions=[0] * m)
    ctx.options["gemm"] = "tcgen05"
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    ops.linear(ctx, x, w, out)
    torch.testing.assert_close(out.double(), x.double() @ w.double().T, atol=1e-4, rtol=1e-4)
    rounded = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.linear(ctx, x, w, rounded)
    assert torch.equal(rounded, out.to(torch.bfloat16))  # the same sums, rounded once
    act = torch.full((m, n // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
    assert ops.linear_swiglu(ctx, x, w, act)
    want = x.double() @ w.double().T
    g, u = want[:, 0::2], want[:, 1::2]
    torch.testing.assert_close(act.double(), g / (1 + torch.exp(-g)) * u, atol=2e-2, rtol=2e-2)
    assert int(ctx.err.item()) == 0


@pytest.mark.parametrize("m,n,k", [(8, 1536, 8960), (40, 2048, 1536), (5, 311, 96)])  # pushed, fetched, no cluster
def test_traced_tcgen05_gemm_gives_the_same_product_and_ordered_timestamps(lib, m, n, k):
    """The instantiation that records a block's timestamps (cli/microbench.py --trace): the product
    itself is unchanged, every block wrote its points, and they follow one another in time."""
    from llm_inference_b200.csrc.library import ptr
    from llm_inference_b200.parts import ops

    torch.manual_seed(n + k)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    ctx = make_ctx(lib, positions=[0] * m)
    ctx.options["gemm"] = "tcgen05"
    plain = torch.empty(m, n, device="cuda", dtype=torch.float32)
    ops.linear(ctx, x, w, plain)
    stamps = lib.lib.b200_stream_gemm_trace_stamps()
    stride = 4096 * stamps
    buffer = torch.zeros(1, stride, dtype=torch.int64, device="cuda")
    lib.lib.b200_stream_gemm_trace(ptr(buffer), 1, stride)
    try:
        traced = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
        ops.linear(ctx, x, w, traced)
    finally:
        lib.lib.b200_stream_gemm_trace(None, 0, 0)
    torch.cuda.synchronize()
    assert torch.equal(traced, plain)
    assert int(ctx.err.item()) == 0
    data = buffer.cpu().numpy().reshape(-1, stamps)
    blocks = data[data[:, 0] != 0]
    assert len(blocks) >= (n + 127) // 128  # at least one block per 128 rows of W
    for row in blocks:
        seen = row[row != 0]  # a block without a cluster leaves the cluster's points empty
        assert len(seen) >= stamps - 2 and all(a <= b for a, b in zip(seen, seen[1:])), row
    # A later launch records nothing once the trace is off.
    buffer.zero_()
    ops.linear(ctx, x, w, traced)
    torch.cuda.synchronize()
    assert int(buffer.abs().sum().item()) == 0


def paged_layout(seq_lens, page_size, extra_pages=3, seed=0):
    """Random, non-contiguous page assignment; returns (tables [S, max_pages], num_pages)."""
    rng = np.random.default_rng(seed)
    need = [math.ceil(n / page_size) for n in seq_lens]
    num_pages = sum(need) + extra_pages
    order = rng.permutation(num_pages)
    max_pages = max(need) + 1
    tables = np.full((len(seq_lens), max_pages), -1, dtype=np.int32)
    at = 0
    for s, count in enumerate(need):
        tables[s, :count] = order[at : at + count]
        at += count
    return tables, num_pages


def gather_cache(arena, table, length, page_size):
    """[length, kv_heads, head_dim] of one request from an arena [pages, kv_heads, page, dim]."""
    rows = []
    for pos in range(length):
        rows.append(arena[int(table[pos // page_size]), :, pos % page_size, :])
    return torch.stack(rows)


@pytest.mark.parametrize("kernel", ["skinny", "tcgen05"])
@pytest.mark.parametrize("m,hidden,inner,wide", [(8, 1536, 1536, 4096), (3, 264, 520, 1000), (16, 3584, 18944, 4608), (1, 1536, 8960, 2048)])
def test_norm_folded_into_the_products_around_it(lib, kernel, m, hidden, inner, wide):
    """A product that adds into the residual stream and hands on the stream times the next norm's
    scale with partial sums of squares, then products that take that form and apply 1 / rms to
    their outputs (plain and SwiGLU): against x + a W^T and RMSNorm in float64."""
    from llm_inference_b200.parts import ops

    torch.manual_seed(m * 31 + hidden)
    eps = 1e-5
    stream = (torch.randn(m, hidden, device="cuda") * 2).contiguous()
    a = torch.randn(m, inner, device="cuda").to(torch.bfloat16)
    w_in = (torch.randn(hidden, inner, device="cuda") / math.sqrt(inner)).to(torch.bfloat16)
    scale = 1 + 0.2 * torch.randn(hidden, device="cuda")
    w_out = (torch.randn(wide, hidden, device="cuda") / math.sqrt(hidden)).to(torch.bfloat16)
    ctx = make_ctx(lib, positions=[0] * m)
    ctx.options.update(gemm=kernel, fold_norms=True)
    norm = SimpleNamespace(weight=scale, eps=eps, foldable=True)
    x = stream.clone()
    folded = ops.linear_into_residual(ctx, a, w_in, ops.ResidualSink(x, norm))
    assert folded is not None and folded.xn.shape == (m, hidden) and folded.ss.shape == (folded.parts, 16)
    want_x = stream.double() + a.double() @ w_in.double().T
    torch.testing.assert_close(x.double(), want_x, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(folded.xn.double(), x.double() * scale.double(), atol=3e-2, rtol=1e-2)
    sums = folded.ss[:, :m].double().sum(0)
    torch.testing.assert_close(sums, (x.double() ** 2).sum(1), atol=1e-2, rtol=1e-5)
    normed = x.double() * torch.rsqrt((x.double() ** 2).mean(1, keepdim=True) + eps) * scale.double()
    # What the separate norm kernel and the plain product give is the yardstick for bfloat16 here.
    h = torch.empty(m, hidden, device="cuda", dtype=torch.bfloat16)
    ops.rmsnorm(ctx, x, None, scale, eps, h)
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, wide), float("nan"), device="cuda", dtype=out_dtype)
        ops.linear(ctx, folded, w_out, out)
        want = normed @ w_out.double().T
        chain = torch.empty_like(out)
        ops.linear(ctx, h, w_out, chain)
        error, floor = (out.double() - want).abs(), (chain.double() - want).abs()
        assert error.max() <= 1.5 * floor.max() + 1e-3 and error.mean() <= 1.2 * floor.mean() + 1e-4, (error.max(), floor.max())
    act = torch.full((m, wide // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
    assert ops.linear_swiglu(ctx, folded, w_out, act)
    y = normed @ w_out.double().T
    gate, up = y[:, 0::2], y[:, 1::2]
    chain = torch.empty_like(act)
    assert ops.linear_swiglu(ctx, h, w_out, chain)
    want = gate / (1 + torch.exp(-gate)) * up
    error, floor = (act.double() - want).abs(), (chain.double() - want).abs()
    assert error.max() <= 1.5 * floor.max() + 1e-3 and error.mean() <= 1.2 * floor.mean() + 1e-4, (error.max(), floor.max())
    # The same launches again give the same bits (partial sums are added in a fixed order).
    first_sums = folded.ss[:, :m].clone()
    x2 = stream.clone()
    again = ops.linear_into_residual(ctx, a, w_in, ops.ResidualSink(x2, norm))
    assert torch.equal(x2, x) and torch.equal(again.ss[:, :m], first_sums)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("runs", [[1, 9, 3], [1, 70, 33]], ids=["few", "many"])  # "many": the one-block-per-token form
@pytest.mark.parametrize("q_heads,kv_heads,head_dim,rot,page", [(4, 2, 16, 16, 4), (6, 1, 48, 32, 8), (5, 5, 128, 128, 16)])
def test_rope_kv_write(lib, dtype, q_heads, kv_heads, head_dim, rot, page, runs):
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.context import CacheView

    torch.manual_seed(4)
    starts = [37, 0, 5]  # a decoded token, a fresh prompt, a later portion
    seq_lens = [s + r for s, r in zip(starts, runs)]
    tables, num_pages = paged_layout(seq_lens, page)
    positions = [p for s, r in zip(starts, runs) for p in range(s, s + r)]
    token_seq = [i for i, r in enumerate(runs) for _ in range(r)]
    t = len(positions)
    width = (q_heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(t, width, device="cuda").to(dtype)
    bias = torch.randn(width, device="cuda") * 0.5
    theta = 1e6
    inv_freq = torch.from_numpy(plain.rope_inverse_frequencies(rot, theta)).cuda()
    keys = torch.full((num_pages, kv_heads, page, head_dim), 7.0, device="cuda", dtype=dtype)
    values = keys.clone()
    q_out = torch.empty(t, q_heads * head_dim, device="cuda", dtype=dtype)
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq, starts=starts, runs=runs)
    table_dev = torch.from_numpy(tables).cuda()
    view = CacheView(0, True, keys, values, table_dev, num_pages, tables.shape[1], page)
    ops.rope_kv_write(ctx, view, qkv, bias, inv_freq, q_out, q_heads, kv_heads, head_dim)
    assert int(ctx.err.item()) == 0

    full = qkv.double().cpu().numpy() + bias.double().cpu().numpy()
    q = full[:, : q_heads * head_dim].reshape(t, q_heads, head_dim)
    k = full[:, q_heads * head_dim : (q_heads + kv_heads) * head_dim].reshape(t, kv_heads, head_dim)
    v = full[:, (q_heads + kv_heads) * head_dim :].reshape(t, kv_heads, head_dim)

    def rotate(x):
        out = x.copy()
        out[..., :rot] = plain.rope(x[..., :rot], positions, theta)
        return out

    kw = tol(dtype)
    np.testing.assert_allclose(q_out.double().cpu().numpy().reshape(t, q_heads, head_dim), rotate(q), **kw)
    k_rot = rotate(k)
    touched = torch.zeros(num_pages, page, dtype=torch.bool)
    for row, (pos, s) in enumerate(zip(positions, token_seq)):
        pg, r = int(tables[s, pos // page]), pos % page
        touched[pg, r] = True
        np.testing.assert_allclose(keys[pg, :, r].double().cpu().numpy(), k_rot[row], **kw)
        np.testing.assert_allclose(values[pg, :, r].double().cpu().numpy(), v[row], **kw)
    # The token that starts a page clears the rows of it that the step does not fill (leftovers of
    # the page's last owner must not reach a PV product); nothing else in the arena was written.
    cleared = torch.zeros(num_pages, page, dtype=torch.bool)
    for pos, s in zip(positions, token_seq):
        if pos % page == 0:
            for r in range(1, page):
                if pos + r >= seq_lens[s]:
                    cleared[int(tables[s, pos // page]), r] = True
    assert not bool((cleared & touched).any()) and bool(cleared.any())
    untouched = ~touched & ~cleared
    for arena in (keys, values):
        rows = arena.float().cpu().permute(0, 2, 1, 3)
        assert torch.all(rows[untouched] == 7.0) and torch.all(rows[cleared] == 0.0)
    # A call that only reads another layer's cache rotates the queries and writes nothing.
    before = keys.clone()
    view.writes = False
    ops.rope_kv_write(ctx, view, qkv, bias, inv_freq, q_out, q_heads, kv_heads, head_dim)
    assert torch.equal(keys, before)
    # A table entry that is not a page is reported.
    bad = table_dev.clone()
    bad[1, 0] = -1
    view = CacheView(0, True, keys, values, bad, num_pages, tables.shape[1], page)
    ops.rope_kv_write(ctx, view, qkv, bias, inv_freq, q_out, q_heads, kv_heads, head_dim)
    assert int(ctx.err.item()) & 1


def test_sampling_rows_with_too_many_equal_logits_take_the_long_way(lib):
    """5,000 equal logits are all candidates and do not fit the list of the many-block path: the
    row falls back to the one-block scan and must give what that gives."""
    vocab, draws = 5000, 64
    logits = torch.zeros(draws, vocab, device="cuda")
    logits[:, 123] = 1.0
    keys = [plain.draw_key(5, i) for i in range(draws)]
    args = ([0.9] * draws, [1.0] * draws, [0.0] * draws, [0] * draws, keys)
    one = run_sampler(lib, logits, *args, many_blocks=False)
    many = run_sampler(lib, logits, *args, many_blocks=True)
    assert one == many and len(set(one)) > 20


def dense_attention(q, k, v, scale, window, start):
    """q [n, heads, d] at positions start..start+n-1 over k, v [start+n, kv_heads, d], float64."""
    n, heads, d = q.shape
    groups = heads // k.shape[1]
    k = k.repeat_interleave(groups, dim=1).permute(1, 0, 2)
    v = v.repeat_interleave(groups, dim=1).permute(1, 0, 2)
    scores = (q.permute(1, 0, 2) * scale) @ k.transpose(1, 2)
    query = torch.arange(start, start + n, device=q.device)[:, None]
    key = torch.arange(k.shape[1], device=q.device)[None, :]
    mask = key <= query
    if window:
        mask &= key > query - window
    scores = scores.masked_fill(~mask[None], float("-inf"))
    return (torch.softmax(scores, -1) @ v).permute(1, 0, 2).reshape(n, heads * d)


def attention_case(dtype, q_heads, kv_heads, head_dim, page, window, starts, runs, seed=5, spike=None, spike_norm=6.0):
    torch.manual_seed(seed)
    seq_lens = [s + r for s, r in zip(starts, runs)]
    tables, num_pages = paged_layout(seq_lens, page, seed=seed)
    keys = torch.randn(num_pages, kv_heads, page, head_dim, device="cuda").to(dtype)
    values = torch.randn(num_pages, kv_heads, page, head_dim, device="cuda").to(dtype)
    positions = [p for s, r in zip(starts, runs) for p in range(s, s + r)]
    token_seq = [i for i, r in enumerate(runs) for _ in range(r)]
    t = len(positions)
    q = torch.randn(t, q_heads, head_dim, device="cuda").to(dtype)
    if spike is not None:
        # One far key lines up with one query so that a single score dominates its row: a
        # wrong page or row for that key cannot hide in the average.
        seq, key_pos, row = spike
        pg, r = int(tables[seq, key_pos // page]), key_pos % page
        direction = torch.randn(head_dim, device="cuda")
        direction = direction / direction.norm() * spike_norm
        keys[pg, :, r, :] = direction.to(dtype)
        q[row] = (direction * 3).to(dtype)
        values[pg, :, r, :] = 10.0
    expected = []
    row = 0
    for s, (start, run) in enumerate(zip(starts, runs)):
        k = gather_cache(keys, tables[s], start + run, page).double()
        v = gather_cache(values, tables[s], start + run, page).double()
        expected.append(dense_attention(q[row : row + run].double(), k, v, head_dim**-0.5, window, start))
        row += run
    return q.reshape(t, -1).contiguous(), keys, values, tables, num_pages, positions, token_seq, torch.cat(expected)


CASES = [
    # q_heads, kv_heads, head_dim, page, window, starts, runs
    (4, 2, 16, 4, 0, [0, 40, 7], [9, 1, 5]),
    (6, 1, 32, 8, 24, [0, 100, 23, 24], [30, 1, 2, 1]),
    (12, 2, 128, 16, 0, [300, 0], [1, 70]),
    (5, 5, 48, 64, 0, [129, 63], [3, 2]),
    (8, 4, 256, 16, 10, [50, 0], [1, 33]),
    (3, 3, 80, 32, 0, [1000], [1]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_paged_attention_plain(lib, dtype, case):
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.context import CacheView

    q_heads, kv_heads, head_dim, page, window, starts, runs = case
    q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
        dtype, q_heads, kv_heads, head_dim, page, window, starts, runs
    )
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq)
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
    out = torch.empty_like(q)
    ops.paged_attention_plain(ctx, view, q, out, q_heads, kv_heads, head_dim, head_dim**-0.5)
    assert int(ctx.err.item()) == 0
    torch.testing.assert_close(out.double(), expected, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(lib, dtype):
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.context import CacheView

    q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
        dtype, 4, 2, 64, 16, 0, [700, 0], [1, 4], spike=(0, 17, 0)
    )
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq)
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], 16)
    out = torch.empty_like(q)
    ops.paged_attention_plain(ctx, view, q, out, 4, 2, 64, 64**-0.5)
    assert expected[0].abs().min() > 9.0  # the spike's value dominates the reference row
    torch.testing.assert_close(out.double(), expected, **tol(dtype))


def test_window_edge_is_exact(lib):
    """The key at position - window must be invisible and the one at position - window + 1 visible."""
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.context import CacheView

    head_dim, page, window, pos = 32, 8, 24, 60
    tables, num_pages = paged_layout([pos + 1], page)
    keys = torch.zeros(num_pages, 1, page, head_dim, device="cuda")
    values = torch.zeros(num_pages, 1, page, head_dim, device="cuda")
    for p in range(pos + 1):
        values[int(tables[0, p // page]), 0, p % page, 0] = float(p)
    q = torch.zeros(1, head_dim, device="cuda")
    ctx = make_ctx(lib, positions=[pos], token_seq=[0])
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
    out = torch.empty_like(q)
    ops.paged_attention_plain(ctx, view, q, out, 1, 1, head_dim, 1.0)
    visible = list(range(pos - window + 1, pos + 1))
    assert abs(out[0, 0].item() - sum(visible) / len(visible)) < 1e-4


FLASH_CASES = [
    # q_heads, kv_heads, head_dim, page, window, starts, runs   (single-token requests lead)
    (12, 2, 128, 64, 0, [2047, 300, 0, 63, 64, 700], [1, 1, 1, 1, 1, 1]),
    (12, 2, 128, 16, 0, [300, 5, 0, 17], [1, 1, 70, 130]),
    (28, 4, 128, 64, 0, [1000, 0], [1, 200]),
    (40, 8, 128, 32, 0, [129, 64, 63], [1, 3, 2]),
    (4, 2, 64, 8, 0, [40, 0, 7], [1, 9, 5]),
    (6, 1, 64, 8, 24, [100, 23, 24, 0, 190], [1, 1, 1, 30, 40]),
    (16, 1, 64, 128, 0, [500, 3], [1, 20]),
    (8, 8, 128, 16, 100, [333, 90, 0], [1, 1, 260]),
    (64, 2, 64, 16, 0, [77, 0], [1, 5]),  # 32 heads per kv head: single tokens take the prefill form
]


@pytest.mark.parametrize("case", FLASH_CASES)
def test_paged_flash_attention(lib, case):
    """The tensor-core kernel, both forms, through the dispatcher the model uses."""
    from llm_inference_b200.parts import attention_dispatch, ops
    from llm_inference_b200.parts.context import CacheView

    q_heads, kv_heads, head_dim, page, window, starts, runs = case
    q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
        torch.bfloat16, q_heads, kv_heads, head_dim, page, window, starts, runs, seed=11
    )
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq, starts=starts, runs=runs)
    ctx.options["attention"] = "flash"
    ctx.options["decode_loader"] = "cp_async"  # the TMA-fed decode kernel has a test of its own
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
    out = torch.full_like(q, float("nan"))
    attention_dispatch.attend(ctx, view, q, out, q_heads, kv_heads, head_dim, head_dim**-0.5)
    assert int(ctx.err.item()) == 0
    torch.testing.assert_close(out.double(), expected, **tol(torch.bfloat16))
    # The same step with every request through the prefill form, and with forced splitting.
    ctx.num_decode_seqs = 0
    out2 = torch.full_like(q, float("nan"))
    attention_dispatch.attend(ctx, view, q, out2, q_heads, kv_heads, head_dim, head_dim**-0.5)
    torch.testing.assert_close(out2.double(), expected, **tol(torch.bfloat16))
    lead = 0
    while lead < len(runs) and runs[lead] == 1:
        lead += 1
    if lead and ops.flash_attention_supported(ctx, q_heads, kv_heads, head_dim, page, True):
        # One block per request; splits merged on chip by a cluster (3, 8, 16 blocks) or through
        # scratch memory by a second kernel (3; 40 and 64: its groups of 16 splits; 100: its loop).
        for splits, merge in ((1, "cluster"), (3, "cluster"), (8, "cluster"), (16, "cluster"), (3, "scratch"), (40, "scratch"),
                              (64, "scratch"), (100, "scratch")):
            ctx.options["attention_merge"] = merge
            out3 = torch.full_like(q, float("nan"))
            ops.paged_flash_attention(ctx, view, q, out3, q_heads, kv_heads, head_dim, head_dim**-0.5,
                                      first_seq=0, num_seqs=lead, decode=True, max_q_len=1, splits=splits)
            torch.testing.assert_close(out3[:lead].double(), expected[:lead], **tol(torch.bfloat16))
    assert int(ctx.err.item()) == 0


TMA_DECODE_CASES = [
    # q_heads, kv_heads, page, window, starts (one new token each)
    (12, 2, 64, 0, [300, 0, 63, 64, 700, 15, 16, 48, 2047]),
    (28, 4, 128, 0, [127, 128, 5, 1000]),
    (40, 8, 64, 100, [333, 90, 99, 100, 1500]),
    (16, 1, 256, 70, [700, 69, 70, 2]),
    (3, 3, 64, 0, [129, 4000]),
    (12, 2, 64, 0, [9000, 40, 2100]),  # a long request beside short ones, whose splits are mostly empty
]


@pytest.mark.parametrize("case", TMA_DECODE_CASES)
def test_decode_attention_with_tma_loads(lib, case):
    """The decode kernel whose warps get their keys and values by TMA: every ring depth, one
    block per request and several, against dense attention in float64; then one far key that
    must dominate its row."""
    from llm_inference_b200.parts import ops
    from llm_inference_b200.parts.context import CacheView

    q_heads, kv_heads, page, window, starts = case
    runs = [1] * len(starts)
    for spike in ((None,) if window else (None, (len(starts) - 1, 3, len(starts) - 1))):
        q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
            torch.bfloat16, q_heads, kv_heads, 128, page, window, starts, runs, seed=17, spike=spike, spike_norm=9.0
        )
        ctx = make_ctx(lib, positions=positions, token_seq=token_seq, starts=starts, runs=runs)
        ctx.options["decode_loader"] = "tma"
        view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
        # Splits merged through scratch memory by a second kernel, or on chip by a cluster.
        for splits, stages, merge in ((1, 2, "scratch"), (1, 6, "scratch"), (3, 2, "scratch"), (3, 3, "scratch"),
                                      (7, 4, "scratch"), (40, 2, "scratch"), (64, 3, "scratch"), (100, 2, "scratch"),
                                      (2, 3, "cluster"), (8, 2, "cluster"), (16, 3, "cluster")):
            ctx.options["decode_stages"] = stages
            ctx.options["attention_merge"] = merge
            out = torch.full_like(q, float("nan"))
            ops.paged_flash_attention(ctx, view, q, out, q_heads, kv_heads, 128, 128**-0.5,
                                      first_seq=0, num_seqs=len(starts), decode=True, max_q_len=1, splits=splits)
            assert int(ctx.err.item()) == 0
            torch.testing.assert_close(out.double(), expected, **tol(torch.bfloat16))
        if spike is not None:
            assert expected[spike[2]].abs().min() > 9.0


TCGEN05_CASES = [
    # q_heads, kv_heads, head_dim, page, window, starts, runs
    (12, 2, 128, 64, 0, [0], [300]),
    (12, 2, 128, 16, 0, [0, 17, 300], [70, 130, 5]),
    (28, 4, 128, 64, 0, [0, 1000], [200, 3]),
    (40, 8, 128, 32, 0, [64, 63, 129], [3, 2, 40]),
    (8, 8, 128, 16, 100, [90, 0], [1, 260]),
    (4, 1, 128, 128, 0, [500, 3], [20, 400]),
    (6, 2, 128, 64, 50, [0, 100], [260, 60]),
]


@pytest.mark.parametrize("case", TCGEN05_CASES)
def test_prefill_attention_on_tcgen05(lib, case):
    from llm_inference_b200.parts import attention_dispatch
    from llm_inference_b200.parts.context import CacheView

    q_heads, kv_heads, head_dim, page, window, starts, runs = case
    q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
        torch.bfloat16, q_heads, kv_heads, head_dim, page, window, starts, runs, seed=13
    )
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq, starts=starts, runs=runs)
    ctx.options["attention"] = "tcgen05"
    ctx.num_decode_seqs = 0  # every request through the prefill kernel, one-token runs too
    # The block table pads rows with a real page (the engine pads with the arena's spare page).
    tables = np.where(tables < 0, num_pages - 1, tables).astype(np.int32)
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
    out = torch.full_like(q, float("nan"))
    attention_dispatch.attend(ctx, view, q, out, q_heads, kv_heads, head_dim, head_dim**-0.5)
    torch.cuda.synchronize()
    assert int(ctx.err.item()) == 0
    torch.testing.assert_close(out.double(), expected, **tol(torch.bfloat16))


def test_flash_attention_finds_one_far_key_and_respects_the_window_edge(lib):
    from llm_inference_b200.parts import attention_dispatch
    from llm_inference_b200.parts.context import CacheView

    starts, runs = [700, 0], [1, 70]
    q, keys, values, tables, num_pages, positions, token_seq, expected = attention_case(
        torch.bfloat16, 4, 2, 64, 16, 0, starts, runs, spike=(0, 17, 0)
    )
    ctx = make_ctx(lib, positions=positions, token_seq=token_seq, starts=starts, runs=runs)
    ctx.options["attention"] = "flash"
    view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], 16)
    out = torch.empty_like(q)
    attention_dispatch.attend(ctx, view, q, out, 4, 2, 64, 64**-0.5)
    assert expected[0].abs().min() > 9.0
    torch.testing.assert_close(out.double(), expected, **tol(torch.bfloat16))
    # Window edge: values encode their position, queries are zero, so the output is the mean
    # of the visible positions.
    head_dim, page, window = 64, 8, 24
    for starts, runs in (([60], [1]), ([40], [30])):
        total = starts[0] + runs[0]
        tables, num_pages = paged_layout([total], page)
        keys = torch.zeros(num_pages, 1, page, head_dim, device="cuda", dtype=torch.bfloat16)
        values = torch.zeros_like(keys)
        for p in range(total):
            values[int(tables[0, p // page]), 0, p % page, 0] = float(p)
        positions = list(range(starts[0], total))
        q = torch.zeros(runs[0], head_dim, device="cuda", dtype=torch.bfloat16)
        ctx = make_ctx(lib, positions=positions, token_seq=[0] * runs[0], starts=starts, runs=runs)
        ctx.options["attention"] = "flash"
        view = CacheView(0, True, keys, values, torch.from_numpy(tables).cuda(), num_pages, tables.shape[1], page, window)
        out = torch.empty_like(q)
        attention_dispatch.attend(ctx, view, q, out, 1, 1, head_dim, 1.0)
        for row, pos in enumerate(positions):
            visible = list(range(max(0, pos - window + 1), pos + 1))
            assert abs(out[row, 0].item() - sum(visible) / len(visible)) < 0.3, (pos, out[row, 0].item())


@pytest.mark.parametrize("vocab,many_blocks", [(1511, False), (1511, True), (151936, True), (40001, True)])
def test_argmax_rows_takes_the_lowest_index_on_ties(lib, vocab, many_blocks):
    """One block per row, and (with scratch, from 4,096 entries on) many blocks per row."""
    torch.manual_seed(vocab)
    logits = torch.randn(6, vocab, device="cuda")
    logits[0, 700] = logits[0, 33] = 50.0
    logits[1, vocab - 1] = 60.0
    logits[2, 0] = 60.0
    logits[3] = 0.0
    logits[5, vocab // 2 + 3] = logits[5, vocab - 2] = 70.0  # a tie across blocks
    out = torch.full((6,), -1, dtype=torch.int32, device="cuda")
    best = torch.zeros(8, dtype=torch.int64, device="cuda")
    arrived = torch.zeros(8, dtype=torch.int32, device="cuda")
    scratch = (c_void_p(best.data_ptr()), c_void_p(arrived.data_ptr())) if many_blocks else (c_void_p(0), c_void_p(0))
    s = c_void_p(torch.cuda.current_stream().cuda_stream)
    want = logits.argmax(-1).tolist()
    want[0], want[3], want[5] = 33, 0, vocab // 2 + 3
    for _ in range(2):  # the scratch serves every launch
        out.fill_(-1)
        lib.call("b200_argmax_rows", c_void_p(logits.data_ptr()), c_int(6), c_int(vocab), c_int64(vocab), c_void_p(0), c_void_p(out.data_ptr()), *scratch, s)
        assert out.tolist() == want
        assert int(best.abs().sum()) == 0 and int(arrived.sum()) == 0
    # Only some rows.
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    out.fill_(-1)
    lib.call("b200_argmax_rows", c_void_p(logits.data_ptr()), c_int(2), c_int(vocab), c_int64(vocab), c_void_p(rows.data_ptr()), c_void_p(out.data_ptr()), *scratch, s)
    assert out.tolist() == [-1, vocab - 1, -1, -1, want[4], -1]


def run_sampler(lib, logits, temperature, top_p, min_p, top_k, keys, many_blocks=False):
    """``many_blocks``: with scratch, so that large vocabularies are scanned by many blocks a row."""
    rows, vocab = logits.shape
    lib.lib.b200_sample_scratch_bytes.restype = c_int64
    scratch = torch.zeros(int(lib.lib.b200_sample_scratch_bytes(rows)) if many_blocks else 16, dtype=torch.uint8, device="cuda")
    f = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")
    t, p, m = f(temperature), f(top_p), f(min_p)
    k = torch.tensor(top_k, dtype=torch.int32, device="cuda")
    key = torch.tensor(np.asarray(keys, dtype=np.uint64).view(np.int64), dtype=torch.int64, device="cuda")
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    lib.call(
        "b200_sample_rows", c_void_p(logits.data_ptr()), c_int(rows), c_int(vocab), c_int64(logits.stride(0)),
        c_void_p(t.data_ptr()), c_void_p(p.data_ptr()), c_void_p(m.data_ptr()), c_void_p(k.data_ptr()),
        c_void_p(key.data_ptr()), c_void_p(0), c_void_p(out.data_ptr()),
        c_void_p(scratch.data_ptr() if many_blocks else 0), c_int64(scratch.numel()), c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    if many_blocks:
        # The histogram (256 words), and after prefix, mask and remaining the arrival counter, the
        # cursor and the overflow flag are back at zero.
        assert int(scratch[:1024].sum()) == 0 and int(scratch[1036:1048].sum()) == 0
    return out.tolist()


@pytest.mark.parametrize(
    "vocab,settings",
    [
        (311, dict(temperature=0.8)),
        (311, dict(temperature=1.3, top_k=7)),
        (311, dict(temperature=0.9, top_p=0.7)),
        (311, dict(temperature=1.0, min_p=0.15)),
        (5000, dict(temperature=1.0)),  # more tokens than candidates: only the top 1024 may be drawn
        (5000, dict(temperature=0.7, top_k=40, top_p=0.9, min_p=0.02)),
        (2000, dict(temperature=1.1, top_p=0.95)),  # with scratch: the whole row is the list
        (50021, dict(temperature=0.9, top_k=300, top_p=0.92, min_p=0.001)),
    ],
)
@pytest.mark.parametrize("many_blocks", [False, True], ids=["one_block", "many_blocks"])
def test_sampling_matches_the_plain_filters_and_draw(lib, vocab, settings, many_blocks):
    rng = np.random.default_rng(vocab)
    base = torch.from_numpy(rng.normal(0, 2.0, vocab).astype(np.float32)).cuda()
    draws = 400
    logits = base.repeat(draws, 1).contiguous()
    keys = [plain.draw_key(99, i) for i in range(draws)]
    temperature = settings.get("temperature", 1.0)
    top_k, top_p, min_p = settings.get("top_k", 0), settings.get("top_p", 1.0), settings.get("min_p", 0.0)
    got = run_sampler(lib, logits, [temperature] * draws, [top_p] * draws, [min_p] * draws, [top_k] * draws, keys, many_blocks)
    probs = plain.surviving_probabilities(base.cpu().numpy(), temperature, top_k, top_p, min_p)
    assert all(probs[t] > 0 for t in got), "a filtered token was drawn"
    # The engine draws by inverse CDF in token order with u = uniform_from_key(key).
    cdf = np.cumsum(probs)
    agree = 0
    for token, key in zip(got, keys):
        u = plain.uniform_from_key(key)
        expected = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
        agree += token == expected
    assert agree >= draws - 2, f"only {agree} of {draws} draws match the plain inverse CDF"
    # Same key, same token; and the result does not depend on the row it sits in.
    again = run_sampler(lib, logits[:3], [temperature] * 3, [top_p] * 3, [min_p] * 3, [top_k] * 3, [keys[7], keys[7], keys[0]], many_blocks)
    assert again[0] == again[1] == got[7] and again[2] == got[0]
