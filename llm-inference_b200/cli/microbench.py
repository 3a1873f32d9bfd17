"""Times one kernel of the library alone, at a given shape, with CUDA events.

    python -m llm_inference_b200.cli.microbench gemm --m 8 --n 17920 --k 1536 [--swiglu] [--library]
    python -m llm_inference_b200.cli.microbench decode_attention --batch 64 --context 2048
    python -m llm_inference_b200.cli.microbench prefill_attention --tokens 2048

Between timed launches a buffer larger than the L2 cache is overwritten, so every launch
reads its operands from HBM. Prints one JSON line with the median time and the bytes or flops
per second it corresponds to. Used for roofline numbers and as the small case for profiler
captures.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from ctypes import c_void_p
from types import SimpleNamespace

import numpy as np
import torch


class _Ctx(SimpleNamespace):
    @property
    def stream(self):
        return c_void_p(torch.cuda.current_stream().cuda_stream)


def make_ctx(positions=None, token_seq=None, starts=None, runs=None, options=None):
    from ..csrc.library import kernels
    from ..parts.context import Workspace

    dev = torch.device("cuda:0")
    ws = Workspace(dev)
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=dev) if v is not None else None
    ctx = _Ctx(
        lib=kernels(), device=dev, err=torch.zeros(1, dtype=torch.int32, device=dev), workspace=ws,
        options=dict(options or {}), positions=as_dev(positions), token_seq=as_dev(token_seq),
        num_tokens=len(positions) if positions is not None else 0,
        buffer=lambda name, shape, dtype=None, per_token=True: ws.get(name, shape, dtype, per_token=per_token),
    )
    if runs is not None:
        ctx.num_seqs = len(runs)
        ctx.seq_q_start = as_dev(np.concatenate([[0], np.cumsum(runs)[:-1]]).tolist())
        ctx.seq_q_len = as_dev(list(runs))
        ctx.seq_kv_len = as_dev([s + r for s, r in zip(starts, runs)])
        ctx.max_q_len = max(runs)
        ctx.max_kv_len = max(s + r for s, r in zip(starts, runs))
        ctx.num_decode_seqs = len(runs) if max(runs) == 1 else 0
    return ctx


def time_launches(fn, iters: int, warmup: int = 3) -> float:
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.fill_(1)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def time_back_to_back(fns, launches: int) -> float:
    """Microseconds per launch when ``fns`` run round-robin back to back on the device. The
    launches are captured in a CUDA graph, so host launch cost does not enter; the operands
    of all of them together must exceed the L2 cache."""
    for fn in fns:
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            fns[i % len(fns)]()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / launches


TRACE_POINTS = ("resident", "predecessor done", "first stage landed", "last stage landed", "accumulator complete",
                "partial tiles met", "slice stored", "leaving")


def trace_back_to_back(lib, fns, launches: int) -> dict:
    """The tcgen05 product's own timeline (b200_stream_gemm_trace) of ``launches`` launches that run
    back to back in a CUDA graph: for every point of a block's life, when the first, the median
    and the last block of a launch passed it, in microseconds after the last block of the launch
    in front left; averaged over the later half of the launches."""
    from ..csrc.library import ptr

    for fn in fns:
        fn()
    torch.cuda.synchronize()
    stamps = lib.b200_stream_gemm_trace_stamps()
    stride = 4096 * stamps
    buffer = torch.zeros(launches, stride, dtype=torch.int64, device="cuda")
    lib.b200_stream_gemm_trace(ptr(buffer), launches, stride)
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(graph):
            for i in range(launches):
                fns[i % len(fns)]()
    finally:
        lib.b200_stream_gemm_trace(None, 0, 0)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    data = buffer.cpu().numpy().reshape(launches, -1, stamps)
    blocks = int((data[1, :, 0] != 0).sum())
    data = data[:, :blocks, :].astype(np.float64) / 1e3  # microseconds
    rows = {name: [] for name in TRACE_POINTS}
    spans = []
    for j in range(launches // 2, launches):
        origin = data[j - 1, :, stamps - 1].max()
        spans.append(data[j, :, stamps - 1].max() - origin)
        for i, name in enumerate(TRACE_POINTS):
            column = data[j, :, i]
            column = column[column != 0]
            if column.size:
                rows[name].append((column.min() - origin, float(np.median(column)) - origin, column.max() - origin))
    table = {name: [round(float(v), 2) for v in np.mean(np.array(values), axis=0)] for name, values in rows.items() if values}
    return {"blocks": blocks, "us_per_launch": round(float(np.mean(spans)), 2), "first_median_last_us": table}


def bench_gemm(args) -> dict:
    from ..parts import ops

    m, n, k = args.m, args.n, args.k
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") / k**0.5).to(torch.bfloat16)
    ctx = make_ctx(positions=[0] * m, options={"gemm": args.gemm})
    if args.plan is not None:
        ctx.lib.lib.b200_stream_gemm_plan_override(*args.plan)
    if args.rotate:
        # Enough copies of the weights that one round exceeds the L2 cache several times.
        copies = max(2, -(-(512 << 20) // (w.numel() * 2)))
        weights = [w] + [w.clone() for _ in range(copies - 1)]
        out = torch.empty(m, n // 2 if args.swiglu else n, device="cuda", dtype=torch.float32 if args.f32_out else torch.bfloat16)
        if args.swiglu and args.gemm == "library":
            mid = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            fns = [lambda wi=wi: (ops.linear(ctx, x, wi, mid), ops.silu_mul(ctx, mid, out)) for wi in weights]
        elif args.swiglu:
            fns = [lambda wi=wi: ops.linear_swiglu(ctx, x, wi, out) for wi in weights]
        else:
            fns = [lambda wi=wi: ops.linear(ctx, x, wi, out) for wi in weights]
        if args.trace:
            if args.gemm != "tcgen05":
                raise SystemExit("--trace records the tcgen05 product's own timestamps: give --gemm tcgen05")
            return {"kernel": "gemm", "m": m, "n": n, "k": k, "swiglu": args.swiglu, "mode": "back-to-back, traced",
                    **trace_back_to_back(ctx.lib.lib, fns, 4 * copies)}
        us = time_back_to_back(fns, 4 * copies)
        nbytes = w.numel() * 2 + x.numel() * 2 + out.numel() * out.element_size()
        return {"kernel": "gemm", "m": m, "n": n, "k": k, "gemm": args.gemm, "swiglu": args.swiglu, "mode": "back-to-back",
                "us": us, "GBps": nbytes / us / 1e3}
    if args.swiglu:
        out = torch.empty(m, n // 2, device="cuda", dtype=torch.bfloat16)
        if args.gemm == "library":
            mid = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

            def fn():
                ops.linear(ctx, x, w, mid)
                ops.silu_mul(ctx, mid, out)
        else:
            fn = lambda: ops.linear_swiglu(ctx, x, w, out)
    else:
        out = torch.empty(m, n, device="cuda", dtype=torch.float32 if args.f32_out else torch.bfloat16)
        fn = lambda: ops.linear(ctx, x, w, out)
    us = time_launches(fn, args.iters)
    nbytes = w.numel() * 2 + x.numel() * 2 + out.numel() * out.element_size()
    return {"kernel": "gemm", "m": m, "n": n, "k": k, "gemm": args.gemm, "swiglu": args.swiglu, "us": us,
            "GBps": nbytes / us / 1e3, "TFLOPs": 2.0 * m * n * k / us / 1e6}


def bench_attention(args, decode: bool) -> dict:
    from ..parts import attention_dispatch
    from ..parts.context import CacheView

    q_heads, kv_heads, dim, page = args.q_heads, args.kv_heads, args.head_dim, args.page
    if decode:
        starts, runs = [args.context - 1] * args.batch, [1] * args.batch
    else:
        starts, runs = [args.context - args.tokens], [args.tokens]
    lens = [s + r for s, r in zip(starts, runs)]
    need = [-(-n // page) for n in lens]
    num_pages = sum(need) + 1
    order = np.random.default_rng(0).permutation(num_pages - 1)
    tables = np.zeros((len(lens), max(need)), dtype=np.int32)
    at = 0
    for s, c in enumerate(need):
        tables[s, :c] = order[at : at + c]
        at += c
    positions = [p for s, r in zip(starts, runs) for p in range(s, s + r)]
    token_seq = [i for i, r in enumerate(runs) for _ in range(r)]
    options = {"attention": "plain" if args.plain else args.attention, "decode_loader": args.loader}
    if args.splits:
        options["decode_splits"] = args.splits
    if args.stages:
        options["decode_stages"] = args.stages
    ctx = make_ctx(positions, token_seq, starts, runs, options)
    q = torch.randn(len(positions), q_heads * dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    table = torch.from_numpy(tables).cuda()
    # --layers N: N arenas of the same geometry, as the layers of a model have; back to back
    # they exceed the L2 cache when one of them does not.
    fns = []
    for _ in range(max(1, args.layers)):
        keys = torch.randn(num_pages, kv_heads, page, dim, device="cuda").to(torch.bfloat16)
        values = torch.randn_like(keys)
        view = CacheView(0, True, keys, values, table, num_pages, tables.shape[1], page, args.window)
        fns.append(lambda view=view: attention_dispatch.attend(ctx, view, q, out, q_heads, kv_heads, dim, dim**-0.5))
    # --rotate: back to back inside a CUDA graph, so that neither the host's launch cost nor
    # the idle gap before a lone launch enters (with one arena the cache stays in L2, as it
    # does in a small model's step, where the layer's keys were written just before).
    us = time_back_to_back(fns, 16 * len(fns)) if args.rotate else time_launches(fns[0], args.iters)
    kv_bytes = sum(lens) * kv_heads * dim * 2 * 2
    flops = sum(4.0 * q_heads * dim * r * (s + (r + 1) / 2) for s, r in zip(starts, runs))
    return {"kernel": "decode_attention" if decode else "prefill_attention", "batch": len(lens), "context": args.context,
            "tokens": len(positions), "loader": args.loader, "splits": args.splits, "stages": args.stages,
            "layers": args.layers, "us": us, "GBps": kv_bytes / us / 1e3, "TFLOPs": flops / us / 1e6}


def bench_resident(args) -> dict:
    """One decode step as the resident kernel at a named shape: time per step, and for each kind of
    phase how long the slowest block takes to ask for its operand, to finish, and how long block 0
    then waits at the barrier (timestamps the kernel records when handed a trace buffer)."""
    import numpy as np

    from .. import models  # noqa: F401
    from ..config import parse_config
    from ..engine.engine import Engine
    from ..engine.loading import random_model
    from ..engine.runner import StepEntry
    from .presets import PRESETS

    _, config = parse_config(dict(PRESETS[args.shape]))
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    engine = Engine(model=model, max_num_sequences=16, max_model_length=2 * args.context, kv_cache_bytes=8 << 30,
                    prefill_chunk_size=2048, prefill_burst_size=2048, max_batch_tokens=2048 + 16, cuda_graphs=False,
                    decode_kernel="resident")
    runner = engine.runner
    if runner.options["resident"] is None:
        raise SystemExit("the resident kernel does not take this shape")
    rng = np.random.default_rng(0)
    ids = list(range(1, args.batch + 1))
    for rid in ids:
        engine.cache.open(rid)
        for begin in range(0, args.context, 2048):
            runner.step([StepEntry(rid, [int(t) for t in rng.integers(0, config.vocab_size, min(2048, args.context - begin))], ())])
    phases = 2 + 5 * len(model.schedule)
    trace = torch.zeros(phases * 4, dtype=torch.int64, device="cuda")
    runner.options["resident_trace"] = trace
    step = lambda: runner.step([StepEntry(rid, (int(rng.integers(0, config.vocab_size)),), (0,)) for rid in ids])
    for _ in range(3):
        step()
    trace.zero_()
    us = time_launches(step, args.iters)
    trace.zero_()
    step()
    torch.cuda.synchronize()
    runner.check()
    stamps = trace.cpu().numpy().reshape(phases, 4).astype(np.float64) / 1e3
    names = ["embedding"] + ["q/k/v", "attention", "output", "gate/up", "down"] * len(model.schedule) + ["head"]
    kinds: dict[str, list] = {}
    for name, (enter, asked, finished, left) in zip(names, stamps):
        asked = asked if asked > 0 else enter
        kinds.setdefault(name, []).append((asked - enter, finished - asked, max(left - finished, 0.0) if left > 0 else 0.0))
    summary = {
        name: dict(zip(("operand_asked_us", "work_us", "barrier_us"), (round(float(v), 2) for v in np.mean(rows, axis=0))))
        for name, rows in kinds.items()
    }
    engine.close()
    return {"kernel": "resident_decode", "shape": args.shape, "batch": args.batch, "context": args.context, "us_per_step": us,
            "kernel_us": float(stamps[-1, 2] - stamps[0, 0]), "phases": summary}


def bench_timeline(args) -> dict:
    """One layer of a replayed decode step on the timeline: for every kernel of the step's second
    layer, when its first block started, when it ended and how long after its predecessor's end
    (Kineto timestamps through torch.profiler; no kernel is replayed or serialised)."""
    import numpy as np
    from torch.profiler import ProfilerActivity, profile

    from .. import models  # noqa: F401
    from ..config import parse_config
    from ..engine.engine import Engine
    from ..engine.loading import random_model
    from ..engine.runner import StepEntry
    from .presets import PRESETS

    _, config = parse_config(dict(PRESETS[args.shape]))
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    kv_bytes = 2 * config.num_hidden_layers * config.num_key_value_heads * config.head_dim * 2 * args.batch * (args.context + 256)
    engine = Engine(model=model, max_num_sequences=max(16, args.batch), max_model_length=2 * args.context,
                    kv_cache_bytes=kv_bytes + (1 << 30), prefill_chunk_size=2048, prefill_burst_size=2048,
                    max_batch_tokens=2048 + max(16, args.batch))
    runner = engine.runner
    rng = np.random.default_rng(0)
    ids = list(range(1, args.batch + 1))
    for rid in ids:
        engine.cache.open(rid)
        for begin in range(0, args.context, 2048):
            runner.step([StepEntry(rid, [int(t) for t in rng.integers(0, config.vocab_size, min(2048, args.context - begin))], ())])
    step = lambda: runner.step([StepEntry(rid, (int(rng.integers(0, config.vocab_size)),), (0,)) for rid in ids])
    for _ in range(6):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    firsts = [i for i, e in enumerate(events) if "embedding" in e.name]
    if len(firsts) < 3:
        raise SystemExit("the profiler did not see three steps")
    per_step = firsts[2] - firsts[1]
    # The second layer of the middle step: from its first norm to the next layer's first norm
    # (two norm kernels per layer in the stock arrangement).
    norms = [i for i in range(firsts[1], firsts[2]) if "rmsnorm" in events[i].name]
    if len(norms) < 5:
        raise SystemExit("the step does not show two norm kernels per layer")
    start, per_layer = norms[2], norms[4] - norms[2]
    origin = events[firsts[1]].time_range.start
    rows, previous_end = [], events[start - 1].time_range.end
    for e in events[start : start + per_layer]:
        rows.append({"kernel": e.name[:60], "start_us": round(e.time_range.start - origin, 1),
                     "end_us": round(e.time_range.end - origin, 1), "after_us": round(e.time_range.end - previous_end, 1)})
        previous_end = e.time_range.end
    engine.close()
    return {"kernel": "decode step timeline", "shape": args.shape, "batch": args.batch, "context": args.context,
            "kernels_per_step": per_step, "layer_us": round(sum(r["after_us"] for r in rows), 1), "layer": rows}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("kernel", choices=["gemm", "decode_attention", "prefill_attention", "resident", "timeline"])
    parser.add_argument("--shape", default="qwen2.5-1.5b", help="resident, timeline: a named model shape")
    parser.add_argument("--m", type=int, default=8)
    parser.add_argument("--n", type=int, default=17920)
    parser.add_argument("--k", type=int, default=1536)
    parser.add_argument("--swiglu", action="store_true")
    parser.add_argument("--f32-out", action="store_true")
    parser.add_argument("--library", action="store_true", help="time the vendor library's product instead")
    parser.add_argument("--gemm", default="auto", choices=["auto", "tcgen05", "skinny", "library"])
    parser.add_argument("--rotate", action="store_true", help="launch back to back over rotating copies of the weights")
    parser.add_argument("--trace", action="store_true",
                        help="with --rotate --gemm tcgen05: the blocks' own timestamps instead of the launch time")
    parser.add_argument("--plan", type=int, nargs=3, metavar=("STAGES", "BLOCKS", "CLUSTER"), default=None,
                        help="tcgen05 product: force ring depth, blocks aimed at and cluster width (0 = the planner's choice)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--q-heads", type=int, default=12)
    parser.add_argument("--kv-heads", type=int, default=2)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page", type=int, default=64)
    parser.add_argument("--window", type=int, default=0)
    parser.add_argument("--plain", action="store_true")
    parser.add_argument("--attention", default="auto", choices=["auto", "flash", "tcgen05"])
    parser.add_argument("--loader", default="auto", choices=["auto", "tma", "cp_async"], help="how decode attention loads keys and values")
    parser.add_argument("--splits", type=int, default=0, help="blocks per (request, kv head) in decode attention (0: the engine's rule)")
    parser.add_argument("--stages", type=int, default=0, help="ring depth of the TMA decode kernel (0: the engine's default)")
    parser.add_argument("--layers", type=int, default=1, help="attention: rotate over this many arenas")
    parser.add_argument("--iters", type=int, default=20)
    args = parser.parse_args(argv)
    if args.library:
        args.gemm = "library"
    if args.kernel == "gemm":
        result = bench_gemm(args)
    elif args.kernel == "resident":
        result = bench_resident(args)
    elif args.kernel == "timeline":
        result = bench_timeline(args)
    else:
        result = bench_attention(args, args.kernel == "decode_attention")
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
