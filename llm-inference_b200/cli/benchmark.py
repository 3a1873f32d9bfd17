"""Continuous-batching benchmark over pre-tokenized prompts, with the options and the output of
the reference's ``instinct-bench`` (python/instinct/benchmark.py:161-425): every prompt is
submitted at once, the engine steps until all are done; reports generated tokens per second
(prefill included, as the reference counts it) and TTFT / TPOT / end-to-end percentiles.

    python -m llm_inference_b200.cli.benchmark --model DIR --prompts prompts.json --output out.json
        [--output-length 32 --warmups 5 --repetitions 3 --max-sequences 16 --max-model-length 2048
         --kv-cache-mib 512 --stop-on-eos]

``prompts.json`` is a JSON array of arrays of token ids.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
import time
from pathlib import Path

from .generate import add_engine_options, engine_from


def percentiles(values: list[float]) -> dict[str, float]:
    """p50 / p95 / p99 by the nearest-rank rule (python/instinct/benchmark.py:94-107)."""
    if not values:
        return {"p50": 0.0, "p95": 0.0, "p99": 0.0}
    ordered = sorted(values)

    def pick(q: float) -> float:
        return ordered[min(len(ordered) - 1, max(0, math.ceil(q * len(ordered)) - 1))]

    return {"p50": pick(0.50), "p95": pick(0.95), "p99": pick(0.99)}


def run_once(engine, prompts, output_length: int, eos) -> tuple[list[dict], float]:
    import torch

    torch.cuda.synchronize()
    begin = time.perf_counter()
    ids = [engine.submit(p, output_length, eos) for p in prompts]
    first: dict[int, float] = {}
    last: dict[int, float] = {}
    counts = {i: 0 for i in ids}
    while engine.has_work():
        events = engine.step()
        now = time.perf_counter()
        for event in events:
            first.setdefault(event.request_id, now)
            last[event.request_id] = now
            counts[event.request_id] += 1
    wall = time.perf_counter() - begin
    metrics = []
    for rid, prompt in zip(ids, prompts):
        n = counts[rid]
        metrics.append({
            "prompt_tokens": len(prompt), "output_tokens": n, "ttft_ms": (first[rid] - begin) * 1e3,
            "tpot_ms": (last[rid] - first[rid]) * 1e3 / (n - 1) if n > 1 else None,
            "e2e_ms": (last[rid] - begin) * 1e3,
        })
        engine.forget(rid)
    return metrics, wall


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    add_engine_options(parser)
    parser.add_argument("--prompts", type=Path, required=True, help="JSON array of pre-tokenized integer arrays")
    parser.add_argument("--output", type=Path, required=True)
    parser.add_argument("--output-length", type=int, default=32)
    parser.add_argument("--warmups", type=int, default=5)
    parser.add_argument("--repetitions", type=int, default=3)
    parser.add_argument("--stop-on-eos", action="store_true", help="allow EOS to shorten requests")
    args = parser.parse_args(argv)

    prompts = [[int(t) for t in p] for p in json.loads(args.prompts.read_text())]
    with engine_from(args) as engine:
        eos = engine.eos_token_ids if args.stop_on_eos else ()
        for _ in range(args.warmups):
            run_once(engine, prompts, args.output_length, eos)
        all_metrics, walls = [], []
        for _ in range(args.repetitions):
            metrics, wall = run_once(engine, prompts, args.output_length, eos)
            all_metrics += metrics
            walls.append(wall)
        stats = engine.stats()
    seconds = sum(walls)
    result = {
        "implementation": "llm-inference_b200",
        "configuration": {
            "model_path": str(args.model), "output_length": args.output_length, "warmups": args.warmups,
            "repetitions": args.repetitions, "concurrency": len(prompts),
            "prompt_token_lengths": [len(p) for p in prompts], "max_model_length": args.max_model_length,
            "kv_cache_mib": args.kv_cache_mib, "stop_on_eos": args.stop_on_eos, "dtype": args.dtype,
        },
        "aggregate": {
            "generated_tokens_per_second": sum(m["output_tokens"] for m in all_metrics) / seconds,
            "prompt_tokens_per_second": sum(m["prompt_tokens"] for m in all_metrics) / seconds,
            "ttft_ms": percentiles([m["ttft_ms"] for m in all_metrics]),
            "tpot_ms": percentiles([m["tpot_ms"] for m in all_metrics if m["tpot_ms"] is not None]),
            "e2e_ms": percentiles([m["e2e_ms"] for m in all_metrics]),
        },
        "engine_stats": {k: v for k, v in stats.items() if not isinstance(v, dict)},
        "requests": all_metrics,
    }
    args.output.parent.mkdir(parents=True, exist_ok=True)
    args.output.write_text(json.dumps(result, indent=2, sort_keys=True) + "\n")
    print(json.dumps(result["aggregate"], indent=2, sort_keys=True))
    return 0


if __name__ == "__main__":
    sys.exit(main())
