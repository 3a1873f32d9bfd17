"""Continuous-batching benchmark over pre-tokenized prompts, with the options and the output of
the reference's ``instinct-bench`` (python/instinct/benchmark.py:161-425): every prompt is
submitted at once, the engine steps until all are done; reports generated tokens per second
(prefill included, as the reference counts it) and TTFT / TPOT / end-to-end percentiles.

    python -m llm_inference_b200.cli.benchmark --model DIR --prompts prompts.json --output out.json
        [--output-length 32 --warmups 5 --repetitions 3 --max-sequences 16 --max-model-length 2048
         --kv-cache-mib 512 --stop-on-eos]

``prompts.json`` is a JSON array of arrays of token ids. Instead of ``--prompts``, ``--mix N``
draws N requests with prompt lengths uniform in ``--mix-prompt-lengths LO HI``, output lengths
uniform in ``--mix-output-lengths LO HI`` and token ids uniform in the vocabulary, from
``--mix-seed``; with ``--random SHAPE`` in place of ``--model`` no file is needed at all:

    python -m llm_inference_b200.cli.benchmark --random qwen2.5-14b --mix 64 --mix-prompt-lengths 128 4096
        --mix-output-lengths 128 512 --max-sequences 64 --max-model-length 8192 --kv-cache-mib 60000
        --prefill-chunk-size 512 --warmups 1 --repetitions 1 --output out.json
"""

from __future__ import annotations

import argparse
import json
import math
import sys
import time

import numpy as np
from pathlib import Path

from .generate import add_engine_options, engine_from


def percentiles(values: list[float]) -> dict[str, float]:
    """p50 / p95 / p99, each interpolated linearly between the two samples around rank
    ``q * (n - 1)``: the rule the reference's benchmark reports with
    (python/instinct/benchmark.py:94-107), so that the same samples give the same figures.
    Empty input gives NaN, as there."""
    ranked = np.sort(np.asarray(values, dtype=np.float64))

    def at(q: float) -> float:
        if ranked.size == 0:
            return math.nan
        rank = q * (ranked.size - 1)
        below = int(rank)
        above = min(below + 1, ranked.size - 1)
        share = rank - below
        return float(ranked[below] + (ranked[above] - ranked[below]) * share)

    return {"p50": at(0.50), "p95": at(0.95), "p99": at(0.99)}


def synthetic_mix(count: int, prompt_lengths, output_lengths, vocab: int, seed: int):
    """``count`` prompts of random ids with their output lengths, both lengths uniform in the
    given inclusive ranges."""
    import numpy as np

    rng = np.random.default_rng(seed)
    prompts, outputs = [], []
    for _ in range(count):
        n = int(rng.integers(prompt_lengths[0], prompt_lengths[1] + 1))
        prompts.append([int(t) for t in rng.integers(0, vocab, n)])
        outputs.append(int(rng.integers(output_lengths[0], output_lengths[1] + 1)))
    return prompts, outputs


def run_once(engine, prompts, output_length, eos) -> tuple[list[dict], float]:
    """Submits every prompt at once and steps until all are done. ``output_length`` is one
    number for all requests or a list with one per prompt."""
    import torch

    lengths = output_length if isinstance(output_length, (list, tuple)) else [output_length] * len(prompts)
    torch.cuda.synchronize()
    begin = time.perf_counter()
    ids = [engine.submit(p, n, eos) for p, n in zip(prompts, lengths)]
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
    parser.add_argument("--prompts", type=Path, default=None, help="JSON array of pre-tokenized integer arrays")
    parser.add_argument("--mix", type=int, default=0, metavar="N", help="instead of --prompts: N synthetic requests")
    parser.add_argument("--mix-prompt-lengths", type=int, nargs=2, default=[128, 4096], metavar=("LO", "HI"))
    parser.add_argument("--mix-output-lengths", type=int, nargs=2, default=[128, 512], metavar=("LO", "HI"))
    parser.add_argument("--mix-seed", type=int, default=0)
    parser.add_argument("--output", type=Path, required=True)
    parser.add_argument("--output-length", type=int, default=32)
    parser.add_argument("--warmups", type=int, default=5)
    parser.add_argument("--repetitions", type=int, default=3)
    parser.add_argument("--stop-on-eos", action="store_true", help="allow EOS to shorten requests")
    args = parser.parse_args(argv)

    if (args.prompts is None) == (args.mix <= 0):
        parser.error("give either --prompts FILE or --mix N")
    with engine_from(args) as engine:
        if args.mix > 0:
            prompts, output_length = synthetic_mix(
                args.mix, args.mix_prompt_lengths, args.mix_output_lengths, engine.vocab_size, args.mix_seed
            )
        else:
            prompts = [[int(t) for t in p] for p in json.loads(args.prompts.read_text())]
            output_length = args.output_length
        eos = engine.eos_token_ids if args.stop_on_eos else ()
        for _ in range(args.warmups):
            run_once(engine, prompts, output_length, eos)
        all_metrics, walls = [], []
        for _ in range(args.repetitions):
            metrics, wall = run_once(engine, prompts, output_length, eos)
            all_metrics += metrics
            walls.append(wall)
        stats = engine.stats()
    seconds = sum(walls)
    result = {
        "implementation": "llm-inference_b200",
        "configuration": {
            "model_path": str(args.model) if args.model else f"random:{args.random}", "warmups": args.warmups,
            "output_length": args.output_length if args.mix <= 0 else list(args.mix_output_lengths),
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
        "engine_stats": {k: v for k, v in stats.items() if not isinstance(v, dict) or k == "step_timing"},
        "requests": all_metrics,
    }
    args.output.parent.mkdir(parents=True, exist_ok=True)
    args.output.write_text(json.dumps(result, indent=2, sort_keys=True) + "\n")
    print(json.dumps(result["aggregate"], indent=2, sort_keys=True))
    return 0


if __name__ == "__main__":
    sys.exit(main())
