"""Generates tokens from token ids with a model folder.

    python -m llm_inference_b200.cli.generate --model DIR --prompt-ids 5,17,3 --max-new-tokens 16
        [--temperature 0.8 --top-k 40 --top-p 0.9 --min-p 0.05 --seed 1] [--dtype bfloat16|float32]

Engine options carry the reference's names (python/instinct/mlx_engine.py:70-80,
python/instinct/benchmark.py:396-425).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def add_engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--model", type=Path, default=None, help="folder with config.json and *.safetensors")
    parser.add_argument("--random", default=None, metavar="SHAPE", help="instead of --model: a named shape (cli/presets.py) with seeded random weights drawn on the device")
    parser.add_argument("--weights-seed", type=int, default=0, help="seed of --random's weights")
    parser.add_argument("--backend", choices=["auto", "cuda", "b200"], default="auto", help="kept from the reference's tools; this engine has one backend")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--max-sequences", type=int, default=16)
    parser.add_argument("--max-model-length", type=int, default=2048)
    parser.add_argument("--kv-cache-mib", type=int, default=512)
    parser.add_argument("--page-size", type=int, default=64)
    parser.add_argument("--prefill-chunk-size", type=int, default=512)
    parser.add_argument("--prefill-burst-size", type=int, default=2048)
    parser.add_argument("--no-cuda-graphs", action="store_true")
    parser.add_argument("--kernels", choices=["tuned", "plain"], default="tuned")
    parser.add_argument("--decode-kernel", choices=["chain", "resident"], default="chain",
                        help="'resident': decode steps of up to 16 requests as one resident kernel (slower; an option)")
    parser.add_argument("--step-timing", action="store_true", help="measure host and device time of every model step (reported in the engine's stats)")
    parser.add_argument("--nvtx", action="store_true", help="name NVTX ranges (step, layer N, head, sample) for a profiler's timeline")
    parser.add_argument("--no-run-ahead", action="store_true", help="never launch a decode step before the previous one was read back")


def engine_from(args):
    from .. import create_engine

    options = dict(
        dtype=args.dtype, max_num_sequences=args.max_sequences, max_model_length=args.max_model_length,
        kv_cache_bytes=args.kv_cache_mib << 20, page_size=args.page_size, prefill_chunk_size=args.prefill_chunk_size,
        prefill_burst_size=max(args.prefill_burst_size, args.prefill_chunk_size), cuda_graphs=not args.no_cuda_graphs,
        run_ahead=not args.no_run_ahead, kernels=args.kernels, decode_kernel=args.decode_kernel, nvtx=args.nvtx, step_timing=args.step_timing,
    )
    if (args.model is None) == (args.random is None):
        raise SystemExit("give either --model DIR or --random SHAPE")
    if args.random is not None:
        from ..config import parse_config
        from ..engine.loading import random_model
        from .presets import PRESETS

        if args.random not in PRESETS:
            raise SystemExit(f"--random {args.random!r}: known shapes are {', '.join(sorted(PRESETS))}")
        _, config = parse_config(PRESETS[args.random])
        options["model"] = random_model(config, seed=args.weights_seed, dtype=args.dtype)
    return create_engine(args.model, backend=args.backend, **options)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    add_engine_options(parser)
    parser.add_argument("--prompt-ids", required=True, help="comma-separated token ids, or @file.json with a list")
    parser.add_argument("--max-new-tokens", type=int, default=32)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=None)
    parser.add_argument("--stop-on-eos", action="store_true", help="stop at the model's end-of-sequence ids")
    args = parser.parse_args(argv)

    from .. import SamplingParams

    if args.prompt_ids.startswith("@"):
        prompt = [int(t) for t in json.loads(Path(args.prompt_ids[1:]).read_text())]
    else:
        prompt = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    sampling = SamplingParams(args.temperature, args.top_p, args.top_k, args.min_p, args.seed)
    with engine_from(args) as engine:
        eos = engine.eos_token_ids if args.stop_on_eos else ()
        tokens = engine.generate(prompt, args.max_new_tokens, eos, sampling=sampling)
    print(json.dumps({"prompt_tokens": len(prompt), "tokens": tokens}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
