"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no model code of its own: it loads the model through the
registry, builds the engine's cache and drives :class:`ModelRunner.step`, the same step
function generation uses. The nearest things in the reference are ``prefill_logits``
(python/instinct/mlx_engine.py:544-571) and ``force`` (:236-238).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, ``<out>/<step>.f32`` receives them as little-endian float32
``[wanted, vocab]`` in the order of the entries and of ``want``; after every step a line
``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

DEFAULT_PAGE_SIZE = 64


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, type=Path, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, type=Path, help="folder the logits are written to")
    parser.add_argument(
        "--max-tokens", required=True, type=int,
        help="most tokens live requests hold at any time (each request rounded up to a multiple of 64)",
    )
    parser.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE, help="tokens per cache page (divides 64)")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument(
        "--kernels", choices=["tuned", "plain"], default="tuned",
        help="'plain': the plain attention kernel and the library's matrix products in every step, as the "
        "engine's kernels='plain' (what the tuned kernels are checked against)",
    )
    args = parser.parse_args(argv)
    if args.max_tokens <= 0:
        parser.error("--max-tokens must be positive")
    if args.page_size <= 0 or 64 % args.page_size:
        parser.error("--page-size must divide 64")

    import numpy as np
    import torch

    from ..cache.paged_cache import PagedCache
    from ..engine.loading import load_model
    from ..engine.runner import ModelRunner, StepEntry

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; the engine has no CPU path", file=sys.stderr)
        return 2
    args.out.mkdir(parents=True, exist_ok=True)
    model = load_model(args.model, args.dtype, args.device)
    pool_tokens = math.ceil(args.max_tokens / 64) * 64
    config = model.config
    cache = PagedCache(
        model.cache_specs(),
        dtype=model.dtype,
        device=model.device,
        page_size=args.page_size,
        max_num_sequences=max(4, pool_tokens // 64),
        max_model_length=min(config.max_position_embeddings, pool_tokens),
        step_tokens=pool_tokens,
        num_pages=pool_tokens // args.page_size,
    )
    options = {"attention": "plain", "gemm": "library"} if args.kernels == "plain" else {}
    runner = ModelRunner(model, cache, max_batch_tokens=pool_tokens, options=options)
    ids: dict[str, int] = {}
    next_id = 1

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            name = str(item["id"])
            if name not in ids:
                ids[name] = next_id
                next_id += 1
                cache.open(ids[name])
            entries.append(StepEntry(ids[name], item["tokens"], item.get("want", ())))
        try:
            logits = runner.step(entries)
        except ValueError as error:
            names = {number: name for name, number in ids.items()}
            live = ", ".join(f"{e.request_id} = {names[e.request_id]!r}" for e in entries)
            print(f"trace_run: step {step} refused: {error} (requests by number: {live})", file=sys.stderr)
            return 1
        if logits.shape[0]:
            host = logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            host.tofile(args.out / f"{step}.f32")
        runner.check()
        for name in record.get("end", []):
            name = str(name)
            if name in ids:
                cache.manager.release(ids.pop(name))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
