"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model SHAPE] [--batch B] [--prompt-len P] [--context C]

A *step* is one decode step. The default run uses the layer sizes of the Qwen2.5-1.5B shape
with seeded random bfloat16 weights, eight requests that each hold a 2,048-token prompt and
decode inside a 4,096-token context; it prints one JSON line. ``value`` is decoded tokens per
second timed on the device with CUDA events over K steps of the engine's own step function
(metadata built on the host, copied, CUDA-graph replay); ``e2e`` is the same through the
public entry point with the sampled tokens read back to the host every step. Also on the
line: a 2,048-token prefill, the decode step's achieved bytes per second against the HBM
peak, and decoding at batch 1 and 64. Peaks come from MEASURED_PEAKS.json beside this file
when present, else the fallback figures below.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

# Layer sizes of the Qwen2.5-1.5B shape (python/instinct/backends/dense.py is the model).
MODEL = {
    "architectures": ["Qwen2ForCausalLM"],
    "model_type": "qwen2",
    "num_hidden_layers": 28,
    "hidden_size": 1536,
    "num_attention_heads": 12,
    "num_key_value_heads": 2,
    "head_dim": 128,
    "intermediate_size": 8960,
    "vocab_size": 151936,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "use_sliding_window": False,
    "sliding_window": 32768,
    "max_window_layers": 28,
    "max_position_embeddings": 32768,
    "eos_token_id": 151643,
}
FULL_LAYERS = MODEL["num_hidden_layers"]
PROMPT = 2048
CONTEXT = 4096
PAGE = 64


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"source": "measured"}
            out["hbm_gbs"] = float(raw.get("hbm_gbs") or raw.get("hbm_gb_s") or FALLBACK_PEAKS["hbm_gbs"])
            out["bf16_tflops"] = float(raw.get("bf16_tflops") or FALLBACK_PEAKS["bf16_tflops"])
            if raw.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = (
        "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self) -> None:
        self.lines: list[str] = []
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin: int = 0, end: int | None = None) -> dict:
        clocks, maxima, reasons = [], [], set()
        for line in self.lines[begin:end]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {
            "sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "reasons": sorted(reasons),
            "samples": len(clocks),
        }


REFERENCE_DIR = ROOT / "baseline" / "_ref"
REFERENCE_CONTEXT = 2048  # the longest request the reference's CUDA engine takes (cuda/qwen_model.cu:60-61)


def reference_arm(args) -> int:
    """The unmodified reference, installed offline into baseline/_ref, through its own public API
    (``instinct.create_engine(path, backend="cuda")``, ``submit`` / ``step``): the same model shape with
    seeded random weights written by its own ``write_engine``, the same batch, greedy decoding.
    Its CUDA engine refuses requests longer than 2,048 tokens, so the prompts are 1,024 tokens
    where the headline configuration has 2,048 (``same_config`` is false in the line)."""

    def unavailable(reason: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": reason}))
        return 0

    if args.gpus != 1:
        return unavailable("the reference's CUDA engine runs on one GPU")
    if not (REFERENCE_DIR / "instinct").is_dir():
        return unavailable(
            "the reference is not installed under baseline/_ref (offline install: pip --no-deps from a writable copy, "
            "with the CMake target CUDA::nvToolsExt supplied by baseline/nvtx_shim/project_include.cmake)"
        )
    sys.path.insert(0, str(REFERENCE_DIR))
    try:
        import numpy as np
        import torch

        if not torch.cuda.is_available():
            return unavailable("no CUDA device is visible")
        import instinct
        from instinct.format import ModelConfig, write_engine

        if instinct.CudaEngine is None:
            return unavailable("the reference's CUDA extension did not import")
    except Exception as error:  # noqa: BLE001 (whatever stops the import is the reason)
        return unavailable(f"importing the reference failed: {type(error).__name__}: {error}")

    import tempfile

    shape = MODEL
    if args.model != "qwen2.5-1.5b":
        return unavailable("the reference arm is set up for the headline shape only")
    batch, steps, warmup = args.batch, args.steps, max(3, args.warmup)
    prompt_len = min(args.prompt_len, REFERENCE_CONTEXT // 2)
    new_tokens = REFERENCE_CONTEXT - prompt_len
    rng = np.random.default_rng(0)
    hidden, inter, layers = shape["hidden_size"], shape["intermediate_size"], shape["num_hidden_layers"]
    heads, kv_heads, vocab = shape["num_attention_heads"], shape["num_key_value_heads"], shape["vocab_size"]
    head_dim = hidden // heads

    def draw(*dims, mean=0.0):
        return (mean + 0.02 * rng.standard_normal(dims, dtype=np.float32)).astype(np.float16)

    tensors = {"model.embed_tokens.weight": draw(vocab, hidden), "model.norm.weight": draw(hidden, mean=1.0)}
    for layer in range(layers):
        p = f"model.layers.{layer}."
        tensors[p + "input_layernorm.weight"] = draw(hidden, mean=1.0)
        tensors[p + "post_attention_layernorm.weight"] = draw(hidden, mean=1.0)
        for name, rows in (("q_proj", heads * head_dim), ("k_proj", kv_heads * head_dim), ("v_proj", kv_heads * head_dim)):
            tensors[p + f"self_attn.{name}.weight"] = draw(rows, hidden)
            tensors[p + f"self_attn.{name}.bias"] = draw(rows)
        tensors[p + "self_attn.o_proj.weight"] = draw(hidden, heads * head_dim)
        tensors[p + "mlp.gate_proj.weight"] = draw(inter, hidden)
        tensors[p + "mlp.up_proj.weight"] = draw(inter, hidden)
        tensors[p + "mlp.down_proj.weight"] = draw(hidden, inter)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"]
    config = ModelConfig(
        vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=shape["max_position_embeddings"],
        eos_token_id=int(shape["eos_token_id"]), rope_theta=float(shape["rope_theta"]), rms_norm_eps=float(shape["rms_norm_eps"]),
    )
    try:
        with tempfile.TemporaryDirectory() as tmp:
            path = Path(tmp) / "model.engine"
            write_engine(path, config, tensors, aliases={"lm_head.weight": "model.embed_tokens.weight"})
            del tensors
            kv_bytes = batch * REFERENCE_CONTEXT * 2 * layers * kv_heads * head_dim * 2 + (64 << 20)
            engine = instinct.create_engine(
                path, backend="cuda", max_num_sequences=batch, max_model_length=REFERENCE_CONTEXT, kv_cache_bytes=kv_bytes
            )
            # Prefill of one prompt of the engine's longest length, timed through its own API.
            long_prompt = [int(t) for t in rng.integers(0, vocab, REFERENCE_CONTEXT - 1)]
            engine.generate(long_prompt[:64], 1, [])  # first use: cuBLASLt plans, module load
            begin = time.perf_counter()
            engine.generate(long_prompt, 1, [])
            prefill_s = time.perf_counter() - begin
            ids = [engine.submit([int(t) for t in rng.integers(0, vocab, prompt_len)], new_tokens, []) for _ in range(batch)]
            for _ in range(batch):  # it prefills one waiting request per step
                engine.step()
            for _ in range(warmup):
                engine.step()
            sampler = ClockSampler()
            sampler.start()
            torch.cuda.synchronize()
            mark = sampler.mark()
            begin = time.perf_counter()
            emitted, timed = 0, 0
            room = new_tokens - batch - warmup - 2
            while timed < steps or (time.perf_counter() - begin < MIN_TIMED_S and timed + steps <= room):
                for _ in range(steps):
                    emitted += len(engine.step())  # synchronises its stream; tokens come back to the host
                timed += steps
            elapsed = time.perf_counter() - begin
            clocks = sampler.summary(mark, sampler.mark())
            sampler.stop()
            for rid in ids:
                engine.cancel(rid)
    except Exception as error:  # noqa: BLE001
        return unavailable(f"the reference's CUDA engine failed: {type(error).__name__}: {error}")
    value = emitted / elapsed
    line = {
        "metric": f"decode tok/s (batch {batch}, {prompt_len:,}-token prompts, Qwen2.5-1.5B shape)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": elapsed / timed * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic: seeded random weights N(0,0.02), token ids uniform in the vocabulary",
        "impl": "reference", "same_config": False,
        "config": {
            "model": "Qwen2.5-1.5B shape", "layers": layers, "layers_full": layers, "hidden": hidden, "q_heads": heads,
            "kv_heads": kv_heads, "head_dim": head_dim, "intermediate": inter, "vocab": vocab, "tied_head": True,
            "global_batch": batch, "seq_len": REFERENCE_CONTEXT, "prompt_len": prompt_len, "parallelism": "single GPU",
            "why_not_same": "the reference's CUDA engine takes at most 2,048 tokens per request",
            "timing": "host clock around its Engine.step, which synchronises every step",
        },
        "e2e": {"value": value, "unit": "tokens/s", "steps": timed},
        "prefill": {"value": (REFERENCE_CONTEXT - 1) / prefill_s, "tokens": REFERENCE_CONTEXT - 1, "ms": prefill_s * 1e3},
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


MIN_TIMED_S = 0.5  # a timed region shorter than this is repeated (and the median pass reported)
MAX_PASSES = 40


def linear_flops_per_token(config, layers: int) -> float:
    h, i, d = config.hidden_size, config.intermediate_size, config.head_dim
    qkv = (config.num_attention_heads + 2 * config.num_key_value_heads) * d * h
    o = config.num_attention_heads * d * h
    return 2.0 * layers * (qkv + o + 3 * i * h)


def attention_flops(config, layers: int, tokens: int) -> float:
    return layers * config.num_attention_heads * 4.0 * config.head_dim * tokens * (tokens + 1) / 2.0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=240)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (both numbers are reported)")
    parser.add_argument(
        "--model", choices=["qwen2.5-1.5b", "qwen2.5-7b", "qwen2.5-14b"], default="qwen2.5-1.5b",
        help="layer sizes of another Qwen2.5 shape (the default is the headline configuration)",
    )
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens each request holds before it decodes")
    parser.add_argument("--context", type=int, default=0, help="longest request the engine is built for (default: twice the prompt)")
    parser.add_argument("--no-graphs", action="store_true")
    parser.add_argument("--fold-norms", action="store_true", help="fold the norms of short steps into the products around them")
    parser.add_argument("--decode-kernel", choices=["chain", "resident"], default="chain",
                        help="'resident': time the one-kernel decode step instead of the chain of kernels")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    prompt_len = args.prompt_len
    steps, warmup = args.steps, args.warmup
    # Every request decodes through the timed steps. A pass of `steps` steps is repeated until
    # the timed region is MIN_TIMED_S long (so that the clock sampler sees it and the median
    # is over several passes), for which the requests need room to grow.
    new_tokens = max(256, MAX_PASSES * steps + warmup + 1)
    # The engine is built for twice the prompt (the headline run: 2,048 in 4,096) or for what
    # the timed steps need, whichever is longer.
    context = args.context or max(CONTEXT, 2 * prompt_len)
    if prompt_len + new_tokens > context:  # fewer passes rather than a longer context than asked for
        new_tokens = max(steps + warmup + 1, context - prompt_len)

    import numpy as np
    import torch

    from llm_inference_b200 import models  # noqa: F401
    from llm_inference_b200.config import parse_config
    from llm_inference_b200.engine.engine import Engine
    from llm_inference_b200.engine.loading import random_model
    from llm_inference_b200.engine.runner import StepEntry

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device is visible", file=sys.stderr)
        return 1
    torch.cuda.set_device(0)
    peak = peaks()
    shape = MODEL
    if args.model != "qwen2.5-1.5b":
        from llm_inference_b200.cli.presets import PRESETS

        shape = PRESETS[args.model]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    shape_name = args.model.replace("qwen", "Qwen").replace("b", "B") + " shape"
    raw = dict(shape, num_hidden_layers=args.layers, max_window_layers=args.layers)
    _, config = parse_config(raw)
    if not args.context:
        context = min(context, config.max_position_embeddings)
    if prompt_len < 1 or context < max(PROMPT, prompt_len + new_tokens) or context > config.max_position_embeddings:
        print(f"bench.py: --context {context} must hold the {PROMPT}-token prefill and {prompt_len} + {new_tokens} tokens "
              f"of each request, within the model's {config.max_position_embeddings} positions")
        return 2
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    max_batch = max(64, args.batch)
    budget_tokens = max_batch * (prompt_len + new_tokens + PAGE)
    kv_bytes_per_token = 2 * args.layers * config.num_key_value_heads * config.head_dim * 2
    engine = Engine(
        model=model, max_num_sequences=max_batch, max_model_length=context, kv_cache_bytes=budget_tokens * kv_bytes_per_token,
        page_size=PAGE, prefill_chunk_size=PROMPT, prefill_burst_size=PROMPT, max_batch_tokens=PROMPT + max_batch,
        cuda_graphs=not args.no_graphs, decode_kernel=args.decode_kernel, fold_norms=args.fold_norms,
    )
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(0)
    vocab = config.vocab_size
    weight_bytes = model.weight_bytes()
    sampler = ClockSampler()
    sampler.start()

    def timed(fn, repeat: int) -> float:
        """Median milliseconds of ``fn`` over ``repeat`` runs, on the device."""
        times = []
        for _ in range(repeat):
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        return statistics.median(times)

    # --- prefill of one 2,048-token prompt -------------------------------------------------------
    prompt = [int(t) for t in rng.integers(0, vocab, PROMPT)]
    scratch_id = [10_000]

    def prefill_once() -> None:
        scratch_id[0] += 1
        cache.open(scratch_id[0])
        runner.step([StepEntry(scratch_id[0], prompt, (PROMPT - 1,))])
        cache.manager.release(scratch_id[0])

    for _ in range(3):
        prefill_once()
    prefill_ms = timed(prefill_once, 5)
    prefill_flops = PROMPT * linear_flops_per_token(config, args.layers) + attention_flops(config, args.layers, PROMPT)
    prefill_flops += 2.0 * vocab * config.hidden_size
    prefill = {
        "value": PROMPT / (prefill_ms / 1e3), "tokens": PROMPT, "ms": prefill_ms,
        "frac": prefill_flops / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12),
    }
    if peak.get("bf16_tflops_sustained"):  # the library's rate in a seconds-long loop under the power cap
        prefill["frac_of_sustained"] = prefill_flops / (prefill_ms / 1e3) / (peak["bf16_tflops_sustained"] * 1e12)

    # --- decode, timed on the device -------------------------------------------------------------
    def decode_point(batch: int, k: int, w: int) -> dict:
        ids = list(range(20_000 + 1000 * batch, 20_000 + 1000 * batch + batch))
        for rid in ids:
            cache.open(rid)
            for begin in range(0, prompt_len, PROMPT):  # the prompt goes in by portions of 2,048
                runner.step([StepEntry(rid, [int(t) for t in rng.integers(0, vocab, min(PROMPT, prompt_len - begin))])])
        most_passes = max(1, min(MAX_PASSES, (new_tokens - w - 1) // k))
        feed = rng.integers(0, vocab, size=(w + most_passes * k, batch))

        def one(step: int) -> None:
            runner.step([StepEntry(rid, (int(feed[step, j]),), (0,)) for j, rid in enumerate(ids)])

        for step in range(w):
            one(step)
        torch.cuda.synchronize()
        calls_before = runner.lib.calls
        replays_before = runner.graph_replays
        mark = sampler.mark()
        torch.cuda.nvtx.range_push(f"decode_timed_b{batch}")
        pass_ms, at = [], w
        # Exactly k steps between two events, device-timed; the pass is repeated until the timed
        # passes add up to MIN_TIMED_S, and the median pass is the one reported.
        while len(pass_ms) < most_passes and (not pass_ms or sum(pass_ms) < MIN_TIMED_S * 1e3):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for step in range(at, at + k):
                one(step)
            end.record()
            torch.cuda.synchronize()
            pass_ms.append(start.elapsed_time(end))
            at += k
        torch.cuda.nvtx.range_pop()
        ms = statistics.median(pass_ms) / k
        replays = runner.graph_replays - replays_before
        launches = (runner.lib.calls - calls_before) + replays * runner.launches_per_graph.get(runner._bucket(batch), 0)
        launches //= len(pass_ms)
        mean_context = prompt_len + (w + at) / 2.0
        step_bytes = weight_bytes + batch * mean_context * kv_bytes_per_token
        runner.check()
        for rid in ids:
            cache.manager.release(rid)
        return {
            "tokens_per_s": batch * 1e3 / ms, "ms_per_step": ms, "bytes": step_bytes, "launches": launches,
            "clocks": sampler.summary(mark, sampler.mark()), "passes": len(pass_ms),
        }

    main_point = decode_point(args.batch, steps, warmup)
    points = {}
    if not args.no_points:
        for batch in (1, 64):
            points[f"decode_b{batch}"] = decode_point(batch, max(16, steps // 2), warmup)["tokens_per_s"]
        # The same steps with the slow, simple kernels the tuned ones are checked against (the plain
        # attention kernel, the library's matrix products everywhere): a stated baseline of this
        # repository's own, since the reference's CUDA engine does not run (see --impl reference).
        saved = {name: runner.options.get(name) for name in ("attention", "gemm")}
        runner.options.update(attention="plain", gemm="library")
        runner._graphs.clear()
        points[f"decode_b{args.batch}_plain_kernels"] = decode_point(args.batch, max(16, steps // 2), warmup)["tokens_per_s"]
        for name, value in saved.items():
            if value is None:
                runner.options.pop(name, None)
            else:
                runner.options[name] = value
        runner._graphs.clear()

    # --- the same through the public entry point: host tokens in and out ------------------------
    prompts = [[int(t) for t in rng.integers(0, vocab, prompt_len)] for _ in range(args.batch)]
    request_ids = [engine.submit(p, new_tokens) for p in prompts]
    while any(engine.request(r).state.value in ("waiting", "prefilling") for r in request_ids):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    begin = time.perf_counter()
    emitted, e2e_steps = 0, 0
    room = new_tokens - warmup - 2  # the requests must still be decoding when the clock stops
    while e2e_steps < steps or (time.perf_counter() - begin < MIN_TIMED_S and e2e_steps + steps <= room):
        for _ in range(steps):
            emitted += len(engine.step())
        e2e_steps += steps
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    for r in request_ids:
        engine.cancel(r)
    # One pinned-to-device copy of the step's metadata (tokens, positions, lengths, block tables,
    # padded to the captured batch size) and one device-to-host read of the sampled tokens.
    bucket = runner._bucket(args.batch)
    layout_words = 3 * bucket + 4 * bucket + bucket + len(cache.groups) * bucket * cache.max_pages_per_request
    e2e = {
        "value": emitted / elapsed, "unit": "tokens/s", "h2d_bytes_per_step": 4 * layout_words,
        "d2h_bytes_per_step": 4 * (args.batch + 1), "steps": e2e_steps,
    }
    sampler.stop()

    achieved = main_point["bytes"] / (main_point["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s (batch {args.batch}, {prompt_len:,}-token prompts, {shape_name})",
        "value": main_point["tokens_per_s"],
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "timed_passes": main_point["passes"],
        "ms_per_step": main_point["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), token ids uniform in the vocabulary",
        "impl": "ours",
        "config": {
            "model": shape_name,
            "layers": args.layers,
            "layers_full": full_layers,
            "hidden": config.hidden_size,
            "q_heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "intermediate": config.intermediate_size,
            "vocab": config.vocab_size,
            "tied_head": config.tie_word_embeddings,
            "global_batch": args.batch,
            "seq_len": context,
            "prompt_len": prompt_len,
            "page_size": PAGE,
            "parallelism": "single GPU",
            "cuda_graphs": not args.no_graphs,
            "decode_kernel": args.decode_kernel,
            "l2": "inputs larger than L2: each step reads all weights (GBs)",
            "peaks": peak["source"],
        },
        "e2e": e2e,
        "gpu_launches": main_point["launches"],
        "prefill": prefill,
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peak["hbm_gbs"],
        },
        "points": points,
        "clocks": main_point["clocks"],
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
