"""Generation through the Python entry point: scheduler, step function, sampling together."""

from __future__ import annotations

import numpy as np
import pytest

from helpers import PAGE_SIZE, TINY, TOLERANCE, make_model_folder, plain_weights, random_tokens
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, tmp_path_factory):
    name = request.param
    folder = make_model_folder(tmp_path_factory.mktemp(f"engine{name}"), TINY[name], seed=23 + ord(name))
    config, weights = plain_weights(folder)
    return name, folder, config, weights


def engine_for(name, folder, dtype="float32", **options):
    from llm_inference_b200 import create_engine

    settings = dict(
        max_num_sequences=4, kv_cache_bytes=1 << 20, prefill_chunk_size=7, prefill_burst_size=16,
        page_size=PAGE_SIZE[name], dtype=dtype,
    )
    settings.update(options)
    return create_engine(folder, **settings)


def drained(engine) -> bool:
    pools = engine.stats()["kv_pools"].values()
    return all(p["used_pages"] == 0 and p["reserved_pages"] == 0 for p in pools)


def run_all(engine, prompts, count, **options):
    ids = [engine.submit(p, count, **options) for p in prompts]
    while engine.has_work():
        engine.step()
    return [engine.request(i).output for i in ids]


@pytest.mark.parametrize("length", [1, 3, 7, 8, 9, 16, 17, 33, 60])
def test_prefill_logits_across_page_and_chunk_edges(tiny, length):
    name, folder, config, weights = tiny
    prompt = random_tokens(np.random.default_rng(length), config["vocab_size"], length)
    with engine_for(name, folder) as engine:
        got = engine.prefill_logits(prompt)
        assert drained(engine)
    want = plain.forward(config, weights, prompt)[-1]
    assert np.abs(got - want).max() <= TOLERANCE["float32"]


def test_greedy_generation_matches_plain(tiny):
    name, folder, config, weights = tiny
    prompt = random_tokens(np.random.default_rng(1), config["vocab_size"], 6)
    count = 90 if name == "A" else 60  # long decoding: many pages, and past the window for B
    want = plain.greedy(config, weights, prompt, count)
    with engine_for(name, folder) as engine:
        assert engine.generate(prompt, count) == want
        assert drained(engine)
        assert engine.stats()["generated_tokens"] == count


def test_bfloat16_greedy_follows_plain_until_a_near_tie(tiny):
    name, folder, config, weights = tiny
    prompt = random_tokens(np.random.default_rng(2), config["vocab_size"], 9)
    with engine_for(name, folder, dtype="bfloat16") as engine:
        got = engine.generate(prompt, 24)
    tokens = list(prompt)
    for step, token in enumerate(got):
        logits = plain.forward(config, weights, tokens)[-1]
        best = int(np.argmax(logits))
        if token != best:
            # Allowed only where bfloat16 rounding can flip the order; later tokens then differ.
            assert logits[best] - logits[token] <= 2 * TOLERANCE["bfloat16"], f"step {step}"
            break
        tokens.append(token)


def test_plain_kernels_option_gives_the_same_greedy_tokens(tiny):
    """`kernels="plain"`: plain attention and library products instead of the tuned kernels."""
    name, folder, config, weights = tiny
    prompt = random_tokens(np.random.default_rng(8), config["vocab_size"], 19)
    want = plain.greedy(config, weights, prompt, 12)
    with engine_for(name, folder, kernels="plain") as engine:
        assert engine.generate(prompt, 12) == want
    with engine_for(name, folder, dtype="bfloat16", kernels="plain") as slow, engine_for(name, folder, dtype="bfloat16") as fast:
        a, b = slow.prefill_logits(prompt), fast.prefill_logits(prompt)
        assert np.abs(a - b).max() <= 2 * TOLERANCE["bfloat16"]
    with pytest.raises(ValueError):
        engine_for(name, folder, kernels="fastest")


def test_batched_requests_match_running_alone(tiny):
    name, folder, config, weights = tiny
    vocab = config["vocab_size"]
    prompts = [[(i * 7 + j) % vocab for i in range(n)] for j, n in enumerate([1, 4, 9, 13, 21, 30])]
    with engine_for(name, folder, max_num_sequences=3) as engine:
        alone = [engine.generate(p, 8) for p in prompts]
        together = run_all(engine, prompts, 8)
        assert together == alone
        assert drained(engine)
    assert alone[2] == plain.greedy(config, weights, prompts[2], 8)


def test_seeded_sampling_is_independent_of_the_batch(tiny):
    from llm_inference_b200 import SamplingParams

    name, folder, config, weights = tiny
    vocab = config["vocab_size"]
    rng = np.random.default_rng(3)
    prompts = [random_tokens(rng, vocab, n) for n in (1, 23, 40, 70)]
    seeded = SamplingParams(temperature=0.8, seed=1234)
    with engine_for(name, folder) as engine:
        alone = engine.generate(prompts[1], 12, sampling=seeded)
        ids = [
            engine.submit(prompts[0], 12),
            engine.submit(prompts[1], 12, sampling=seeded),
            engine.submit(prompts[2], 12, sampling=SamplingParams(temperature=0.8, seed=77)),
            engine.submit(prompts[3], 12, sampling=SamplingParams(temperature=1.5, top_k=5)),
        ]
        # Staggered arrivals: the later prompts join while the first are decoding.
        while engine.has_work():
            engine.step()
        outputs = [engine.request(i).output for i in ids]
        assert outputs[1] == alone
        assert outputs[0] == plain.greedy(config, weights, prompts[0], 12)
        assert engine.generate(prompts[1], 12, sampling=SamplingParams(temperature=0.8, top_k=1)) == plain.greedy(
            config, weights, prompts[1], 12
        )
        assert drained(engine)
    # Each seeded draw is the plain sampler's inverse-CDF pick at the engine's own uniform.
    tokens = list(prompts[1])
    for step, token in enumerate(alone):
        logits = plain.forward(config, weights, tokens)[-1]
        probs = plain.surviving_probabilities(logits, 0.8)
        cdf = np.cumsum(probs)
        u = plain.uniform_from_key(plain.draw_key(1234, step))
        expected = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
        if token != expected:
            # Only a draw that lands within rounding of a boundary of the CDF may differ.
            assert min(abs(u * cdf[-1] - cdf[expected]), abs(u * cdf[-1] - cdf[max(expected - 1, 0)])) < 1e-4
            break
        tokens.append(token)


def test_window_pool_stays_bounded(tmp_path_factory):
    folder = make_model_folder(tmp_path_factory.mktemp("window"), TINY["B"], seed=5)
    with engine_for("B", folder, prefill_chunk_size=8, prefill_burst_size=8) as engine:
        rid = engine.submit([1] * 40, 150)
        peak_window, peak_full = 0, 0
        while engine.has_work():
            engine.step()
            pools = engine.stats()["kv_pools"]
            peak_window = max(peak_window, pools["window24"]["used_pages"])
            peak_full = max(peak_full, pools["full"]["used_pages"])
        assert len(engine.request(rid).output) == 150
        assert peak_window <= 5  # ceil((24 + 8) / 8) + 1
        assert peak_full == (40 + 150 - 1 + 7) // 8
        assert drained(engine)


def test_cancel_errors_and_close(tiny):
    name, folder, config, weights = tiny
    engine = engine_for(name, folder)
    rid = engine.submit([1] * 30, 4)
    engine.step()  # part of the prompt is in the cache
    assert engine.request(rid).state.value == "prefilling"
    engine.cancel(rid)
    assert engine.request(rid).state.value == "cancelled" and drained(engine)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.submit([config["vocab_size"]], 1)
    with pytest.raises(ValueError, match="exceed"):
        engine.submit([1] * 100, config["max_position_embeddings"])
    with pytest.raises(ValueError, match="positive integer"):
        engine.submit([1], 0)
    with pytest.raises(ValueError, match="non-empty"):
        engine.submit([], 3)
    rid = engine.submit([3, 4], 5, eos_token_ids=[9])
    engine.force(rid, [8, 9])
    events = []
    while engine.has_work():
        events += engine.step()
    assert [(e.token, e.finished, e.reason) for e in events] == [(8, False, ""), (9, True, "stop")]
    stats = engine.stats()
    for key in ("submitted", "completed", "cancelled", "prompt_tokens", "generated_tokens", "steps", "running",
                "waiting", "kv_pools", "kv_device_bytes", "allocation_failures", "live_tokens", "weight_bytes"):
        assert key in stats
    engine.close()
    with pytest.raises(RuntimeError, match="closed"):
        engine.step()


def test_requests_wait_when_pages_run_out(tiny):
    name, folder, config, weights = tiny
    page = PAGE_SIZE[name]
    # Room for about two of these requests at a time.
    with engine_for(name, folder, num_pages=(2 * 48) // page + 1, max_num_sequences=4) as engine:
        prompts = [[(3 * i + j) % 200 + 1 for i in range(30)] for j in range(5)]
        ids = [engine.submit(p, 12) for p in prompts]
        most_running = 0
        while engine.has_work():
            engine.step()
            most_running = max(most_running, engine.stats()["running"])
        assert most_running <= 2 and engine.stats()["allocation_failures"] > 0
        assert [engine.request(i).output for i in ids] == [plain.greedy(config, weights, p, 12) for p in prompts]
        assert drained(engine)
        with pytest.raises(ValueError, match="more K/V memory than the cache has"):
            engine.submit([1] * 100, 20)


def test_steps_launched_ahead_change_nothing(tiny):
    """With `run_ahead` a decode step is launched before the previous step's tokens reach the
    host. A request that ends on a stop token, one that is cancelled, one submitted late and a
    forced token all make such a step unwanted; the tokens must be those of an engine that
    never runs ahead, and those of the plain implementation."""
    name, folder, config, weights = tiny
    rng = np.random.default_rng(11)
    vocab = config["vocab_size"]
    prompts = [random_tokens(rng, vocab, n) for n in (5, 9, 3, 12)]
    long = plain.greedy(config, weights, prompts[0], 40)
    stop = long[17]  # request 0 ends on this token (its first occurrence decides where)

    def scenario(run_ahead: bool):
        with engine_for(name, folder, run_ahead=run_ahead) as engine:
            a = engine.submit(prompts[0], 40, [stop])
            b = engine.submit(prompts[1], 33)
            c = engine.submit(prompts[2], 50)
            steps = 0
            late = None
            while engine.has_work():
                engine.step()
                steps += 1
                if steps == 12:
                    engine.cancel(c)
                if steps == 20:
                    late = engine.submit(prompts[3], 14)
                if steps == 25:
                    engine.force(b, [1])
            outputs = [list(engine.request(r).output) for r in (a, b, c, late)]
            stats = engine.stats()
            assert drained(engine)
        return outputs, stats

    with_ahead, stats = scenario(True)
    without, stats_without = scenario(False)
    assert with_ahead == without
    assert stats_without["steps_ahead_used"] == 0 and stats_without["steps_ahead_dropped"] == 0
    assert stats["steps_ahead_used"] > 10 and stats["steps_ahead_dropped"] >= 1
    assert with_ahead[0] == long[: long.index(stop) + 1]
    assert with_ahead[3] == plain.greedy(config, weights, prompts[3], 14)


def test_sampled_tokens_do_not_depend_on_running_ahead(tiny):
    name, folder, config, _ = tiny
    rng = np.random.default_rng(12)
    prompts = [random_tokens(rng, config["vocab_size"], n) for n in (4, 11)]
    from llm_inference_b200 import SamplingParams

    options = dict(sampling=SamplingParams(temperature=0.9, top_k=20, top_p=0.95, seed=77))
    with engine_for(name, folder, run_ahead=True) as engine:
        ahead = run_all(engine, prompts, 30, **options)
        assert engine.stats()["steps_ahead_used"] > 10
    with engine_for(name, folder, run_ahead=False) as engine:
        assert run_all(engine, prompts, 30, **options) == ahead


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_workloads_are_the_same_with_and_without_running_ahead(tiny, seed):
    """Requests of random lengths arrive, stop on tokens, hit their limits and are cancelled at
    random steps; every request's tokens must not depend on whether steps are launched ahead."""
    name, folder, config, _ = tiny
    vocab = config["vocab_size"]

    def scenario(run_ahead: bool):
        rng = np.random.default_rng(100 + seed)
        with engine_for(name, folder, run_ahead=run_ahead, kv_cache_bytes=1 << 20) as engine:
            ids = []
            for step in range(160):
                if step < 90 and rng.random() < 0.18:
                    prompt = random_tokens(rng, vocab, int(rng.integers(1, 30)))
                    stops = [int(t) for t in rng.integers(0, vocab, int(rng.integers(0, 4)))]
                    ids.append(engine.submit(prompt, int(rng.integers(1, 40)), stops))
                if ids and rng.random() < 0.04:
                    engine.cancel(ids[int(rng.integers(0, len(ids)))])
                engine.step()
            while engine.has_work():
                engine.step()
            outputs = [(engine.request(r).state, list(engine.request(r).output)) for r in ids]
            stats = engine.stats()
            assert drained(engine)
        return outputs, stats

    ahead, stats = scenario(True)
    behind, _ = scenario(False)
    assert ahead == behind
    assert stats["steps_ahead_used"] > 0 and stats["steps_ahead_dropped"] > 0


@pytest.mark.parametrize("where", ["model step", "sampler"])
def test_a_failing_step_cancels_its_requests_and_the_engine_goes_on(tiny, where):
    """What the reference does when a step throws (python/instinct/mlx_engine.py:419-423,
    cuda/engine.cu:85-89,108-112): every request of that step ends as cancelled with reason
    "error", what they held goes back, the error reaches the caller, and the engine serves
    the next request. The failure is made on the host: the model step (or the sampler's
    launch) is replaced by a function that raises."""
    name, folder, config, weights = tiny
    rng = np.random.default_rng(31)
    prompts = [random_tokens(rng, config["vocab_size"], n) for n in (6, 11, 4)]

    class Injected(RuntimeError):
        pass

    with engine_for(name, folder) as engine:
        a, b = engine.submit(prompts[0], 30), engine.submit(prompts[1], 30)
        for _ in range(6):  # both are decoding by now, and a step launched ahead is in flight
            engine.step()
        assert engine.request(a).state.value == "running" and engine.request(b).state.value == "running"
        assert engine._ahead is not None
        waiting = engine.submit(prompts[2], 5)  # admitted by the failing step's plan: part of it
        target, attribute = (engine.runner, "step") if where == "model step" else (engine.sampler, "launch")
        original = getattr(target, attribute)

        def fail(*args, **kwargs):
            raise Injected("injected on the host")

        setattr(target, attribute, fail)
        with pytest.raises(Injected):
            engine.step()
        setattr(target, attribute, original)
        for rid in (a, b, waiting):
            view = engine.request(rid)
            assert view.state.value == "cancelled" and view.reason == "error", (rid, view.state, view.reason)
        assert engine._ahead is None and not engine.has_work() and drained(engine)
        engine.cache.manager.check_invariants()
        # The engine is still good: a new request gets the plain implementation's tokens.
        assert engine.generate(prompts[1], 8) == plain.greedy(config, weights, prompts[1], 8)
        # generate() itself: the failing request is cancelled and forgotten, the error re-raised.
        setattr(target, attribute, fail)
        before = engine.stats()["cancelled"]
        with pytest.raises(Injected):
            engine.generate(prompts[0], 4)
        setattr(target, attribute, original)
        assert engine.stats()["cancelled"] == before + 1 and not engine.has_work() and drained(engine)
        assert engine.generate(prompts[2], 5) == plain.greedy(config, weights, prompts[2], 5)


# --- the scheduler's path over the tensor-core kernels ---------------------------------------------
#
# The tiny configurations have heads of 16 and 32, which in bfloat16 run the plain attention
# kernel. These two models have heads of 128 and 64 and pages of 64: their prompt portions run the
# tcgen05 (or mma.sync) prefill kernel, their decode steps the split-key kernels fed by TMA (or
# cp.async), replayed from captured graphs and launched ahead of the host. Queries and keys are
# scaled up so that attention picks few keys and a wrong one changes the greedy token.


@pytest.fixture(scope="module", params=["heads_of_128", "heads_of_64"])
def heads(request, tmp_path_factory):
    from helpers import OTHER_SIZES, SHARPENED, sharpen_attention

    name = request.param
    folder = make_model_folder(tmp_path_factory.mktemp(name), OTHER_SIZES[name], seed=41)
    sharpen_attention(folder, SHARPENED[name])
    config, weights = plain_weights(folder)
    return name, folder, config, weights


def heads_engine(folder, **options):
    from llm_inference_b200 import create_engine

    settings = dict(max_num_sequences=4, kv_cache_bytes=8 << 20, prefill_chunk_size=48, prefill_burst_size=96, dtype="bfloat16")
    settings.update(options)
    return create_engine(folder, **settings)


def follows_plain_until_a_near_tie(config, weights, prompt, got, what) -> int:
    """Every token is the plain implementation's greedy pick, up to the first place where the
    plain logits of the two picks lie within bfloat16's reach of each other; returns how many
    tokens were checked."""
    tokens = list(prompt)
    for step, token in enumerate(got):
        logits = plain.forward(config, weights, tokens)[-1]
        best = int(np.argmax(logits))
        if token != best:
            assert logits[best] - logits[token] <= 2 * TOLERANCE["bfloat16"], f"{what}: step {step}"
            return step
        tokens.append(token)
    return len(got)


def test_scheduler_over_the_tensor_core_kernels_follows_plain(heads):
    name, folder, config, weights = heads
    rng = np.random.default_rng(5)
    prompts = [random_tokens(rng, config["vocab_size"], n) for n in (150, 70, 97, 201)]
    with heads_engine(folder) as engine:
        alone = [engine.generate(p, 20) for p in prompts]
        together = run_all(engine, prompts, 20)
        stats = engine.stats()
        assert drained(engine)
    assert engine.runner.graph_replays > 20 and stats["steps_ahead_used"] > 20
    checked = [follows_plain_until_a_near_tie(config, weights, p, out, f"{name} alone {i}") for i, (p, out) in enumerate(zip(prompts, alone))]
    assert sum(checked) >= 40, checked  # most tokens are decided well clear of a tie
    for i, (p, out) in enumerate(zip(prompts, together)):
        follows_plain_until_a_near_tie(config, weights, p, out, f"{name} together {i}")
    # Batched beside other requests or alone: the same kernels at other batch sizes; the tokens
    # agree until a near-tie (equality across batch sizes is to rounding, not to the bit).
    for p, a, b in zip(prompts, alone, together):
        if a != b:
            first = next(i for i, (x, y) in enumerate(zip(a, b)) if x != y)
            logits = plain.forward(config, weights, list(p) + a[:first])[-1]
            assert abs(logits[a[first]] - logits[b[first]]) <= 2 * TOLERANCE["bfloat16"]


def test_run_ahead_over_the_tensor_core_kernels_changes_nothing(heads):
    """The run-ahead scenario (a stop token, a cancel, a late submit, a forced token) at heads of
    128 and 64: the same tokens with and without steps launched ahead."""
    name, folder, config, weights = heads
    rng = np.random.default_rng(6)
    prompts = [random_tokens(rng, config["vocab_size"], n) for n in (90, 130, 65, 77)]
    with heads_engine(folder, run_ahead=False) as engine:
        long = engine.generate(prompts[0], 40)
    stop = long[17]

    def scenario(run_ahead: bool):
        with heads_engine(folder, run_ahead=run_ahead) as engine:
            a = engine.submit(prompts[0], 40, [stop])
            b = engine.submit(prompts[1], 33)
            c = engine.submit(prompts[2], 50)
            steps, late = 0, None
            while engine.has_work():
                engine.step()
                steps += 1
                if steps == 12:
                    engine.cancel(c)
                if steps == 20:
                    late = engine.submit(prompts[3], 14)
                if steps == 25:
                    engine.force(b, [1])
            outputs = [list(engine.request(r).output) for r in (a, b, c, late)]
            stats = engine.stats()
            assert drained(engine)
        return outputs, stats

    with_ahead, stats = scenario(True)
    without, _ = scenario(False)
    assert with_ahead == without
    assert stats["steps_ahead_used"] > 10 and stats["steps_ahead_dropped"] >= 1
    assert with_ahead[0] == long[: long.index(stop) + 1]
    follows_plain_until_a_near_tie(config, weights, prompts[3], with_ahead[3], f"{name} late request")


def test_pages_with_non_finite_leftovers_are_harmless(heads):
    """Pages go from request to request without being cleared, and the tensor-core attention
    kernels load whole tiles of a page, masking rows past a request's last key only in the
    scores. Here every page is filled with NaN between two runs of the same request: the
    token that starts a page clears the rows its request has not written yet, so the second
    run gives the first run's tokens and logits (prefill, then decode steps from graphs)."""
    import torch

    name, folder, config, weights = heads
    prompt = random_tokens(np.random.default_rng(7), config["vocab_size"], 150)
    with heads_engine(folder) as engine:
        first_logits = engine.prefill_logits(prompt)
        first = engine.generate(prompt, 12)
        assert drained(engine)
        torch.cuda.synchronize()
        for group in engine.cache.groups:
            group.arena[:, :, : group.capacity_pages].fill_(float("nan"))  # all but the spare page of padded rows
        again_logits = engine.prefill_logits(prompt)
        again = engine.generate(prompt, 12)
    assert np.isfinite(again_logits).all()
    assert np.array_equal(first_logits, again_logits) and first == again
    follows_plain_until_a_near_tie(config, weights, prompt, first, f"{name} after NaN pages")
