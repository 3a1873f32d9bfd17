"""Each part alone against the plain implementation, and toy architectures defined here only:
a mixer with state of its own; another position encoding, a routed feed-forward in some layers
and a layer that runs twice. Each is registered, built and stepped without touching the
framework."""

from __future__ import annotations

import json
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from helpers import TOLERANCE
from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu


def context_for(cache_specs, dtype, runs, starts=None, page_size=8, wanted=()):
    """A real step context (and cache) for requests that feed ``runs[i]`` tokens each."""
    from llm_inference_b200.cache import PagedCache
    from llm_inference_b200.engine.runner import ModelRunner, StepEntry

    device = torch.device("cuda:0")
    cache = PagedCache(cache_specs, dtype=dtype, device=device, page_size=page_size, max_num_sequences=8,
                       max_model_length=256, step_tokens=64, num_pages=64)
    stub = SimpleNamespace(device=device, dtype=dtype)
    runner = ModelRunner(stub, cache, max_batch_tokens=512)
    entries = []
    starts = starts or [0] * len(runs)
    for i, (run, start) in enumerate(zip(runs, starts)):
        cache.open(i + 1)
        cache.manager.ensure(i + 1, start)
        cache.manager.advance(i + 1, start)
        entries.append(StepEntry(i + 1, [0] * run))
    ctx = runner._build_context(entries, starts, list(wanted))
    return runner, cache, ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_feed_forward_embedding_and_head_parts(dtype):
    from llm_inference_b200.parts import PartSpec, build_part
    from llm_inference_b200.weights import random_weights

    name = "float32" if dtype == torch.float32 else "bfloat16"
    hidden, inter, vocab, tokens = 72, 200, 130, 11
    runner, cache, ctx = context_for({}, dtype, [tokens], wanted=[0, 10, 3])
    norm = build_part("norm", PartSpec("rmsnorm", dict(name="n", hidden_size=hidden, eps=1e-5)))
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(prefix="mlp.", hidden_size=hidden, intermediate_size=inter)))
    embedding = build_part("embedding", PartSpec("token_embedding", dict(name="emb", vocab_size=vocab, hidden_size=hidden)))
    head = build_part("head", PartSpec("linear_head", dict(name="head", vocab_size=vocab, hidden_size=hidden, tied_to="emb")))
    specs = norm.tensor_specs() + ffn.tensor_specs() + embedding.tensor_specs()
    weights = random_weights(specs, seed=9, std=0.3)
    for part in (norm, ffn, embedding, head):
        part.load(weights, dtype, ctx.device)
    as64 = {k: v.double().numpy() for k, v in weights.items()}
    ids = torch.randint(0, vocab, (tokens,), dtype=torch.int32)
    ctx.token_ids.copy_(ids.cuda())
    x = embedding.forward(ctx)
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), weights["emb.weight"].float()[ids.long()])
    delta = (torch.randn(tokens, hidden) * 0.5).to(dtype).cuda()
    want_x = x.double().cpu().numpy() + delta.double().cpu().numpy()
    h = norm.forward(ctx, x, delta)
    np.testing.assert_allclose(h.double().cpu().numpy(), plain.rms_norm(want_x, as64["n.weight"], 1e-5), atol=TOLERANCE[name], rtol=1e-2)
    out = ffn.forward(ctx, h)
    want = plain.swiglu(h.double().cpu().numpy(), as64["mlp.gate_proj.weight"], as64["mlp.up_proj.weight"], as64["mlp.down_proj.weight"])
    np.testing.assert_allclose(out.double().cpu().numpy(), want, atol=20 * TOLERANCE[name], rtol=2e-2)
    rows = norm.forward(ctx, x, None, rows=ctx.logit_rows, out_name="rows")
    logits = head.forward(ctx, rows)
    assert logits.dtype == torch.float32 and logits.shape == (3, vocab)
    want = plain.linear(rows.double().cpu().numpy(), as64["emb.weight"])
    np.testing.assert_allclose(logits.double().cpu().numpy(), want, atol=10 * TOLERANCE[name], rtol=1e-2)
    head.share(embedding)  # what Model.load does for a tied head
    assert head.weight is embedding.table


def test_rotary_table_matches_plain():
    from llm_inference_b200.parts import PartSpec, build_part

    for dims, theta in ((16, 1e4), (32, 1e6), (128, 1e6)):
        part = build_part("position", PartSpec("rotary", dict(head_dim=dims, theta=theta)))
        assert np.array_equal(part.table(), plain.rope_inverse_frequencies(dims, theta))
    partial = build_part("position", PartSpec("rotary", dict(head_dim=64, theta=1e4, rotary_dims=16)))
    assert np.array_equal(partial.table(), plain.rope_inverse_frequencies(16, 1e4))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 5])
def test_attention_mixer_alone_in_portions(dtype, window):
    """One attention part, fed a sequence in three portions beside another request."""
    from llm_inference_b200.engine.runner import StepEntry
    from llm_inference_b200.parts import PartSpec, build_part
    from llm_inference_b200.weights import random_weights

    name = "float32" if dtype == torch.float32 else "bfloat16"
    hidden, q_heads, kv_heads, dim, theta = 40, 6, 2, 16, 5e4
    mixer = build_part("mixer", PartSpec("gqa_attention", dict(
        prefix="layers.0.self_attn.", hidden_size=hidden, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim,
        window=window, position=PartSpec("rotary", dict(head_dim=dim, theta=theta)))))
    weights = random_weights(mixer.tensor_specs(), seed=4, std=0.2)
    as64 = {("model." + k): v.double().numpy() for k, v in weights.items()}
    config = dict(num_attention_heads=q_heads, num_key_value_heads=kv_heads, hidden_size=hidden, head_dim=dim,
                  rope_theta=theta, use_sliding_window=bool(window), sliding_window=window, max_window_layers=0)
    total = 19
    h_all = (torch.randn(total, hidden) * 0.7).to(dtype)
    other = (torch.randn(6, hidden) * 0.7).to(dtype)
    want = plain.attention_block(config, as64, 0, h_all.double().numpy(), np.arange(total))
    runner, cache, _ = context_for({0: mixer.cache_spec()}, dtype, [1])
    mixer.load(weights, dtype, torch.device("cuda:0"))
    cache.open(10), cache.open(11)
    got, at = [], 0
    for portion in (7, 2, 10):
        entries = [StepEntry(11, [0] * min(2, 6 - 2 * len(got))), StepEntry(10, [0] * portion)]
        starts = [cache.manager.length(e.request_id) for e in entries]
        for e, s in zip(entries, starts):
            cache.manager.ensure(e.request_id, s + len(e.tokens))
        ctx = runner._build_context(entries, starts, [])
        h = torch.cat([other[starts[0] : starts[0] + len(entries[0].tokens)], h_all[at : at + portion]]).cuda()
        out = mixer.forward(ctx, cache.view(0, True, runner._tables), h)
        got.append(out[len(entries[0].tokens) :].double().cpu().numpy())
        for e, s in zip(entries, starts):
            cache.manager.advance(e.request_id, s + len(e.tokens))
        at += portion
    runner.check()
    np.testing.assert_allclose(np.concatenate(got), want, atol=10 * TOLERANCE[name], rtol=2e-2)


# --- a toy architecture whose mixer keeps state of its own -------------------------------------


def register_toy():
    from llm_inference_b200.config import ModelConfig, register_architecture
    from llm_inference_b200.parts import ModelRecipe, Part, PartSpec, StateSpec, register_part
    from llm_inference_b200.weights import TensorSpec

    class RunningMeanMixer(Part):
        """out[t] = W * mean(h[0..t]) of the request: needs a running sum and a count per request."""

        graph_safe = False

        def __init__(self, *, prefix: str, hidden_size: int) -> None:
            self.prefix, self.hidden_size = prefix, hidden_size

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size))]

        def load(self, tensors, dtype, device):
            self.weight = tensors[self.prefix + "mix.weight"].to(device=device, dtype=dtype)

        def cache_spec(self):
            return StateSpec(((self.hidden_size,), (1,)), (torch.float32, torch.float32))

        def forward(self, ctx, cache, h):
            sums, counts = cache.state
            out = torch.empty_like(h)
            for s in range(ctx.num_seqs):
                slot = int(ctx.host.seq_slot[s])
                a, n = int(ctx.host.seq_q_start[s]), int(ctx.host.seq_q_len[s])
                running = sums[slot] + torch.cumsum(h[a : a + n].float(), 0)
                seen = counts[slot] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)[:, None]
                out[a : a + n] = ((running / seen).to(h.dtype) @ self.weight.t())
                sums[slot] = running[-1]
                counts[slot] = seen[-1]
            return out

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        intermediate_size: int = 0
        rms_norm_eps: float = 1e-6

        @classmethod
        def from_json_dict(cls, raw):
            return cls("ToyStateForCausalLM", raw["vocab_size"], raw["hidden_size"], raw["num_hidden_layers"],
                       raw["max_position_embeddings"], (), raw["intermediate_size"], raw["rms_norm_eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        num_hidden_layers=self.num_hidden_layers, max_position_embeddings=self.max_position_embeddings,
                        intermediate_size=self.intermediate_size, rms_norm_eps=self.rms_norm_eps)

    def recipe(config):
        def norm(name):
            return PartSpec("rmsnorm", dict(name=name, hidden_size=config.hidden_size, eps=config.rms_norm_eps))

        layers = [
            PartSpec("pre_norm_residual", dict(
                mixer=PartSpec("running_mean", dict(prefix=f"layers.{i}.", hidden_size=config.hidden_size)),
                feed_forward=PartSpec("swiglu", dict(prefix=f"layers.{i}.mlp.", hidden_size=config.hidden_size,
                                                     intermediate_size=config.intermediate_size)),
                mixer_norm=norm(f"layers.{i}.norm1"), feed_forward_norm=norm(f"layers.{i}.norm2")))
            for i in range(config.num_hidden_layers)
        ]
        return ModelRecipe(
            config=config,
            embedding=PartSpec("token_embedding", dict(name="embed", vocab_size=config.vocab_size, hidden_size=config.hidden_size)),
            layers=layers, final_norm=norm("norm"),
            head=PartSpec("linear_head", dict(name="head", vocab_size=config.vocab_size, hidden_size=config.hidden_size)))

    register_part("mixer", "running_mean", RunningMeanMixer, replace=True)
    register_architecture("ToyStateForCausalLM", ToyConfig.from_json_dict, recipe, replace=True)
    return ToyConfig


def toy_plain(config, weights, tokens):
    x = weights["embed.weight"][tokens]
    for i in range(config["num_hidden_layers"]):
        p = f"layers.{i}."
        h = plain.rms_norm(x, weights[p + "norm1.weight"], config["rms_norm_eps"])
        means = np.cumsum(h, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
        x = x + means @ weights[p + "mix.weight"].T
        h = plain.rms_norm(x, weights[p + "norm2.weight"], config["rms_norm_eps"])
        x = x + plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, weights["norm.weight"], config["rms_norm_eps"]), weights["head.weight"])


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    from helpers import plain_weights, run_trace
    from llm_inference_b200 import create_engine
    from llm_inference_b200.weights import write_model_folder

    ToyConfig = register_toy()
    config = ToyConfig("ToyStateForCausalLM", 97, 48, 2, 64, (), 80, 1e-6)
    folder = write_model_folder(tmp_path / "toy", config, seed=2, std=0.2)
    raw, weights = plain_weights(folder)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyStateForCausalLM"]
    rng = np.random.default_rng(0)
    a = [int(t) for t in rng.integers(0, 97, 21)]
    b = [int(t) for t in rng.integers(0, 97, 9)]
    with create_engine(folder, dtype="float32", max_num_sequences=3, kv_cache_bytes=1 << 20, page_size=8,
                       prefill_chunk_size=4, prefill_burst_size=6) as engine:
        assert engine.cache.state_slots == 3 and not engine.cache.groups
        # Whole, then in portions beside another request: the state carries across steps,
        # and a slot that is handed out again starts from zero.
        whole = engine.prefill_logits(a)
        np.testing.assert_allclose(whole, toy_plain(raw, weights, a)[-1], atol=1e-4)
        ids = [engine.submit(a, 3), engine.submit(b, 3)]
        while engine.has_work():
            engine.step()
        for rid, prompt in zip(ids, (a, b)):
            tokens, out = list(prompt), []
            for _ in range(3):
                out.append(int(np.argmax(toy_plain(raw, weights, tokens)[-1])))
                tokens.append(out[-1])
            assert engine.request(rid).output == out
        assert engine.stats()["free_state_slots"] == 3


def test_graph_safe_mixer_with_state_is_replayed_but_never_run_ahead(tmp_path):
    """The running-mean mixer again, written with device-side operations only, so that its
    decode steps replay a captured graph. A decode step launched ahead and then dropped would
    advance its state twice: an engine whose model keeps per-request state does not run ahead,
    and the stop token, cancel, late submit and forced token below cost nothing."""
    from helpers import plain_weights
    from llm_inference_b200 import create_engine
    from llm_inference_b200.parts import Part, StateSpec, register_part
    from llm_inference_b200.weights import TensorSpec, write_model_folder

    ToyConfig = register_toy()

    class DeviceRunningMean(Part):
        graph_safe = True

        def __init__(self, *, prefix: str, hidden_size: int) -> None:
            self.prefix, self.hidden_size = prefix, hidden_size

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size))]

        def load(self, tensors, dtype, device):
            self.weight = tensors[self.prefix + "mix.weight"].to(device=device, dtype=dtype)

        def cache_spec(self):
            return StateSpec(((self.hidden_size,), (1,)), (torch.float32, torch.float32))

        def forward(self, ctx, cache, h):
            sums, counts = cache.state
            seq = ctx.token_seq.long()
            first = ctx.seq_q_start.long()
            slots = ctx.seq_slot.long()
            total = torch.cumsum(h.float(), 0)
            inside = total - (total[first] - h.float()[first])[seq]  # running sum within each request's run
            index = torch.arange(h.shape[0], device=h.device) - first[seq]
            running = sums[slots][seq] + inside
            seen = counts[slots][seq] + (index + 1).float()[:, None]
            last = first + ctx.seq_q_len.long() - 1
            sums.index_copy_(0, slots, running[last])
            counts.index_copy_(0, slots, seen[last])
            return (running / seen).to(h.dtype) @ self.weight.t()

    register_part("mixer", "running_mean", DeviceRunningMean, replace=True)
    try:
        config = ToyConfig("ToyStateForCausalLM", 97, 48, 2, 96, (), 80, 1e-6)
        folder = write_model_folder(tmp_path / "toy", config, seed=5, std=0.2)
        raw, weights = plain_weights(folder)
        rng = np.random.default_rng(1)
        prompts = [[int(t) for t in rng.integers(0, 97, n)] for n in (7, 12, 3, 9)]

        def greedy(prompt, count):
            tokens, out = list(prompt), []
            for _ in range(count):
                out.append(int(np.argmax(toy_plain(raw, weights, tokens)[-1])))
                tokens.append(out[-1])
            return out

        long = greedy(prompts[0], 30)
        stop = long[13]
        with create_engine(folder, dtype="float32", max_num_sequences=4, kv_cache_bytes=1 << 20, page_size=8,
                           prefill_chunk_size=4, prefill_burst_size=6, run_ahead=True) as engine:
            assert engine.runner.use_graphs and not engine.run_ahead
            a = engine.submit(prompts[0], 30, [stop])
            b = engine.submit(prompts[1], 24)
            c = engine.submit(prompts[2], 40)
            steps, late = 0, None
            while engine.has_work():
                engine.step()
                steps += 1
                if steps == 9:
                    engine.cancel(c)
                if steps == 14:
                    late = engine.submit(prompts[3], 10)
                if steps == 18:
                    engine.force(b, [1])
            assert engine.runner.graph_replays > 10
            assert engine.stats()["steps_ahead_used"] == 0 and engine.stats()["steps_ahead_dropped"] == 0
            assert engine.request(a).output == long[: long.index(stop) + 1]
            assert engine.request(late).output == greedy(prompts[3], 10)
            got_b = engine.request(b).output
            forced_at = got_b.index(1, 0) if 1 in got_b else None
            assert forced_at is not None
            # Up to the forced token b follows its own greedy path, and after it the path from there.
            assert got_b[:forced_at] == greedy(prompts[1], forced_at)
            assert got_b[forced_at + 1 :] == greedy(prompts[1] + got_b[: forced_at + 1], len(got_b) - forced_at - 1)
            assert engine.stats()["free_state_slots"] == 4
    finally:
        register_toy()  # the host-side mixer again, for whichever test runs next


def register_routed_toy():
    """A second toy architecture, defined here only: a norm of its own (mean-subtracting, with a
    bias) in one layer and before the head, the stock attention mixer with two other
    position encodings (rotary angles of position / 4, as position interpolation does, and in
    the last layer learned per-position offsets, which have no frequency table at all), a routed
    feed-forward (two experts, the better one per token by a 32-bit router) in the odd layers and
    the stock SwiGLU in the even ones, and a run order that visits layer 0 twice."""
    from dataclasses import dataclass

    from llm_inference_b200.config import ModelConfig, register_architecture
    from llm_inference_b200.parts.base import Part, PartSpec, register_part
    from llm_inference_b200.parts.model import LayerCall, ModelRecipe
    from llm_inference_b200.parts.positions import RotaryEncoding
    from llm_inference_b200.weights.loader import TensorSpec

    class SquashedRotary(RotaryEncoding):
        """Rotary encoding at ``position / factor``: the stock rotary part with another table of
        inverse frequencies."""

        def __init__(self, *, head_dim: int, theta: float, factor: float) -> None:
            super().__init__(head_dim=head_dim, theta=theta)
            self.factor = float(factor)

        def table(self):
            return (plain.rope_inverse_frequencies(self.head_dim, self.theta) / np.float32(self.factor)).astype(np.float32)

    class LearnedOffset(Part):
        """No rotation and no frequency table: a learned vector per position, added to every
        query and key head. Written with torch operations on the step's device metadata, which
        is all the mixer's contract with its position part asks for."""

        graph_safe = False

        def __init__(self, *, prefix: str, head_dim: int, max_positions: int) -> None:
            self.prefix, self.head_dim, self.max_positions = prefix, head_dim, max_positions

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "position_offset.weight", (self.max_positions, self.head_dim))]

        def load(self, tensors, dtype, device):
            self.offsets = tensors[self.prefix + "position_offset.weight"].to(device=device, dtype=torch.float32)

        def apply(self, ctx, cache, qkv, bias, q_out, q_heads, kv_heads, head_dim):
            t, d = qkv.shape[0], head_dim
            rows = qkv.float() if bias is None else qkv.float() + bias
            positions = ctx.positions.long()
            offset = self.offsets[positions][:, None, :]
            q = rows[:, : q_heads * d].view(t, q_heads, d) + offset
            k = rows[:, q_heads * d : (q_heads + kv_heads) * d].view(t, kv_heads, d) + offset
            v = rows[:, (q_heads + kv_heads) * d :].view(t, kv_heads, d)
            q_out.copy_(q.reshape(t, q_heads * d))
            if cache.writes:
                page = cache.block_table[ctx.token_seq.long(), positions // cache.page_size].long()
                row = positions % cache.page_size
                cache.keys[page, :, row] = k.to(cache.keys.dtype)
                cache.values[page, :, row] = v.to(cache.values.dtype)
            return q_out

    class CenteredNorm(Part):
        """A norm the framework has never seen: mean-subtracting, with a bias,
        ``y = (v - mean v) / sqrt(var v + eps) * w + b`` for ``v = x + delta``. What the block asks of a
        norm is all it provides: add the pending branch output into the 32-bit stream, return the
        normalised rows in the compute dtype; only the given rows, stream untouched, when asked."""

        graph_safe = False

        def __init__(self, *, name: str, hidden_size: int, eps: float) -> None:
            self.name, self.hidden_size, self.eps = name, hidden_size, float(eps)

        def tensor_specs(self):
            return [TensorSpec(self.name + ".weight", (self.hidden_size,), init="one_plus_normal"),
                    TensorSpec(self.name + ".bias", (self.hidden_size,))]

        def load(self, tensors, dtype, device):
            self.weight = tensors[self.name + ".weight"].to(device=device, dtype=torch.float32)
            self.bias = tensors[self.name + ".bias"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, x, delta, rows=None, out_name="normed"):
            if rows is None:
                if delta is not None:
                    x += delta.float()
                v = x
            else:
                picked = rows.long()
                v = x[picked] if delta is None else x[picked] + delta[picked].float()
            centred = v - v.mean(-1, keepdim=True)
            y = centred * torch.rsqrt(centred.square().mean(-1, keepdim=True) + self.eps) * self.weight + self.bias
            return y.to(ctx.dtype)

    class TwoExperts(Part):
        """``out = p * expert_e(h)`` with ``e = argmax(router(h))`` and ``p`` its softmax
        probability, the router in 32-bit; each expert is down(silu(gate h) * up h)."""

        graph_safe = False

        def __init__(self, *, prefix: str, hidden_size: int, intermediate_size: int) -> None:
            self.prefix, self.hidden_size, self.intermediate_size = prefix, hidden_size, intermediate_size

        def tensor_specs(self):
            p, h, i = self.prefix, self.hidden_size, self.intermediate_size
            specs = [TensorSpec(p + "router.weight", (2, h))]
            for e in range(2):
                specs += [TensorSpec(f"{p}experts.{e}.gate.weight", (i, h)), TensorSpec(f"{p}experts.{e}.up.weight", (i, h)),
                          TensorSpec(f"{p}experts.{e}.down.weight", (h, i))]
            return specs

        def load(self, tensors, dtype, device):
            self.router = tensors[self.prefix + "router.weight"].to(device=device, dtype=torch.float32)
            self.experts = [
                tuple(tensors[f"{self.prefix}experts.{e}.{n}.weight"].to(device=device, dtype=dtype) for n in ("gate", "up", "down"))
                for e in range(2)
            ]

        def weight_bytes(self):
            return sum(t.numel() * t.element_size() for expert in self.experts for t in expert) + self.router.numel() * 4

        def forward(self, ctx, h):
            probs = torch.softmax(h.float() @ self.router.t(), dim=-1)
            choice = probs.argmax(dim=-1)
            out = torch.zeros_like(h)
            for e, (gate, up, down) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows]
                    y = (torch.nn.functional.silu(x @ gate.t()) * (x @ up.t())) @ down.t()
                    out[rows] = (y.float() * probs[rows, e : e + 1]).to(h.dtype)
            return out

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        intermediate_size: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        theta: float = 10000.0
        eps: float = 1e-6

        @classmethod
        def from_json_dict(cls, raw):
            return cls("ToyRoutedForCausalLM", raw["vocab_size"], raw["hidden_size"], raw["num_hidden_layers"],
                       raw["max_position_embeddings"], (), raw["intermediate_size"], raw["heads"], raw["kv_heads"],
                       raw["head_dim"], raw["theta"], raw["eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                        num_hidden_layers=self.num_hidden_layers, max_position_embeddings=self.max_position_embeddings,
                        intermediate_size=self.intermediate_size, heads=self.heads, kv_heads=self.kv_heads,
                        head_dim=self.head_dim, theta=self.theta, eps=self.eps)

    def recipe(config):
        def norm(name):
            return PartSpec("rmsnorm", dict(name=name, hidden_size=config.hidden_size, eps=config.eps))

        def centered(name):
            return PartSpec("centered_norm", dict(name=name, hidden_size=config.hidden_size, eps=config.eps))

        def position(i):
            # The last layer encodes positions by learned offsets, the others by squashed rotation.
            if i == config.num_hidden_layers - 1:
                return PartSpec("learned_offset", dict(prefix=f"layers.{i}.attn.", head_dim=config.head_dim,
                                                       max_positions=config.max_position_embeddings))
            return PartSpec("squashed_rotary", dict(head_dim=config.head_dim, theta=config.theta, factor=4.0))

        def feed_forward(i):
            kind = "two_experts" if i % 2 else "swiglu"
            return PartSpec(kind, dict(prefix=f"layers.{i}.mlp.", hidden_size=config.hidden_size, intermediate_size=config.intermediate_size))

        layers = [
            PartSpec("pre_norm_residual", dict(
                mixer=PartSpec("gqa_attention", dict(
                    prefix=f"layers.{i}.attn.", hidden_size=config.hidden_size, q_heads=config.heads, kv_heads=config.kv_heads,
                    head_dim=config.head_dim, qkv_bias=False, position=position(i))),
                feed_forward=feed_forward(i), mixer_norm=norm(f"layers.{i}.norm1"),
                # Layer 1 normalises its feed-forward input with the toy norm, as the model does its last rows.
                feed_forward_norm=(centered if i == 1 else norm)(f"layers.{i}.norm2")))
            for i in range(config.num_hidden_layers)
        ]
        # Layer 0 runs twice, the second time with a cache of its own.
        order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)] + [LayerCall(i, i + 1) for i in range(2, config.num_hidden_layers)]
        return ModelRecipe(
            config=config,
            embedding=PartSpec("token_embedding", dict(name="embed", vocab_size=config.vocab_size, hidden_size=config.hidden_size)),
            layers=layers, final_norm=centered("norm"), schedule=order,
            head=PartSpec("linear_head", dict(name="head", vocab_size=config.vocab_size, hidden_size=config.hidden_size)))

    register_part("norm", "centered_norm", CenteredNorm, replace=True)
    register_part("position", "squashed_rotary", SquashedRotary, replace=True)
    register_part("position", "learned_offset", LearnedOffset, replace=True)
    register_part("feed_forward", "two_experts", TwoExperts, replace=True)
    register_architecture("ToyRoutedForCausalLM", RoutedConfig.from_json_dict, recipe, replace=True)
    return RoutedConfig


def centered_plain(v, weight, bias, eps):
    centred = v - v.mean(-1, keepdims=True)
    return centred / np.sqrt((centred * centred).mean(-1, keepdims=True) + eps) * weight + bias


def routed_plain(config, weights, tokens):
    positions = np.arange(len(tokens), dtype=np.float32) / np.float32(4.0)
    x = weights["embed.weight"][tokens]
    heads, kv_heads, d = config["heads"], config["kv_heads"], config["head_dim"]
    for i in [0, 1, 0] + list(range(2, config["num_hidden_layers"])):
        p = f"layers.{i}."
        h = plain.rms_norm(x, weights[p + "norm1.weight"], config["eps"])
        q = plain.linear(h, weights[p + "attn.q_proj.weight"]).reshape(len(tokens), heads, d)
        k = plain.linear(h, weights[p + "attn.k_proj.weight"]).reshape(len(tokens), kv_heads, d)
        v = plain.linear(h, weights[p + "attn.v_proj.weight"]).reshape(len(tokens), kv_heads, d)
        if i == config["num_hidden_layers"] - 1:
            offset = weights[p + "attn.position_offset.weight"][: len(tokens), None, :]
            q, k = q + offset, k + offset
        else:
            q, k = plain.rope(q, positions, config["theta"]), plain.rope(k, positions, config["theta"])
        x = x + plain.linear(plain.attention(q, k, v, d**-0.5), weights[p + "attn.o_proj.weight"])
        if i == 1:
            h = centered_plain(x, weights[p + "norm2.weight"], weights[p + "norm2.bias"], config["eps"])
        else:
            h = plain.rms_norm(x, weights[p + "norm2.weight"], config["eps"])
        if i % 2:
            probs = plain.softmax(h @ weights[p + "mlp.router.weight"].T)
            choice = probs.argmax(-1)
            out = np.zeros_like(x)
            for t, e in enumerate(choice):
                w = [weights[f"{p}mlp.experts.{e}.{n}.weight"] for n in ("gate", "up", "down")]
                out[t] = probs[t, e] * plain.swiglu(h[t : t + 1], *w)[0]
            x = x + out
        else:
            x = x + plain.swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"])
    return plain.linear(centered_plain(x, weights["norm.weight"], weights["norm.bias"], config["eps"]), weights["head.weight"])


def test_toy_position_encoding_and_routed_feed_forward_without_touching_the_framework(tmp_path):
    from helpers import plain_weights
    from llm_inference_b200 import create_engine
    from llm_inference_b200.weights import write_model_folder

    RoutedConfig = register_routed_toy()
    config = RoutedConfig("ToyRoutedForCausalLM", 131, 64, 3, 96, (), 48, 4, 2, 16, 500.0, 1e-5)
    folder = write_model_folder(tmp_path / "routed", config, seed=3, std=0.3)
    raw, weights = plain_weights(folder)
    rng = np.random.default_rng(4)
    a = [int(t) for t in rng.integers(0, 131, 37)]
    b = [int(t) for t in rng.integers(0, 131, 11)]
    with create_engine(folder, dtype="float32", max_num_sequences=3, kv_cache_bytes=1 << 20, page_size=8,
                       prefill_chunk_size=5, prefill_burst_size=9) as engine:
        # Layer 0 is called twice: four caches for three layers.
        assert sum(len(g.entries) for g in engine.cache.groups) == 4
        np.testing.assert_allclose(engine.prefill_logits(a), routed_plain(raw, weights, a)[-1], atol=2e-4)
        ids = [engine.submit(a, 4), engine.submit(b, 4)]
        while engine.has_work():
            engine.step()
        for rid, prompt in zip(ids, (a, b)):
            tokens, out = list(prompt), []
            for _ in range(4):
                out.append(int(np.argmax(routed_plain(raw, weights, tokens)[-1])))
                tokens.append(out[-1])
            assert engine.request(rid).output == out
