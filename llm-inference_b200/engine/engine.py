"""The request API: ``create_engine`` and :class:`Engine` (submit / step / cancel / generate / stats).

Names and meanings follow the reference's engines: ``MlxEngine``
(python/instinct/mlx_engine.py:64-625) for behaviour and options, and the native module's
``Engine`` (python/bindings.cpp:47-90) for the constructor's positional form. Admission,
the step's plan and finishing are the C++ scheduler's; the model step is
:class:`ModelRunner.step`; sampling runs on the device.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Iterable

import numpy as np
import torch

from ..cache.paged_cache import PagedCache
from ..csrc import build
from ..csrc.host_module import host
from ..csrc.library import KernelError, check_error_word
from ..parts.model import Model
from ..sampling.params import GREEDY, SamplingParams
from ..sampling.sampler import Sampler
from .loading import load_model, parse_dtype
from .runner import ModelRunner, StepEntry

PAGE_SIZE = 64


class SequenceState(Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    RUNNING = "running"
    COMPLETED = "completed"
    CANCELLED = "cancelled"
    REJECTED = "rejected"


TERMINAL = frozenset({SequenceState.COMPLETED, SequenceState.CANCELLED, SequenceState.REJECTED})


@dataclass(frozen=True)
class TokenEvent:
    request_id: int
    token: int
    finished: bool
    # Set together with `finished`: "stop" when one of the request's stop tokens came out,
    # "length" when max_new_tokens were produced, "context" when the next position would pass
    # the engine's length limit.
    reason: str = ""


@dataclass(frozen=True)
class RequestView:
    """A snapshot of one request."""

    request_id: int
    state: SequenceState
    prompt: np.ndarray
    output: list[int]
    reason: str
    length: int
    max_new_tokens: int


def build_info() -> dict[str, object]:
    info: dict[str, object] = {
        "backend": "b200",
        "arch": "sm_100a",
        "build_dir": str(build.build_dir()),
        "torch": torch.__version__,
        "cuda_available": torch.cuda.is_available(),
    }
    if torch.cuda.is_available():
        info["device"] = torch.cuda.get_device_name(0)
    return info


class Engine:
    backend = "b200"

    def __init__(
        self,
        model_path: str | Path | None = None,
        max_num_sequences: int = 16,
        max_model_length: int | None = None,
        kv_cache_bytes: int = 4 << 30,
        *,
        prefill_chunk_size: int = 512,
        prefill_burst_size: int = 2048,
        max_batch_tokens: int | None = None,
        page_size: int = PAGE_SIZE,
        dtype: str | torch.dtype = "bfloat16",
        device: str | torch.device = "cuda:0",
        seed: int = 0,
        num_pages: int | None = None,
        cuda_graphs: bool = True,
        run_ahead: bool = True,
        kernels: str = "tuned",
        decode_kernel: str = "chain",
        fold_norms: bool = False,
        nvtx: bool = False,
        step_timing: bool = False,
        model: Model | None = None,
    ) -> None:
        if kernels not in ("tuned", "plain"):
            raise ValueError(f"kernels={kernels!r}; expected 'tuned' or 'plain'")
        if decode_kernel not in ("chain", "resident"):
            raise ValueError(f"decode_kernel={decode_kernel!r}; expected 'chain' or 'resident'")
        if max_num_sequences <= 0 or kv_cache_bytes <= 0 or page_size <= 0:
            raise ValueError("sequences, cache bytes and page size must be positive")
        if not 0 < prefill_chunk_size <= prefill_burst_size:
            raise ValueError("prefill chunk sizes must be positive, the burst no smaller")
        if not torch.cuda.is_available():
            raise RuntimeError("the engine needs a CUDA device (sm_100a); there is no CPU path")
        if model is None:
            if model_path is None:
                raise ValueError("give the engine a model folder (config.json plus safetensors)")
            model = load_model(model_path, dtype, device)
        elif model.device is None:
            raise ValueError("the model's weights are not loaded")
        self.model = model
        self.device = model.device
        self.dtype = parse_dtype(model.dtype)
        config = model.config
        self.vocab_size = int(config.vocab_size)
        self.eos_token_ids = tuple(getattr(config, "eos_token_ids", ()))
        self.max_num_sequences = max_num_sequences
        self.max_model_length = min(
            config.max_position_embeddings, max_model_length or config.max_position_embeddings
        )
        self.prefill_chunk_size = prefill_chunk_size
        self.prefill_burst_size = prefill_burst_size
        self.max_batch_tokens = max_batch_tokens or (prefill_burst_size + max_num_sequences)
        self.page_size = page_size
        self.cache = PagedCache(
            model.cache_specs(),
            dtype=self.dtype,
            device=self.device,
            page_size=page_size,
            max_num_sequences=max_num_sequences,
            max_model_length=self.max_model_length,
            step_tokens=prefill_burst_size,
            kv_cache_bytes=None if num_pages is not None else kv_cache_bytes,
            num_pages=num_pages,
        )
        self.runner = ModelRunner(
            model,
            self.cache,
            max_batch_tokens=self.max_batch_tokens,
            # "plain": the plain attention kernel and the library's matrix products everywhere (the
            # slow, simple kernels the tuned ones are checked against); "tuned": each step's best.
            options={
                "cuda_graphs": cuda_graphs, "workspace_rows": self.max_batch_tokens, "nvtx": bool(nvtx),
                # "chain": every step is a chain of kernels; "resident": decode steps of up to 16
                # requests as one resident kernel where the model allows it (slower; kept as an option).
                "decode_kernel": "chain" if kernels == "plain" else decode_kernel,
                "step_timing": bool(step_timing),
                # Norms folded into the products around them in short steps (parts/ops.py::fold_enabled):
                # fewer launches, measured no faster; an option.
                "fold_norms": bool(fold_norms) and kernels != "plain",
                **({"attention": "plain", "gemm": "library"} if kernels == "plain" else {}),
            },
        )
        # `nvtx=True` names ranges for a profiler's timeline: "step ..." around each model step,
        # "layer N" and "head" inside it, "sample" around the sampling kernels (the reference's
        # include/instinct/nvtx.h:9-24 and its uses). Off by default; host-side marks only.
        self.nvtx = bool(nvtx)
        self.sampler = Sampler(self.device, max_num_sequences)
        # While a decode step's tokens travel to the host, the next step may already run (see
        # ModelRunner.step_ahead); `run_ahead=False` keeps every step behind the host. A step
        # launched ahead may be dropped, which is harmless for paged keys and values (the same
        # numbers get written again) and not for per-request state that a step advances: a model
        # with such state never runs ahead.
        self.run_ahead = bool(run_ahead) and self.runner.use_graphs and not self.cache.state_specs
        self._ahead = None
        self.steps_ahead_used = 0
        self.steps_ahead_dropped = 0
        self._host = host()
        self.scheduler = self._host.Scheduler(
            self.cache.manager,
            max_num_sequences,
            self.max_model_length,
            self.max_batch_tokens,
            prefill_chunk_size,
            prefill_burst_size,
            self.vocab_size,
            seed,
        )
        self._closed = False

    # -- requests --------------------------------------------------------------------------------

    def submit(
        self,
        input_ids: Iterable[int],
        max_new_tokens: int,
        eos_token_ids: Iterable[int] = (),
        *,
        sampling: SamplingParams | None = None,
    ) -> int:
        """Queue a prompt; returns the request id. Raises ``ValueError`` for an empty prompt,
        ids outside the vocabulary, a non-positive token budget, a request longer than the
        context, or one the cache could never hold."""
        self._check_open()
        if type(max_new_tokens) is not int or max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be a positive integer")
        prompt = [int(t) for t in input_ids]
        params = sampling or GREEDY
        native = self._host.SamplingParams(
            float(params.temperature), float(params.top_p), int(params.top_k), float(params.min_p), params.seed
        )
        return int(self.scheduler.submit(prompt, max_new_tokens, [int(t) for t in eos_token_ids], native))

    def force(self, request_id: int, tokens: Iterable[int]) -> None:
        """Emit ``tokens`` next instead of sampling."""
        self.scheduler.force(int(request_id), [int(t) for t in tokens])

    def cancel(self, request_id: int) -> None:
        self.scheduler.cancel(int(request_id))

    def forget(self, request_id: int) -> None:
        self.scheduler.forget(int(request_id))

    def request(self, request_id: int) -> RequestView:
        r = self.scheduler.request(int(request_id))
        return RequestView(
            r.request_id, SequenceState(r.state), r.prompt, list(r.output), r.reason, r.length, r.max_new_tokens
        )

    def has_work(self) -> bool:
        return bool(self.scheduler.has_work())

    # -- execution -------------------------------------------------------------------------------

    def step(self) -> list[TokenEvent]:
        """One model step: a token for every running request and portions of admitted
        prompts. Returns the tokens emitted."""
        self._check_open()
        plan = self.scheduler.plan()
        self.cache.clear_new_slots()
        entries = plan.entries
        ahead, self._ahead = self._ahead, None
        if not entries:
            return []
        try:
            tokens = plan.tokens
            if ahead is not None and self._is_this_step(ahead, plan, tokens):
                logits = self.runner.accept_ahead(ahead)
                self.steps_ahead_used += 1
            else:
                if ahead is not None:
                    self.steps_ahead_dropped += 1
                batch = [
                    StepEntry(
                        e.request_id,
                        tokens[e.token_offset : e.token_offset + e.count],
                        (e.count - 1,) if e.wants_token else (),
                    )
                    for e in entries
                ]
                logits = self.runner.step(batch)
            wanting = [e for e in entries if e.wants_token]
            if wanting:
                requests = [self.scheduler.request(e.request_id) for e in wanting]
                if self.nvtx:
                    torch.cuda.nvtx.range_push("sample")
                try:
                    rows = self.sampler.launch(
                        logits,
                        [r.sampling for r in requests],
                        [self.scheduler.draw_key(r.request_id) for r in requests],
                        self.runner.err,
                    )
                finally:
                    if self.nvtx:
                        torch.cuda.nvtx.range_pop()
                if self.run_ahead and self.scheduler.repeats(plan):
                    # The next step will feed these tokens to the same requests unless one of
                    # them ends a request: launch it now, behind the sampling kernels.
                    self._ahead = self.runner.step_ahead([e.request_id for e in entries], self.sampler.tokens_device)
                chosen, err = self.sampler.result(rows)
                if err:
                    check_error_word(self.runner.err, "step")
            else:
                chosen = []
            events = self.scheduler.commit(plan, chosen)
            if self._ahead is not None:
                emitted = {e.request_id: e.token for e in events}
                self._ahead.tokens = [emitted.get(r) for r in self._ahead.request_ids]
        except Exception:
            self._ahead = None
            self.scheduler.abandon(plan)
            raise
        return [TokenEvent(e.request_id, e.token, e.finished, e.reason) for e in events]

    def _is_this_step(self, ahead, plan, tokens) -> bool:
        """Whether the step launched ahead fed exactly what ``plan`` asks for now."""
        entries = plan.entries
        if ahead.issue != self.runner.issue or ahead.tokens is None or len(entries) != len(ahead.request_ids):
            return False
        for e, request_id, start, token in zip(entries, ahead.request_ids, ahead.starts, ahead.tokens):
            if e.request_id != request_id or e.count != 1 or not e.wants_token or e.start != start:
                return False
            if int(tokens[e.token_offset]) != token:
                return False
        return True

    def generate(
        self,
        input_ids: Iterable[int],
        max_new_tokens: int,
        eos_token_ids: Iterable[int] = (),
        **options: Any,
    ) -> list[int]:
        request_id = self.submit(input_ids, max_new_tokens, eos_token_ids, **options)
        try:
            while self.request(request_id).state not in TERMINAL:
                self.step()
        except Exception:
            self.cancel(request_id)
            self.forget(request_id)
            raise
        request = self.request(request_id)
        self.forget(request_id)
        if request.state is not SequenceState.COMPLETED:
            raise RuntimeError("generation ended without completing")
        return list(request.output)

    def prefill_logits(self, input_ids: Iterable[int]) -> np.ndarray:
        """Last-position logits of a prompt, outside the scheduler (for checks); every page is
        given back afterwards (python/instinct/mlx_engine.py:544-571)."""
        self._check_open()
        prompt = [int(t) for t in input_ids]
        if not 0 < len(prompt) < self.max_model_length:
            raise ValueError("the prompt length is outside the context limit")
        if any(not 0 <= t < self.vocab_size for t in prompt):
            raise ValueError("token id is outside the vocabulary")
        request_id = -1
        if not self.cache.admit(request_id, len(prompt) + 1):
            raise RuntimeError("no K/V room for the prompt")
        try:
            logits = None
            for start in range(0, len(prompt), self.prefill_chunk_size):
                chunk = prompt[start : start + self.prefill_chunk_size]
                last = start + len(chunk) == len(prompt)
                logits = self.runner.step([StepEntry(request_id, chunk, (len(chunk) - 1,) if last else ())])
            out = logits[0].to("cpu", torch.float32).numpy().copy()
            self.runner.check()
            return out
        finally:
            self.cache.manager.release(request_id)

    # -- housekeeping ----------------------------------------------------------------------------

    def stats(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "backend": self.backend,
            "model_type": getattr(self.model.config, "MODEL_TYPE", self.model.config.architecture),
            "dtype": str(self.dtype).removeprefix("torch."),
            "max_num_sequences": self.max_num_sequences,
            "max_model_length": self.max_model_length,
            "page_size": self.page_size,
            "model_steps": self.runner.steps,
            "steps_ahead_used": self.steps_ahead_used,
            "steps_ahead_dropped": self.steps_ahead_dropped,
            "weight_bytes": self.model.weight_bytes(),
        }
        out.update(self.scheduler.stats())
        out.update(self.cache.stats())
        if self.runner.step_timing:
            # Where a step's time goes: the host inside the step function against the device's time
            # for the same steps (steps launched ahead of the host are not among them).
            timing = self.runner.timing()
            out["step_timing"] = timing
        return out

    def build_info(self) -> dict[str, object]:
        return build_info()

    def _check_open(self) -> None:
        if self._closed:
            raise RuntimeError("engine is closed")

    def close(self) -> None:
        if self._closed:
            return
        # Cancel whatever is still active; ids are dense from 1.
        stats = self.scheduler.stats()
        for request_id in range(1, int(stats["submitted"]) + int(stats["rejected"]) + 1):
            self.scheduler.cancel(request_id)
        self._ahead = None
        torch.cuda.synchronize(self.device)  # a step launched ahead may still be running
        self._closed = True

    def __enter__(self) -> "Engine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()


def create_engine(model_path: str | Path | None = None, *, backend: str = "auto", **kwargs: Any) -> Engine:
    """Build an engine for a model folder. ``backend`` is kept for callers of the reference's
    ``create_engine`` (python/instinct/__init__.py:27-50); this engine has one backend,
    CUDA on sm_100a, chosen by ``"auto"``, ``"cuda"`` or ``"b200"``."""
    selected = backend.lower()
    if selected not in {"auto", "cuda", "b200"}:
        raise ValueError(f"unknown backend {backend!r}; expected 'auto', 'cuda' or 'b200'")
    if model_path is None and "model" not in kwargs:
        raise ValueError("the engine needs a model folder (config.json plus safetensors)")
    return Engine(model_path, **kwargs)


__all__ = [
    "Engine",
    "KernelError",
    "RequestView",
    "SamplingParams",
    "SequenceState",
    "TERMINAL",
    "TokenEvent",
    "build_info",
    "create_engine",
]
